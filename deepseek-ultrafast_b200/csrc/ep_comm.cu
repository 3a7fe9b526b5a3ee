// Exchanges of bf16 activation rows over NVLink peer memory for the expert-parallel stack: a one-shot all-reduce, the
// combine (this rank's sum of every token's expert rows, then the all-reduce, optionally leaving the result quantized for
// the next projection) and an all-gather of column slices (an output-sharded projection's dispatch).
//
// Replaces comm_push / comm_push2_body / nv_contrib (crates/kernels/cu/comm.cu:134-279, 355-375, 559-584): the
// reference pushes partial rows into every peer and sums what arrived.  Here every rank leaves its partial where the
// producing kernel wrote it (a buffer all ranks mapped at set-up), announces it to its peers with a release store of
// the call's epoch, waits for the peers' announcements, then READS the peers' partials with plain peer loads and
// adds them up in rank order in fp32 (so every rank rounds the same sum to the same bf16).  At 0.9 MB per rank
// (64 tokens x 7168) that is 7 peer reads of 0.9 MB per rank: latency-, not bandwidth-bound, which is why it is one
// kernel with one hand-shake instead of a ring or a tree.
//
// Every wait is bounded (dsuf_ctx_set_wait_budget_us, default common.cuh WAIT_BUDGET_TICKS): a rank that never announces
// makes the others record DEVERR_WAIT_TIMEOUT in the context's status word and finish with an incomplete sum instead of
// hanging; a peer more than one call ahead is reported as DEVERR_EPOCH_DRIFT.
// The only peer accesses are plain ld / st on peer pointers.
#include "internal.h"
#include "quant_core.cuh"

namespace dsuf {

constexpr int KID_EPCOMM = 5;
constexpr int EPC_MAX_WORLD = 8;
constexpr int EPC_CTAS = 128;     // flag slots per rank: [EPC_CTAS][world]; enough threads that a 0.9 MB sum is 1-2 loads per rank and thread
constexpr int EPC_THREADS = 256;

struct EpcArgs {
    const uint4* data[EPC_MAX_WORLD];  // every rank's partial buffer (index = rank), n_elems bf16 each
    uint32_t* flags[EPC_MAX_WORLD];    // every rank's flag block: [EPC_CTAS][world] epochs
    bf16* out;                         // local result
    DevStatus* status;
    long long n_vec;                   // n_elems / 8
    int rank, world;
    int gather_vec, row_vec;           // all-gather of column slices: 16-byte vectors per slice / per row (0: all-reduce)
    long long wait_ticks;              // clock64 budget of the wait for the peers' announcements
    uint8_t* q_out;                    // optional: FP8 codes of `out` (the next GEMM's activation operand), [n_elems]
    void* q_scales;                    //           their block scales, row-major (MX u8 per 32, DS f32 per 128 elements)
    int q_mode;                        //           DSUF_MODE_MX / DSUF_MODE_DS
    uint32_t* state;                   // local: [0] calls completed (the epoch lives on the device so that a captured
                                       // graph advances it on every replay), [1] CTAs finished in this call
};

DSUF_DEV void st_release_sys(uint32_t* p, uint32_t v) { asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
DSUF_DEV uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// system-scope relaxed load: never served from this SM's L1, which is not coherent with a peer's writes
DSUF_DEV uint4 ld_relaxed_sys_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}

// Waits until the peer's flag has reached this call's epoch, for at most a.wait_ticks.  A peer runs at most one call
// ahead of this rank (it needs this rank's announcement of call n + 1 to finish that call), so a flag further ahead
// means the two ranks no longer count the same calls (a launch that failed or timed out on one side): reported as
// DEVERR_EPOCH_DRIFT instead of summing partials of different calls in silence.
DSUF_DEV void exchange_wait(const EpcArgs& a, const uint32_t* f, uint32_t epoch, long long t0, int site) {
    for (;;) {
        const int32_t ahead = (int32_t)(ld_acquire_sys(f) - epoch);
        if (ahead >= 0) {
            if (ahead > 1) report(a.status, DEVERR_EPOCH_DRIFT, KID_EPCOMM, site);
            return;
        }
        if (clock64() - t0 > a.wait_ticks) {
            report(a.status, DEVERR_WAIT_TIMEOUT, KID_EPCOMM, site);
            return;
        }
    }
}

// out[i] = sum over the ranks, in rank order, of vector i of every rank's partial (fp32 adds, one rounding to bf16: all
// ranks round the same sum).  Peer latency, not bandwidth, bounds this step, so a thread's loads of two rounds
// (2 x world 16-byte vectors) are all issued before the first add.  With q_out set the rounded sums are also quantized
// to FP8 exactly as dsuf_act_quant_fp8 would quantize `out` (a scale block is 4 or 16 neighbouring threads of a warp).
DSUF_DEV void sum_vec(const EpcArgs& a, const uint4 (&v)[EPC_MAX_WORLD], long long i, bool live, int lane) {
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = 0.f;
#pragma unroll
    for (int r = 0; r < EPC_MAX_WORLD; ++r)
        if (r < a.world) {
            const bf16* h = (const bf16*)&v[r];
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] += __bfloat162float(h[e]);
        }
    uint4 o;
    bf16* ho = (bf16*)&o;
#pragma unroll
    for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16(live ? s[e] : 0.f);
    if (live) *(uint4*)(a.out + i * 8) = o;
    if (a.q_out) {   // (uniform over the grid)
        float q[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = __bfloat162float(ho[e]);
        uint2 codes;
        float sc;
        if (a.q_mode == DSUF_MODE_MX) {
            quant8<DSUF_MODE_MX>(q, codes, sc);
            if (live && (lane & 3) == 0) ((uint8_t*)a.q_scales)[i >> 2] = (uint8_t)(__float_as_uint(sc) >> 23);
        } else {
            quant8<DSUF_MODE_DS>(q, codes, sc);
            if (live && (lane & 15) == 0) ((float*)a.q_scales)[i >> 4] = sc;
        }
        if (live) *(uint2*)(a.q_out + i * 8) = codes;
    }
}

DSUF_DEV void sum_over_ranks(const EpcArgs& a, int b, int tid) {
    const int lane = tid & 31;
    const long long stride = (long long)gridDim.x * EPC_THREADS;
    // whole warps run every round (the quantizer shuffles): the bound is on the warp's first vector
    for (long long w0 = (long long)b * EPC_THREADS + (tid & ~31); w0 < a.n_vec; w0 += 2 * stride) {
        const long long i0 = w0 + lane, i1 = i0 + stride;
        const bool live0 = i0 < a.n_vec, live1 = i1 < a.n_vec, round1 = w0 + stride < a.n_vec;
        uint4 v0[EPC_MAX_WORLD], v1[EPC_MAX_WORLD];
#pragma unroll
        for (int r = 0; r < EPC_MAX_WORLD; ++r) {
            v0[r] = make_uint4(0, 0, 0, 0);
            v1[r] = make_uint4(0, 0, 0, 0);
            if (r < a.world && live0) v0[r] = ld_relaxed_sys_v4(a.data[r] + i0);
            if (r < a.world && live1) v1[r] = ld_relaxed_sys_v4(a.data[r] + i1);
        }
        sum_vec(a, v0, i0, live0, lane);
        if (round1) sum_vec(a, v1, i1, live1, lane);
    }
}

__global__ void __launch_bounds__(EPC_THREADS) ep_allreduce_kernel(const EpcArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const int tid = threadIdx.x, b = blockIdx.x;
    const uint32_t epoch = *(volatile uint32_t*)a.state + 1;  // every rank makes the same sequence of calls
    // ---- announce: this rank's partial (written by earlier kernels of this stream) is complete ----
    // (the partial was written by kernels that completed before this grid started, so it is already in this GPU's
    // L2 / HBM, which is where peer loads are served from; the release store orders it before the flag)
    if (tid < a.world) st_release_sys(a.flags[tid] + b * a.world + a.rank, epoch);
    // ---- wait for every peer's announcement of this epoch (a peer can be at most one epoch ahead) ----
    if (tid < a.world) {
        const uint32_t* f = a.flags[a.rank] + b * a.world + tid;
        const long long t0 = clock64();
        exchange_wait(a, f, epoch, t0, tid);
    }
    __syncthreads();
    // ---- sum in rank order; all of an element's loads are issued before the first add (peer latency, not bandwidth,
    //      bounds this kernel: sum_over_ranks) ----
    if (a.gather_vec) {
        // all-gather of column slices: every element has one owner (the rank that computed that column range)
        for (long long i = (long long)b * EPC_THREADS + tid; i < a.n_vec; i += (long long)gridDim.x * EPC_THREADS) {
            const int owner = (int)((i % a.row_vec) / a.gather_vec);
            *(uint4*)(a.out + i * 8) = ld_relaxed_sys_v4(a.data[owner] + i);
        }
    } else {
        sum_over_ranks(a, b, tid);
    }
    // ---- the last CTA to finish closes the call: the next call (stream-ordered behind this grid) sees epoch + 1 ----
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {
            a.state[1] = 0;
            __threadfence();
            *(volatile uint32_t*)a.state = epoch;
        }
    }
}

// Combine fused with its exchange: every thread first forms this rank's partial of its own elements
// (out[tok][c] = sum of the token's top-k expert rows that live on this rank, unpermute_kernel's sum), publishes it in the
// mapped partial buffer, and after the hand-shake adds the peers' partials of the SAME elements.  A rank's CTA b
// produces exactly the elements the peers' CTA b consume, so the per-CTA hand-shake is all the ordering needed: no
// grid-wide barrier and no separate unpermute launch.
struct EpCombineArgs {
    EpcArgs c;
    const int* pair_row;   // [t][topk] permuted row of every (token, choice), < 0: not on this rank
    const float* yrows;    // fp32 [rows][h] output of the down projection
    const bf16* shared;    // optional bf16 [t][h] added by THIS rank (pass it on one rank only)
    bf16* partial;         // = c.data[c.rank], writable
    int topk, h;
};

__global__ void __launch_bounds__(EPC_THREADS) ep_combine_kernel(const EpCombineArgs p) {
    pdl_wait();
    pdl_launch_dependents();
    const EpcArgs& a = p.c;
    const int tid = threadIdx.x, b = blockIdx.x;
    const uint32_t epoch = *(volatile uint32_t*)a.state + 1;
    // ---- this rank's partial of this thread's elements ----
    for (long long i = (long long)b * EPC_THREADS + tid; i < a.n_vec; i += (long long)gridDim.x * EPC_THREADS) {
        const long long el = i * 8;
        const int tok = (int)(el / p.h), col = (int)(el - (long long)tok * p.h);
        float s[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) s[e] = 0.f;
        for (int j = 0; j < p.topk; ++j) {
            const int r = __ldg(p.pair_row + (size_t)tok * p.topk + j);
            if (r < 0) continue;
            const float4 v0 = __ldcs((const float4*)(p.yrows + (size_t)r * p.h + col));
            const float4 v1 = __ldcs((const float4*)(p.yrows + (size_t)r * p.h + col + 4));
            s[0] += v0.x; s[1] += v0.y; s[2] += v0.z; s[3] += v0.w;
            s[4] += v1.x; s[5] += v1.y; s[6] += v1.z; s[7] += v1.w;
        }
        if (p.shared) {
            const uint4 raw = *(const uint4*)(p.shared + el);
            const bf16* sh = (const bf16*)&raw;
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] += __bfloat162float(sh[e]);
        }
        uint4 o;
        bf16* ho = (bf16*)&o;
#pragma unroll
        for (int e = 0; e < 8; ++e) ho[e] = __float2bfloat16(s[e]);
        *(uint4*)(p.partial + el) = o;
    }
    __threadfence_system();
    __syncthreads();
    // ---- announce, wait (bounded), sum in rank order: as ep_allreduce_kernel ----
    if (tid < a.world) st_release_sys(a.flags[tid] + b * a.world + a.rank, epoch);
    if (tid < a.world) {
        const uint32_t* f = a.flags[a.rank] + b * a.world + tid;
        const long long t0 = clock64();
        exchange_wait(a, f, epoch, t0, 16 + tid);
    }
    __syncthreads();
    sum_over_ranks(a, b, tid);
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(a.state + 1, 1u) == gridDim.x - 1) {
            a.state[1] = 0;
            __threadfence();
            *(volatile uint32_t*)a.state = epoch;
        }
    }
}

}  // namespace dsuf

using namespace dsuf;

static int fill_epc(dsuf_ctx* ctx, EpcArgs& a, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank, int32_t world,
                    int64_t n_elems, uint64_t state, uint64_t out) {
    DSUF_REQUIRE(ctx, world >= 1 && world <= EPC_MAX_WORLD && rank >= 0 && rank < world, "ep exchange: rank %d of world %d", rank, world);
    DSUF_REQUIRE(ctx, n_elems >= 0 && n_elems % 8 == 0, "ep exchange: n_elems must be a multiple of 8");
    DSUF_REQUIRE(ctx, peer_data && peer_flags && out && (out & 15) == 0, "ep exchange: null or misaligned pointer");
    DSUF_REQUIRE(ctx, state && (state & 3) == 0, "ep exchange: null or misaligned state");
    memset(&a, 0, sizeof(a));
    for (int r = 0; r < world; ++r) {
        DSUF_REQUIRE(ctx, peer_data[r] && peer_flags[r] && (peer_data[r] & 15) == 0, "ep exchange: null or misaligned peer pointer %d", r);
        DSUF_REQUIRE(ctx, peer_data[r] != out, "ep exchange: out must not be a partial buffer (peers still read it)");
        a.data[r] = (const uint4*)peer_data[r];
        a.flags[r] = (uint32_t*)peer_flags[r];
    }
    a.out = (bf16*)out;
    a.status = ctx->dev_status;
    a.wait_ticks = ctx->xchg_wait_ticks;
    a.n_vec = n_elems / 8;
    a.rank = rank;
    a.world = world;
    a.state = (uint32_t*)state;
    return DSUF_OK;
}

extern "C" size_t dsuf_ep_flag_bytes(int32_t world) { return (size_t)EPC_CTAS * (world > 0 ? world : 0) * sizeof(uint32_t); }

extern "C" int32_t dsuf_ep_allreduce_bf16(dsuf_ctx* ctx, void* stream, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                                          int32_t world, int64_t n_elems, uint64_t state, uint64_t out) {
    if (!ctx) return DSUF_E_BADARG;
    EpcArgs a;
    int rc = fill_epc(ctx, a, peer_data, peer_flags, rank, world, n_elems, state, out);
    if (rc) return rc;
    if (n_elems == 0) return DSUF_OK;
    return launch(ctx, (cudaStream_t)stream, ep_allreduce_kernel, dim3(EPC_CTAS), dim3(EPC_THREADS), 0, a);
}

extern "C" int32_t dsuf_ep_allgather_cols_bf16(dsuf_ctx* ctx, void* stream, const uint64_t* peer_data, const uint64_t* peer_flags,
                                               int32_t rank, int32_t world, int32_t rows, int32_t cols, uint64_t state, uint64_t out) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, rows >= 0 && cols > 0 && world >= 1 && cols % (8 * world) == 0, "ep_allgather_cols: cols (%d) must be a multiple of 8 * world", cols);
    EpcArgs a;
    int rc = fill_epc(ctx, a, peer_data, peer_flags, rank, world, (int64_t)rows * cols, state, out);
    if (rc) return rc;
    a.row_vec = cols / 8;
    a.gather_vec = cols / world / 8;
    if (rows == 0) return DSUF_OK;
    return launch(ctx, (cudaStream_t)stream, ep_allreduce_kernel, dim3(EPC_CTAS), dim3(EPC_THREADS), 0, a);
}

extern "C" int32_t dsuf_ep_combine_bf16(dsuf_ctx* ctx, void* stream, uint64_t pair_row, uint64_t yrows, uint64_t shared, int32_t t,
                                        int32_t topk, int32_t h, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                                        int32_t world, uint64_t state, uint64_t out) {
    return dsuf_ep_combine_quant_bf16(ctx, stream, pair_row, yrows, shared, t, topk, h, peer_data, peer_flags, rank, world, state, out,
                                      DSUF_MODE_DS, 0, 0);
}

extern "C" int32_t dsuf_ep_combine_quant_bf16(dsuf_ctx* ctx, void* stream, uint64_t pair_row, uint64_t yrows, uint64_t shared, int32_t t,
                                              int32_t topk, int32_t h, const uint64_t* peer_data, const uint64_t* peer_flags,
                                              int32_t rank, int32_t world, uint64_t state, uint64_t out, int32_t mode, uint64_t xq,
                                              uint64_t xs) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, (xq == 0) == (xs == 0), "ep_combine_quant: xq and xs go together");
    DSUF_REQUIRE(ctx, !xq || ((mode == DSUF_MODE_MX || mode == DSUF_MODE_DS) && h % 128 == 0 && (xq & 7) == 0 && (xs & 3) == 0),
                 "ep_combine_quant: mode MX/DS, h a multiple of 128, xq 8-byte and xs 4-byte aligned");
    DSUF_REQUIRE(ctx, t >= 0 && topk >= 1 && topk <= 16 && h > 0 && h % 8 == 0, "ep_combine: t >= 0, topk in 1..16, h a multiple of 8");
    DSUF_REQUIRE(ctx, pair_row && yrows && (yrows & 15) == 0 && (shared & 15) == 0, "ep_combine: null or misaligned pointer");
    EpCombineArgs p;
    int rc = fill_epc(ctx, p.c, peer_data, peer_flags, rank, world, (int64_t)t * h, state, out);
    if (rc) return rc;
    p.pair_row = (const int*)pair_row;
    p.yrows = (const float*)yrows;
    p.shared = (const bf16*)shared;
    p.partial = (bf16*)peer_data[rank];
    p.topk = topk;
    p.h = h;
    p.c.q_out = (uint8_t*)xq;
    p.c.q_scales = (void*)xs;
    p.c.q_mode = mode;
    if (t == 0) return DSUF_OK;
    return launch(ctx, (cudaStream_t)stream, ep_combine_kernel, dim3(EPC_CTAS), dim3(EPC_THREADS), 0, p);
}
