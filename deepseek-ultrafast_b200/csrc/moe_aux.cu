// Routing, permute plan and unpermute/combine of the routed-expert layer.
//
//   route_kernel        <- moe_route_tokens / route_token   (crates/kernels/cu/ops.cu:615-623, cu/route.cuh:3-56)
//   plan_*_kernel       <- moe_perm                         (cu/tcmoe.cu:19-69; decode slots: cu/gemv.cu:715-776)
//   unpermute_kernel    <- the nsum/src2 sum in comm_push   (cu/comm.cu:167-180)
//
// The reference builds its prefill plan in ONE 1024-thread CTA with shared-memory atomics (order inside an
// expert depends on timing) and rebuilds the decode plan inside every GEMV CTA.  Here the plan is built once,
// by a stable counting sort (one fused launch for decode-sized plans, three phases that scale over CTAs above
// that), and every consumer (decode or prefill) reads it.
#include "internal.h"
#include "quant_core.cuh"

namespace dsuf {

// ---------------------------------------------------------------- router
constexpr int ROUTE_MAX_PER_LANE = 16;  // n_exp <= 512

// One token by one warp: top-k of score + bias (ties to the lower id), weights = score / sum of the picked scores * scale.
// ids_out / w_out point at the token's topk entries (global or shared memory).
DSUF_DEV void route_one_token(int score_fn, const float* s, const float* bias, int n_exp, int topk, float route_scale, int lane,
                              int* ids_out, float* w_out) {
    float sc[ROUTE_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        sc[i] = e < n_exp ? s[e] : -INFINITY;
        mx = fmaxf(mx, sc[i]);
    }
    if (score_fn == DSUF_SCORE_SOFTMAX) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
            sc[i] = lane + 32 * i < n_exp ? expf(sc[i] - mx) : 0.f;
            sum += sc[i];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) sc[i] = __fdiv_rn(sc[i], sum);
    } else if (score_fn == DSUF_SCORE_SQRT_SOFTPLUS) {
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
            if (lane + 32 * i < n_exp) sc[i] = sqrtf(sc[i] > 20.f ? sc[i] : log1pf(expf(sc[i])));
    }
    // Selection works on one 64-bit word per candidate: the biased score mapped to an unsigned integer that orders like
    // the float (high half) and the complement of the expert id (low half).  The largest word is the best score and,
    // among equal scores, the lowest id -- the reference's tie rule (cu/route.cuh:3-56) -- and it names its own expert,
    // so one butterfly maximum per pick is the whole selection.  A picked candidate is retired by zeroing its word.
    unsigned long long cand[ROUTE_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        cand[i] = 0ull;
        if (e < n_exp) {
            const float biased = sc[i] + (bias ? bias[e] : 0.f) + 0.0f;  // + 0.0f: -0 and +0 compare equal, as floats do
            const unsigned bits = __float_as_uint(biased);
            const unsigned ordered = (bits >> 31) ? ~bits : (bits | 0x80000000u);
            cand[i] = ((unsigned long long)ordered << 32) | (unsigned)(0xffffffffu - (unsigned)e);
        }
    }
    float wsum = 0.f, myw = 0.f;
    int myid = 0;
    for (int j = 0; j < topk; ++j) {
        unsigned long long best = cand[0];
#pragma unroll
        for (int i = 1; i < ROUTE_MAX_PER_LANE; ++i) best = cand[i] > best ? cand[i] : best;
        // warp maximum of the 64-bit words in two 32-bit hardware reductions: the best score first, then the best
        // (complemented) id among the lanes that hold that score
        const unsigned hi = (unsigned)(best >> 32);
        const unsigned top_hi = __reduce_max_sync(0xffffffffu, hi);
        const unsigned top_lo = __reduce_max_sync(0xffffffffu, hi == top_hi ? (unsigned)best : 0u);
        best = ((unsigned long long)top_hi << 32) | top_lo;
        const int picked = (int)(0xffffffffu - (unsigned)(best & 0xffffffffull));  // every lane holds the same word
        // exactly one lane holds the winning word: it retires the candidate, and an OR over the warp hands everybody the bits
        // of its unbiased score (all other lanes contribute zero)
        unsigned wbits = 0u;
#pragma unroll
        for (int i = 0; i < ROUTE_MAX_PER_LANE; ++i)
            if (cand[i] == best) { wbits = __float_as_uint(sc[i]); cand[i] = 0ull; }
        const float wv = __uint_as_float(__reduce_or_sync(0xffffffffu, wbits));
        wsum += wv;
        if (lane == j) { myw = wv; myid = picked; }
    }
    if (lane < topk) {
        const float v = topk > 1 ? __fdiv_rn(myw, wsum + 1e-20f) : myw;
        ids_out[lane] = myid;
        w_out[lane] = v * route_scale;
    }
}

__global__ void __launch_bounds__(256) route_kernel(int score_fn, const float* scores, const float* bias, int t, int n_exp,
                                                    int topk, float route_scale, int* ids, float* w) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int tok = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (tok >= t) return;
    route_one_token(score_fn, scores + (size_t)tok * n_exp, bias, n_exp, topk, route_scale, lane, ids + (size_t)tok * topk,
                    w + (size_t)tok * topk);
}

int launch_route(dsuf_ctx* ctx, cudaStream_t stream, int score_fn, const float* scores, const float* bias, int t, int n_exp,
                 int topk, float route_scale, int* ids, float* w) {
    if (t == 0) return DSUF_OK;
    return launch(ctx, stream, route_kernel, dim3((t + 7) / 8), dim3(256), 0, score_fn, scores, bias, t, n_exp, topk,
                  route_scale, ids, w);
}

// ---------------------------------------------------------------- permute plan
// scratch layout (ints): block_cnt[nblk][n_exp] | local_rank[p]
constexpr int PLAN_BLOCK = 1024;
constexpr int PLAN_MAX_EXP = 512;

struct PlanArgs {
    const int* ids;
    const float* w;
    int e_lo, n_exp, p, tile_rows, max_tiles, nblk;
    int* expert_off;
    int* row_pair;
    int* pair_row;
    float* row_w;
    int4* tiles;
    int* ntiles;
    int* block_cnt;
    int* local_rank;
    DevStatus* status;
};

// Exclusive scan of one value per thread over a block of up to 1024 threads (two values scanned together).
__device__ __forceinline__ void block_exscan2(int a, int b, int& ea, int& eb, int& ta, int& tb, int* s_wa, int* s_wb) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    int ia = a, ib = b;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int ua = __shfl_up_sync(0xffffffffu, ia, o), ub = __shfl_up_sync(0xffffffffu, ib, o);
        if (lane >= o) { ia += ua; ib += ub; }
    }
    if (lane == 31) { s_wa[warp] = ia; s_wb[warp] = ib; }
    __syncthreads();
    if (warp == 0) {
        int wa = lane < nw ? s_wa[lane] : 0, wb = lane < nw ? s_wb[lane] : 0;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int ua = __shfl_up_sync(0xffffffffu, wa, o), ub = __shfl_up_sync(0xffffffffu, wb, o);
            if (lane >= o) { wa += ua; wb += ub; }
        }
        s_wa[lane] = wa;  // inclusive warp totals
        s_wb[lane] = wb;
    }
    __syncthreads();
    const int ba = warp ? s_wa[warp - 1] : 0, bb = warp ? s_wb[warp - 1] : 0;
    ea = ba + ia - a;
    eb = bb + ib - b;
    ta = s_wa[nw - 1];
    tb = s_wb[nw - 1];
    __syncthreads();
}

// Phase A: per-block histogram and each pair's stable rank inside its block.
__global__ void __launch_bounds__(PLAN_BLOCK) plan_count_kernel(const PlanArgs a) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    __shared__ unsigned short warp_hist[32][PLAN_MAX_EXP];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 32 * PLAN_MAX_EXP; i += PLAN_BLOCK) (&warp_hist[0][0])[i] = 0;
    __syncthreads();
    const int i = blockIdx.x * PLAN_BLOCK + tid;
    int e = -1;
    if (i < a.p) {
        e = a.ids[i] - a.e_lo;
        if (e < 0 || e >= a.n_exp) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_hist[warp][e] = (unsigned short)__popc(peers);
    __syncthreads();
    for (int x = tid; x < a.n_exp; x += PLAN_BLOCK) {
        int run = 0;
        for (int wv = 0; wv < 32; ++wv) {
            const int c = warp_hist[wv][x];
            warp_hist[wv][x] = (unsigned short)run;
            run += c;
        }
        a.block_cnt[(size_t)blockIdx.x * a.n_exp + x] = run;
    }
    __syncthreads();
    if (i < a.p) a.local_rank[i] = e >= 0 ? warp_hist[warp][e] + rank_in_warp : -1;
}

// Phase B (one CTA): scan blocks per expert, scan experts, emit the tile list.
__global__ void __launch_bounds__(PLAN_MAX_EXP) plan_scan_kernel(const PlanArgs a) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    __shared__ int s_cnt[32], s_off[32];
    const int e = threadIdx.x;
    int total = 0;
    if (e < a.n_exp) {
        for (int b = 0; b < a.nblk; ++b) {
            const int c = a.block_cnt[(size_t)b * a.n_exp + e];
            a.block_cnt[(size_t)b * a.n_exp + e] = total;
            total += c;
        }
    }
    const int cnt = e < a.n_exp ? total : 0;
    const int ntile = (cnt + a.tile_rows - 1) / a.tile_rows;
    int off, toff, rows, tiles_total;
    block_exscan2(cnt, ntile, off, toff, rows, tiles_total, s_cnt, s_off);
    if (e == 0) {
        a.expert_off[a.n_exp] = rows;
        a.ntiles[0] = tiles_total <= a.max_tiles ? tiles_total : a.max_tiles;
        a.ntiles[1] = rows;
        if (tiles_total > a.max_tiles) report(a.status, DEVERR_BAD_PLAN, 2, tiles_total);
    }
    if (e < a.n_exp) {
        a.expert_off[e] = off;
        int ti = toff;
        for (int r0 = 0; r0 < cnt; r0 += a.tile_rows, ++ti)
            if (ti < a.max_tiles) a.tiles[ti] = make_int4(e, off + r0, min(a.tile_rows, cnt - r0), 0);
    }
}

// Phase C: place every pair.
__global__ void __launch_bounds__(PLAN_BLOCK) plan_place_kernel(const PlanArgs a) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int i = blockIdx.x * PLAN_BLOCK + threadIdx.x;
    if (i >= a.p) return;
    const int lr = a.local_rank[i];
    if (lr < 0) { a.pair_row[i] = -1; return; }
    const int e = a.ids[i] - a.e_lo;
    const int row = a.expert_off[e] + a.block_cnt[(size_t)blockIdx.x * a.n_exp + e] + lr;
    a.row_pair[row] = i;
    a.pair_row[i] = row;
    a.row_w[row] = a.w[i];
}


// Decode-sized plans (all pairs fit one block of PLAN_BLOCK threads): histogram, scans, tile list and placement in one
// pass.  Same result as the three-phase path, bit for bit (the order inside an expert is the pair order either way).
// `write` = this CTA stores the plan to global memory; `s_pair_row` (optional, shared) receives pair_row as well.
struct PlanSmem {
    alignas(16) unsigned short warp_hist[32][PLAN_MAX_EXP];
    int off[PLAN_MAX_EXP + 1], wa[32], wb[32];
};
DSUF_DEV void plan_small_body(const PlanArgs& a, PlanSmem& sm, bool write, int* s_pair_row) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 32 * PLAN_MAX_EXP / 8; i += PLAN_BLOCK) ((uint4*)&sm.warp_hist[0][0])[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    int e = -1;
    if (tid < a.p) {
        e = a.ids[tid] - a.e_lo;
        if (e < 0 || e >= a.n_exp) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) sm.warp_hist[warp][e] = (unsigned short)__popc(peers);
    __syncthreads();
    int cnt = 0;
    if (tid < a.n_exp) {
        for (int wv = 0; wv < 32; ++wv) {
            const int c = sm.warp_hist[wv][tid];
            sm.warp_hist[wv][tid] = (unsigned short)cnt;
            cnt += c;
        }
    }
    const int ntile = (cnt + a.tile_rows - 1) / a.tile_rows;
    int off, toff, rows, tiles_total;
    block_exscan2(cnt, ntile, off, toff, rows, tiles_total, sm.wa, sm.wb);
    if (tid < a.n_exp) {
        sm.off[tid] = off;
        if (write) {
            a.expert_off[tid] = off;
            int ti = toff;
            for (int r0 = 0; r0 < cnt; r0 += a.tile_rows, ++ti)
                if (ti < a.max_tiles) a.tiles[ti] = make_int4(tid, off + r0, min(a.tile_rows, cnt - r0), 0);
        }
    }
    if (tid == 0 && write) {
        a.expert_off[a.n_exp] = rows;
        a.ntiles[0] = tiles_total <= a.max_tiles ? tiles_total : a.max_tiles;
        a.ntiles[1] = rows;
        if (tiles_total > a.max_tiles) report(a.status, DEVERR_BAD_PLAN, 2, tiles_total);
    }
    __syncthreads();
    if (tid < a.p) {
        const int row = e < 0 ? -1 : sm.off[e] + sm.warp_hist[warp][e] + rank_in_warp;
        if (s_pair_row) s_pair_row[tid] = row;
        if (write) {
            a.pair_row[tid] = row;
            if (row >= 0) {
                a.row_pair[row] = tid;
                a.row_w[row] = a.w[tid];
            }
        }
    }
}

__global__ void __launch_bounds__(PLAN_BLOCK) plan_small_kernel(const PlanArgs a) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    __shared__ PlanSmem sm;
    plan_small_body(a, sm, true, nullptr);
}

// Decode front end in ONE launch: router, permute plan and gather + quant for batches of at most 1024 (token, expert)
// pairs -- the counterpart of the routing the reference runs inside its decode MoE launch (route_plan,
// cu/gemv.cu:715-776).  The CTAs of a cluster of 8 route the tokens between them (one token per warp) and read one
// another's picks through distributed shared memory; every CTA then builds the whole plan in its own shared memory
// (512 pairs at the decode size: no second and third launch); CTA 0 stores ids, weights and the plan; CTA b quantizes
// token rows b, b + gridDim.x, ... and writes each to its top-k permuted rows.
struct FrontArgs {
    PlanArgs plan;          // ids / w point at the routing outputs in global memory (written by CTA 0)
    const float* scores;    // [t][n_exp_all]
    const float* bias;      // [n_exp_all] or null
    int score_fn, t, n_exp_all, topk;
    float route_scale;
    int* ids_out;           // [t][topk]
    float* w_out;
    const bf16* x;          // [t][ldx]
    int ldx, h;
    uint8_t* xq;            // [p][h]
    void* xs;               // MX u8 [p][h/32], DS f32 [p][h/128]
};

template <int MODE>
__global__ void __launch_bounds__(PLAN_BLOCK) moe_front_kernel(const FrontArgs f) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    __shared__ PlanSmem sm;
    __shared__ int s_ids[PLAN_BLOCK], s_pair_row[PLAN_BLOCK];
    __shared__ float s_w[PLAN_BLOCK];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool first = blockIdx.x == 0;
    // the CTAs of a cluster share the routing: CTA r routes tokens r, r + cs, ... (one per warp) and the others read its
    // picks through distributed shared memory; every CTA then holds all picks and builds the (same) plan by itself
    const int cs = (int)cluster_num_ctas(), crank = (int)cluster_cta_rank();
    for (int tok = crank + cs * warp; tok < f.t; tok += cs * (PLAN_BLOCK / 32))
        route_one_token(f.score_fn, f.scores + (size_t)tok * f.n_exp_all, f.bias, f.n_exp_all, f.topk, f.route_scale, lane,
                        s_ids + tok * f.topk, s_w + tok * f.topk);
    if (cs > 1) {
        cluster_barrier();
        if (tid < f.plan.p) {
            const int owner = (tid / f.topk) % cs;
            if (owner != crank) {
                s_ids[tid] = (int)ld_cluster_u32(s_ids + tid, owner);
                s_w[tid] = ld_cluster_f32(s_w + tid, owner);
            }
        }
        cluster_barrier();   // no CTA goes on (and none exits) while a peer still reads its picks
    } else {
        __syncthreads();
    }
    if (first && tid < f.plan.p) {
        f.ids_out[tid] = s_ids[tid];
        f.w_out[tid] = s_w[tid];
    }
    PlanArgs pa = f.plan;
    pa.ids = s_ids;
    pa.w = s_w;
    plan_small_body(pa, sm, first, s_pair_row);
    __syncthreads();
    constexpr int LANES = MODE == DSUF_MODE_MX ? 4 : 16;
    for (int tok = blockIdx.x; tok < f.t; tok += gridDim.x) {
        for (int base = 0; base < f.h; base += PLAN_BLOCK * 8) {   // every thread makes every pass (the quantizer shuffles)
            const int k0 = base + tid * 8;
            const bool live = k0 < f.h;   // h % 128 == 0: a scale block is live or dead as a whole
            float v[8];
            if (live) {
                const uint4 raw = *(const uint4*)(f.x + (size_t)tok * f.ldx + k0);
                const bf16* hh = (const bf16*)&raw;
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(hh[e]);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = 0.f;
            }
            uint2 codes;
            float sc;
            quant8<MODE>(v, codes, sc);
            if (!live) continue;
            for (int j = 0; j < f.topk; ++j) {
                const int dst = s_pair_row[tok * f.topk + j];
                if (dst < 0) continue;
                *(uint2*)(f.xq + (size_t)dst * f.h + k0) = codes;
                if ((tid & (LANES - 1)) == 0) {
                    if (MODE == DSUF_MODE_MX) ((uint8_t*)f.xs)[(size_t)dst * (f.h >> 5) + (k0 >> 5)] = (uint8_t)(__float_as_uint(sc) >> 23);
                    else ((float*)f.xs)[(size_t)dst * (f.h >> 7) + (k0 >> 7)] = sc;
                }
            }
        }
    }
}

int launch_plan(dsuf_ctx* ctx, cudaStream_t stream, const int* ids, const float* w, int e_lo, const dsuf_moe_plan* plan) {
    PlanArgs a;
    a.ids = ids; a.w = w; a.e_lo = e_lo; a.n_exp = plan->n_exp; a.p = plan->p; a.tile_rows = plan->tile_rows;
    a.max_tiles = plan->max_tiles;
    a.nblk = (plan->p + PLAN_BLOCK - 1) / PLAN_BLOCK;
    a.expert_off = (int*)plan->expert_off; a.row_pair = (int*)plan->row_pair; a.pair_row = (int*)plan->pair_row;
    a.row_w = (float*)plan->row_w; a.tiles = (int4*)plan->tiles; a.ntiles = (int*)plan->ntiles;
    a.block_cnt = (int*)plan->scratch;
    a.local_rank = a.block_cnt + (size_t)a.nblk * a.n_exp;
    a.status = ctx->dev_status;
    if (a.nblk <= 1) return launch(ctx, stream, plan_small_kernel, dim3(1), dim3(PLAN_BLOCK), 0, a);
    int rc = launch(ctx, stream, plan_count_kernel, dim3(a.nblk > 0 ? a.nblk : 1), dim3(PLAN_BLOCK), 0, a);
    if (rc) return rc;
    rc = launch(ctx, stream, plan_scan_kernel, dim3(1), dim3(PLAN_MAX_EXP), 0, a);
    if (rc) return rc;
    if (a.nblk == 0) return DSUF_OK;
    return launch(ctx, stream, plan_place_kernel, dim3(a.nblk), dim3(PLAN_BLOCK), 0, a);
}

int launch_front(dsuf_ctx* ctx, cudaStream_t stream, int score_fn, const float* scores, const float* bias, int t, int n_exp_all,
                 int topk, float route_scale, int* ids, float* w, int e_lo, const dsuf_moe_plan* plan, int mode, const void* x, int ldx,
                 int h, void* xq, void* xs) {
    FrontArgs f;
    PlanArgs& a = f.plan;
    a.ids = ids; a.w = w; a.e_lo = e_lo; a.n_exp = plan->n_exp; a.p = plan->p; a.tile_rows = plan->tile_rows;
    a.max_tiles = plan->max_tiles; a.nblk = 1;
    a.expert_off = (int*)plan->expert_off; a.row_pair = (int*)plan->row_pair; a.pair_row = (int*)plan->pair_row;
    a.row_w = (float*)plan->row_w; a.tiles = (int4*)plan->tiles; a.ntiles = (int*)plan->ntiles;
    a.block_cnt = nullptr; a.local_rank = nullptr;
    a.status = ctx->dev_status;
    f.scores = scores; f.bias = bias; f.score_fn = score_fn; f.t = t; f.n_exp_all = n_exp_all; f.topk = topk; f.route_scale = route_scale;
    f.ids_out = ids; f.w_out = w; f.x = (const bf16*)x; f.ldx = ldx; f.h = h; f.xq = (uint8_t*)xq; f.xs = xs;
    const int cs = t >= 8 ? 8 : 1;
    int grid = t < ctx->sm_count ? t : ctx->sm_count;
    grid = grid / cs * cs;   // whole clusters; the quantizer strides over the tokens by the grid size
    if (mode == DSUF_MODE_MX) return launch_cluster(ctx, stream, moe_front_kernel<DSUF_MODE_MX>, dim3(grid), dim3(PLAN_BLOCK), 0, cs, f);
    return launch_cluster(ctx, stream, moe_front_kernel<DSUF_MODE_DS>, dim3(grid), dim3(PLAN_BLOCK), 0, cs, f);
}

// ---------------------------------------------------------------- unpermute / combine
__global__ void __launch_bounds__(256) unpermute_kernel(const int* pair_row, const float* yrows, const bf16* shared, int topk,
                                                        int h, bf16* out, int ldo) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int tok = blockIdx.x;
    __shared__ int rows[16];
    if (threadIdx.x < topk) rows[threadIdx.x] = pair_row[(size_t)tok * topk + threadIdx.x];
    __syncthreads();
    for (int c = (blockIdx.y * 256 + threadIdx.x) * 4; c < h; c += gridDim.y * 1024) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j < topk; ++j) {
            const int r = rows[j];
            if (r < 0) continue;
            const float4 v = __ldcs((const float4*)(yrows + (size_t)r * h + c));
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        if (shared) {
            const uint2 raw = *(const uint2*)(shared + (size_t)tok * h + c);
            const bf16* sh = (const bf16*)&raw;
            s.x += __bfloat162float(sh[0]); s.y += __bfloat162float(sh[1]);
            s.z += __bfloat162float(sh[2]); s.w += __bfloat162float(sh[3]);
        }
        uint2 o;
        bf16* ob = (bf16*)&o;
        ob[0] = __float2bfloat16(s.x); ob[1] = __float2bfloat16(s.y);
        ob[2] = __float2bfloat16(s.z); ob[3] = __float2bfloat16(s.w);
        *(uint2*)(out + (size_t)tok * ldo + c) = o;
    }
}

// The same sum, eight columns per thread, with the result also quantized for the next projection (the quantizer's step:
// quant_core.cuh): one launch instead of unpermute + act_quant between two layers.
template <int MODE>
__global__ void __launch_bounds__(256) unpermute_quant_kernel(const int* pair_row, const float* yrows, const bf16* shared, int topk,
                                                              int h, bf16* out, int ldo, uint8_t* q_out, void* s_out) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int tok = blockIdx.x;
    __shared__ int rows[16];
    if (threadIdx.x < topk) rows[threadIdx.x] = pair_row[(size_t)tok * topk + threadIdx.x];
    __syncthreads();
    const int c = (blockIdx.y * 256 + threadIdx.x) * 8;
    const bool live = c < h;      // h % 128 == 0: a scale block is live or dead as a whole
    float s[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) s[e] = 0.f;
    if (live) {
        for (int j = 0; j < topk; ++j) {
            const int r = rows[j];
            if (r < 0) continue;
            const float4 v0 = __ldcs((const float4*)(yrows + (size_t)r * h + c));
            const float4 v1 = __ldcs((const float4*)(yrows + (size_t)r * h + c + 4));
            s[0] += v0.x; s[1] += v0.y; s[2] += v0.z; s[3] += v0.w;
            s[4] += v1.x; s[5] += v1.y; s[6] += v1.z; s[7] += v1.w;
        }
        if (shared) {
            const uint4 raw = *(const uint4*)(shared + (size_t)tok * h + c);
            const bf16* sh = (const bf16*)&raw;
#pragma unroll
            for (int e = 0; e < 8; ++e) s[e] += __bfloat162float(sh[e]);
        }
    }
    uint4 o;
    bf16* ob = (bf16*)&o;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        ob[e] = __float2bfloat16(s[e]);
        v[e] = __bfloat162float(ob[e]);      // the quantizer sees the bf16 row the next layer would read
    }
    uint2 codes;
    float sc;
    quant8<MODE>(v, codes, sc);   // every lane takes part in the block's amax
    if (!live) return;
    *(uint4*)(out + (size_t)tok * ldo + c) = o;
    *(uint2*)(q_out + (size_t)tok * h + c) = codes;
    if (MODE == DSUF_MODE_MX) {
        if ((threadIdx.x & 3) == 0) ((uint8_t*)s_out)[(size_t)tok * (h >> 5) + (c >> 5)] = (uint8_t)(__float_as_uint(sc) >> 23);
    } else {
        if ((threadIdx.x & 15) == 0) ((float*)s_out)[(size_t)tok * (h >> 7) + (c >> 7)] = sc;
    }
}

int launch_unpermute_quant(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_moe_plan* plan, const float* yrows, const void* shared,
                           int t, int topk, int h, void* out, int ldo, int mode, void* q_out, void* s_out) {
    if (t == 0) return DSUF_OK;
    const dim3 grid(t, (h + 2047) / 2048);
    if (mode == DSUF_MODE_MX)
        return launch(ctx, stream, unpermute_quant_kernel<DSUF_MODE_MX>, grid, dim3(256), 0, (const int*)plan->pair_row, yrows,
                      (const bf16*)shared, topk, h, (bf16*)out, ldo, (uint8_t*)q_out, s_out);
    return launch(ctx, stream, unpermute_quant_kernel<DSUF_MODE_DS>, grid, dim3(256), 0, (const int*)plan->pair_row, yrows,
                  (const bf16*)shared, topk, h, (bf16*)out, ldo, (uint8_t*)q_out, s_out);
}

int launch_unpermute(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_moe_plan* plan, const float* yrows, const void* shared,
                     int t, int topk, int h, void* out, int ldo) {
    if (t == 0) return DSUF_OK;
    const int gy = t >= 1024 ? 1 : (h + 1023) / 1024;
    return launch(ctx, stream, unpermute_kernel, dim3(t, gy), dim3(256), 0, (const int*)plan->pair_row, yrows,
                  (const bf16*)shared, topk, h, (bf16*)out, ldo);
}

}  // namespace dsuf
