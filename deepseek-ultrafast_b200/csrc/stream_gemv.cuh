// Decode-shape weight streaming kernel: out[tok][row] = sum_k W[row][k] * x[tok][k] for at most 16 token rows
// per work item, with the weights read exactly once from HBM.
//
// Replaces, for decode shapes, the reference's mma.sync GEMV family
//   gemv_{fp8,fp4}_n{1,2}_p{1,2,4}   crates/kernels/cu/gemv.cu:133-540      (dense, launched by ops.rs:331-474)
//   moe_fp4_swiglu / moe_fp4_store   crates/kernels/cu/gemv.cu:1016-1692    (grouped, launched by ops.rs:482-634)
// with one persistent kernel:
//   * weights live in HBM as contiguous 128-row x 128-K tile records, so a CTA's stream is one linear read;
//   * one producer thread keeps an S-stage ring of {weight tile, activation tile, scale atom} full with TMA,
//     so tens of KB per SM stay in flight for the whole kernel instead of draining at every row tile;
//   * eight consumer warps (16 weight rows each) run m16n8k32 e4m3 MMAs straight on the quantized codes:
//     FP8 weights need no conversion at all, FP4 weights are widened to e4m3 by three logic ops per 4 codes;
//   * block scales are applied to the fp32 partial of each 32-K (MX) or 128-K (DS) block, as the reference does
//     (cu/gemv.cu:354-396);
//   * dense work is cut stream-K style (equal tile spans per CTA); the CTA that completes a row tile last sums
//     the partials in a fixed order, so results do not depend on timing.  Grouped (expert) work is cut at item
//     boundaries and needs no partials.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace dsuf {

enum { FMT_FP8 = 0, FMT_FP4 = 1 };
enum { EPI_DENSE = 0, EPI_W13 = 1, EPI_W2 = 2 };
constexpr int KID_STREAM = 1;
constexpr int STREAM_CONSUMER_WARPS = 8;
constexpr int STREAM_THREADS = (STREAM_CONSUMER_WARPS + 1) * 32;

struct StreamArgs {
    CUtensorMap tm_w;          // weight tile records: {row bytes, 128 rows, tiles}
    CUtensorMap tm_x;          // quantized activation rows: {K bytes, rows}
    const uint8_t* wtiles;     // base of the tile records (scale atoms are bulk-copied from here)
    const float* wscale_ds;    // dense DS geometry: fp32 [RT][KT]
    const void* xscale;        // activation scales: fp32 [rows][KT] (DS) or UE8M0 [rows][4*KT] (MX)
    const int4* slots;         // grouped: (expert, first permuted row, rows<=8*NT8, 0) per slot; null for dense
    const int* nslots;         // grouped: number of slots (device value)
    const float* row_w;        // w13 epilogue: routing weight per permuted row
    void* out;                 // dense: bf16 [m][ldo]; w13: bf16 [rows][ldo]; w2: fp32 [rows][ldo]
    float* partial;            // dense stream-K partials: [grid][2][4*NT8][256]
    int* counters;             // dense: arrivals per row tile, all zero between launches
    DevStatus* status;
    int RT, KT;                // row tiles per matrix, K tiles per row
    int rec_bytes, codes_bytes;
    int n_rows;                // valid weight rows (stores beyond are dropped)
    int m;                     // dense: token rows
    int x_rows;                // rows addressable in xscale
    int ldo;
    float alpha;
    float swiglu_limit;
    int whole_items;  // dense: give every CTA whole row tiles (no stream-K partials) when that costs no extra wave
    int swiglu;       // dense: 1 = the weight holds interleaved gate / up rows and the epilogue is SwiGLU (bf16 [m][n/2] out)
    int out_f32;      // dense: 1 = fp32 output instead of bf16 (GemvOpts.out_f32, crates/engine/src/ops.rs:165-193)
    int accumulate;   // dense: 1 = fp32 out += v instead of out = v (each element is written by one thread of the launch)
    int ssp;          // dense: 1 = store sqrt(softplus(v)) (the router-gate epilogue, crates/kernels/cu/gemv.cu:523); fp32 output
    int n_split;      // dense: > 0 = weight rows >= n_split go to out2 (row stride ldo2) at column row - n_split (GemvOpts.split)
    void* out2;
    int ldo2;
    const float* rope_cos;   // dense, tcgen05 kernels: rotary tables [position][32] (null: no rotation), GemvOpts.rope
    const float* rope_sin;
    const int* rope_pos;     // device int: position of token row 0 (row m sits at rope_pos[0] + m)
    int rope_head, rope_off; // rows r with (r % rope_head) >= rope_off are rotated in (even, odd) pairs
    int kslices;      // dense, tcgen05 kernel: > 0 = one row tile per cluster of `kslices` CTAs, each taking a slice of K;
                      // the slices are summed through distributed shared memory (no global partials)
};

// The dense epilogue's store: output element (token row `tok`, weight row `row`) with the caller's options -- the Store
// epilogue of the reference's GEMV with out_f32 and n_split (crates/kernels/cu/gemv.cu:510-517, cu/tcgemm.cu:117-134).
DSUF_DEV void dense_store(const StreamArgs& a, int tok, int row, float v) {
    void* ob = a.out;
    int ld = a.ldo, col = row;
    if (a.n_split > 0 && row >= a.n_split) { ob = a.out2; ld = a.ldo2; col = row - a.n_split; }
    if (a.ssp) v = sqrtf(v > 20.f ? v : log1pf(expf(v)));
    if (a.accumulate) ((float*)ob)[(size_t)tok * ld + col] += v;
    else if (a.out_f32) ((float*)ob)[(size_t)tok * ld + col] = v;
    else ((__nv_bfloat16*)ob)[(size_t)tok * ld + col] = __float2bfloat16(v);
}

// The same store with the reference's fused rotary embedding (crates/kernels/cu/gemv.cu:508-516): rows of the first output
// whose position inside their head is at least rope_off are rotated in (even, odd) pairs with the token's cos / sin,
// operands rounded to bf16 first, one fma per output as the reference writes them; every other row is stored as usual.
// `v` is this row's value, `partner` the value of row ^ 1 (the neighbouring lane).  bf16 output.
DSUF_DEV void dense_store_rope(const StreamArgs& a, int tok, int row, float v, float partner) {
    const int hd = row % a.rope_head;
    if ((a.n_split > 0 && row >= a.n_split) || hd < a.rope_off) {
        dense_store(a, tok, row, v);
        return;
    }
    const float x = __bfloat162float(__float2bfloat16(v)), y = __bfloat162float(__float2bfloat16(partner));
    const int pos = a.rope_pos[0] + tok, f = (hd - a.rope_off) >> 1;
    const float c = a.rope_cos[(size_t)pos * 32 + f], sn = a.rope_sin[(size_t)pos * 32 + f];
    const float o = (row & 1) ? __fmaf_rn(y, sn, __fmul_rn(x, c)) : __fmaf_rn(x, c, -__fmul_rn(y, sn));
    ((__nv_bfloat16*)a.out)[(size_t)tok * a.ldo + row] = __float2bfloat16(o);
}

template <int FMT>
struct StreamCfg {
    static constexpr int W_BYTES = FMT == FMT_FP8 ? 16384 : 8192;
    static constexpr int X_OFF = W_BYTES;
    static constexpr int SF_OFF = W_BYTES + 2048;   // 512-byte weight scale atom
    static constexpr int XS_OFF = SF_OFF + 512;     // 16 activation block scales (4 bytes each)
    static constexpr int WS_OFF = XS_OFF + 64;      // dense DS geometry: the tile's fp32 weight scale
    static constexpr int STAGE = W_BYTES + 2048 + 1024;
    static constexpr int STAGES = FMT == FMT_FP8 ? 10 : 16;
    static constexpr int SMEM = STAGE * STAGES + 1024;  // +1024: manual alignment of the ring
};

template <int FMT, int WMX, int AMX, int NT8, int EPI>
__global__ void __launch_bounds__(STREAM_THREADS, 1) stream_gemv_kernel(const __grid_constant__ StreamArgs a) {
    using Cfg = StreamCfg<FMT>;
    constexpr int S = Cfg::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t full_bar[S], empty_bar[S];
    __shared__ int s_flag;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, c = blockIdx.x;
    const int RT = a.RT, KT = a.KT;
    bool dead = false;

    if (tid == 0) {
        for (int s = 0; s < S; ++s) {
            mbar_init(&full_bar[s], 1 + 32);  // expect_tx arrival + one cp.async arrival per producer lane
            mbar_init(&empty_bar[s], STREAM_CONSUMER_WARPS);
        }
        mbar_fence_init();
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap

    // ---- this CTA's span of the global tile sequence ----
    long long beg, end;
    if (EPI == EPI_DENSE && a.whole_items) {
        beg = ((long long)c * RT / G) * KT;
        end = ((long long)(c + 1) * RT / G) * KT;
    } else if (EPI == EPI_DENSE) {
        const long long tot = (long long)RT * KT;
        beg = (long long)c * tot / G;
        end = (long long)(c + 1) * tot / G;
    } else {
        const long long q = (long long)(*a.nslots) * RT;
        beg = ((long long)c * q / G) * KT;
        end = ((long long)(c + 1) * q / G) * KT;
    }

    if (warp == STREAM_CONSUMER_WARPS) {
        // ================= producer =================
        // lane 0 feeds the ring with TMA (weight tile, scale atom, activation tile); lanes 0..16 add the tile's
        // activation / weight block scales with 4-byte asynchronous copies, so consumers never touch global memory.
        if (beg < end) {
            if (lane == 0) {
                prefetch_tmap(&a.tm_w);
                prefetch_tmap(&a.tm_x);
            }
            const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
            long long q = beg / KT;
            int kt = (int)(beg - q * KT);
            int rt = 0, xrow0 = 0;
            long long wbase = 0;
            bool fresh = true;
            int n = 0;
            for (long long i = beg; i < end; ++i, ++n) {
                if (fresh) {
                    if (EPI == EPI_DENSE) {
                        rt = (int)q;
                        wbase = (long long)rt * KT;
                        xrow0 = 0;
                    } else {
                        const int slot = (int)(q / RT);
                        rt = (int)(q - (long long)slot * RT);
                        const int4 sl = a.slots[slot];
                        wbase = ((long long)sl.x * RT + rt) * KT;
                        xrow0 = sl.y;
                    }
                    fresh = false;
                }
                const int s = n % S;
                // after the first expired wait nothing is waited for again: the loops stay finite and short
                if (n >= S && !dead && !mbar_wait(&empty_bar[s], ((n / S) - 1) & 1, a.status, KID_STREAM, 1)) dead = true;
                uint8_t* st = ring + (size_t)s * Cfg::STAGE;
                if (lane == 0) {
                    const uint32_t bytes = Cfg::W_BYTES + NT8 * 1024 + (WMX ? 512 : 0);
                    mbar_expect_tx(&full_bar[s], bytes);
                    const long long tile = wbase + kt;
                    tma_3d(st, &a.tm_w, 0, 0, (int)tile, &full_bar[s], pol_w);
                    if (WMX) bulk_g2s(st + Cfg::SF_OFF, a.wtiles + (size_t)tile * a.rec_bytes + a.codes_bytes, 512, &full_bar[s], pol_w);
                    tma_2d(st + Cfg::X_OFF, &a.tm_x, kt * 128, xrow0, &full_bar[s], pol_x);
                }
                if (lane < 8 * NT8) {
                    const int r = min(xrow0 + lane, a.x_rows - 1);
                    cp_async4(st + Cfg::XS_OFF + 4 * lane, (const uint32_t*)a.xscale + (size_t)r * KT + kt);
                } else if (!WMX && lane == 16) {
                    cp_async4(st + Cfg::WS_OFF, a.wscale_ds + (size_t)rt * KT + kt);
                }
                cp_async_arrive_noinc(&full_bar[s]);
                __syncwarp();
                if (++kt == KT) { kt = 0; ++q; fresh = true; }
            }
        }
    } else {
        // ================= consumers =================
        const int g = lane >> 2, t = lane & 3;
        const int rg = rowmap8(g);                  // tile row (mod 8) this lane's fragment rows map to
        const int ra = warp * 16 + rg, rb = ra + 8; // rows inside the 128-row tile
        const int ca = rowmap8(2 * t), cb = rowmap8(2 * t + 1);  // activation-box rows of fragment columns 2t, 2t+1
        float acc[NT8][4];
#pragma unroll
        for (int u = 0; u < NT8; ++u)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[u][i] = 0.f;

        long long q = beg / KT;
        int kt = (int)(beg - q * KT);
        int rt = 0, xrow0 = 0, cnt = 0;
        bool fresh = true;
        int n = 0;
        for (long long i = beg; i < end; ++i, ++n) {
            if (fresh) {
                if (EPI == EPI_DENSE) {
                    rt = (int)q;
                    xrow0 = 0;
                    cnt = a.m;
                } else {
                    const int slot = (int)(q / RT);
                    rt = (int)(q - (long long)slot * RT);
                    const int4 sl = a.slots[slot];
                    xrow0 = sl.y;
                    cnt = sl.z;
                }
                fresh = false;
            }
            const int s = n % S;
            if (!dead && !mbar_wait(&full_bar[s], (n / S) & 1, a.status, KID_STREAM, 2)) dead = true;
            const uint8_t* st = ring + (size_t)s * Cfg::STAGE;
            // block scales of this tile, staged next to it by the producer warp
            float xsa[NT8], xsb[NT8];
            uint32_t xma[NT8], xmb[NT8];
#pragma unroll
            for (int u = 0; u < NT8; ++u) {
                xma[u] = *(const uint32_t*)(st + Cfg::XS_OFF + 4 * (8 * u + ca));
                xmb[u] = *(const uint32_t*)(st + Cfg::XS_OFF + 4 * (8 * u + cb));
                xsa[u] = __uint_as_float(xma[u]);
                xsb[u] = __uint_as_float(xmb[u]);
            }
            float wds = 1.f;
            if (!WMX) wds = *(const float*)(st + Cfg::WS_OFF);
            uint32_t wsa = 0, wsb = 0;
            if (WMX) {
                wsa = *(const uint32_t*)(st + Cfg::SF_OFF + (ra & 31) * 16 + (ra >> 5) * 4);
                wsb = *(const uint32_t*)(st + Cfg::SF_OFF + (rb & 31) * 16 + (rb >> 5) * 4);
            }
            float tacc[NT8][4];
#pragma unroll
            for (int u = 0; u < NT8; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e) tacc[u][e] = 0.f;

#pragma unroll
            for (int j = 0; j < 4; ++j) {
                uint32_t a0, a1, a2, a3;
                if (FMT == FMT_FP8) {
                    const int ch = (((2 * j + (t >> 1)) ^ rg) << 4) + 8 * (t & 1);
                    const uint2 va = *(const uint2*)(st + ra * 128 + ch);
                    const uint2 vb = *(const uint2*)(st + rb * 128 + ch);
                    a0 = va.x; a2 = va.y; a1 = vb.x; a3 = vb.y;
                } else {
                    const int ch = ((j ^ ((rg >> 1) & 3)) << 4) + 4 * t;
                    const uint32_t wa = *(const uint32_t*)(st + ra * 64 + ch);
                    const uint32_t wb = *(const uint32_t*)(st + rb * 64 + ch);
                    e2m1x8_to_e4m3(wa, a0, a2);
                    e2m1x8_to_e4m3(wb, a1, a3);
                }
#pragma unroll
                for (int u = 0; u < NT8; ++u) {
                    const int xr = 8 * u + rg;
                    const uint2 vx = *(const uint2*)(st + Cfg::X_OFF + xr * 128 + (((2 * j + (t >> 1)) ^ rg) << 4) + 8 * (t & 1));
                    uint32_t b0 = vx.x, b1 = vx.y;
                    if (FMT == FMT_FP4) {
                        b0 = __byte_perm(vx.x, vx.y, 0x6420);
                        b1 = __byte_perm(vx.x, vx.y, 0x7531);
                    }
                    if (FMT == FMT_FP8 && !WMX) {
                        mma_e4m3(tacc[u], a0, a1, a2, a3, b0, b1);  // one 128-K block, one scale pair
                    } else {
                        float cfr[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_e4m3(cfr, a0, a1, a2, a3, b0, b1);
                        const float fa = e8m0_to_f32(wsa >> (8 * j)), fb = e8m0_to_f32(wsb >> (8 * j));
                        if (AMX) {
                            const float ya = e8m0_to_f32(xma[u] >> (8 * j)), yb = e8m0_to_f32(xmb[u] >> (8 * j));
                            acc[u][0] = fmaf(cfr[0], fa * ya, acc[u][0]);
                            acc[u][1] = fmaf(cfr[1], fa * yb, acc[u][1]);
                            acc[u][2] = fmaf(cfr[2], fb * ya, acc[u][2]);
                            acc[u][3] = fmaf(cfr[3], fb * yb, acc[u][3]);
                        } else {
                            tacc[u][0] = fmaf(cfr[0], fa, tacc[u][0]);
                            tacc[u][1] = fmaf(cfr[1], fa, tacc[u][1]);
                            tacc[u][2] = fmaf(cfr[2], fb, tacc[u][2]);
                            tacc[u][3] = fmaf(cfr[3], fb, tacc[u][3]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[s]);
            if (!AMX) {
#pragma unroll
                for (int u = 0; u < NT8; ++u) {
                    const float fa = wds * xsa[u], fb = wds * xsb[u];
                    acc[u][0] = fmaf(tacc[u][0], fa, acc[u][0]);
                    acc[u][1] = fmaf(tacc[u][1], fb, acc[u][1]);
                    acc[u][2] = fmaf(tacc[u][2], fa, acc[u][2]);
                    acc[u][3] = fmaf(tacc[u][3], fb, acc[u][3]);
                }
            }

            if (++kt == KT || i + 1 == end) {
                // ---------------- flush the item ----------------
                const float unscale = FMT == FMT_FP4 ? E2M1_UNSCALE : 1.0f;
                if (EPI == EPI_DENSE) {
                    const long long it0 = q * KT;
                    const bool whole = beg <= it0 && end >= it0 + KT;
                    const int ctid = tid;  // consumer threads are 0..255
                    bool do_store = whole;
                    if (!whole) {
                        const int slot = (q == beg / KT) ? 0 : 1;
                        float* pw = a.partial + ((size_t)(c * 2 + slot) * (4 * NT8)) * 256 + ctid;
#pragma unroll
                        for (int u = 0; u < NT8; ++u)
#pragma unroll
                            for (int e = 0; e < 4; ++e) __stcg(pw + (size_t)(u * 4 + e) * 256, acc[u][e]);
                        __threadfence();
                        named_bar_sync(1, STREAM_CONSUMER_WARPS * 32);
                        const long long tot = (long long)RT * KT;
                        const int first = (int)(((it0 + 1) * G - 1) / tot);
                        const int last = (int)(((it0 + KT) * G - 1) / tot);
                        if (ctid == 0) {
                            const int old = atomicAdd(a.counters + q, 1);
                            s_flag = (old == last - first);
                            if (old == last - first) a.counters[q] = 0;  // self-resetting for the next launch
                        }
                        named_bar_sync(1, STREAM_CONSUMER_WARPS * 32);
                        do_store = s_flag != 0;
                        named_bar_sync(1, STREAM_CONSUMER_WARPS * 32);
                        if (do_store) {
                            __threadfence();
#pragma unroll
                            for (int u = 0; u < NT8; ++u)
#pragma unroll
                                for (int e = 0; e < 4; ++e) acc[u][e] = 0.f;
                            for (int cc = first; cc <= last; ++cc) {  // fixed order: results do not depend on arrival order
                                const long long cbeg = (long long)cc * tot / G;
                                const int cslot = (q == cbeg / KT) ? 0 : 1;
                                const float* pr = a.partial + ((size_t)(cc * 2 + cslot) * (4 * NT8)) * 256 + ctid;
#pragma unroll
                                for (int u = 0; u < NT8; ++u)
#pragma unroll
                                    for (int e = 0; e < 4; ++e) acc[u][e] += __ldcg(pr + (size_t)(u * 4 + e) * 256);
                            }
                        }
                    }
                    if (do_store) {
#pragma unroll
                        for (int u = 0; u < NT8; ++u)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int tok = 8 * u + ((e & 1) ? cb : ca);
                                const int row = rt * 128 + ((e & 2) ? rb : ra);
                                if (tok < cnt && row < a.n_rows) dense_store(a, tok, row, acc[u][e] * a.alpha * unscale);
                            }
                    }
                } else if (EPI == EPI_W13) {
                    // rows 0..7 of each 16-row group are gate rows, rows 8..15 the matching up rows
                    // (SwiGLU as cu/gemv.cu:470-483: bf16 rounds, optional clamp, routing weight folded in)
                    bf16* o = (bf16*)a.out;
                    const float L = a.swiglu_limit;
#pragma unroll
                    for (int u = 0; u < NT8; ++u)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const int tk = 8 * u + (e ? cb : ca);
                            if (tk < cnt) {
                                const int row = xrow0 + tk;
                                float gt = bf16_round(acc[u][e] * unscale), up = bf16_round(acc[u][2 + e] * unscale);
                                if (L > 0.f) { up = fminf(fmaxf(up, -L), L); gt = fminf(gt, L); }
                                const float v = gt / (1.0f + expf(-gt)) * up * __ldg(a.row_w + row);
                                o[(size_t)row * a.ldo + rt * 64 + warp * 8 + rg] = __float2bfloat16(v);
                            }
                        }
                } else {
                    float* o = (float*)a.out;
#pragma unroll
                    for (int u = 0; u < NT8; ++u)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int tk = 8 * u + ((e & 1) ? cb : ca);
                            const int col = rt * 128 + ((e & 2) ? rb : ra);
                            if (tk < cnt && col < a.n_rows) o[(size_t)(xrow0 + tk) * a.ldo + col] = acc[u][e] * unscale;
                        }
                }
#pragma unroll
                for (int u = 0; u < NT8; ++u)
#pragma unroll
                    for (int e = 0; e < 4; ++e) acc[u][e] = 0.f;
                if (kt == KT) { kt = 0; ++q; fresh = true; }
            }
        }
    }
}

}  // namespace dsuf
