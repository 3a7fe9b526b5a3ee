// Output-head projection of a decode step: logits[m][v] = alpha * <x[m], W[v]> over a bf16 [vocab][K] weight, for up to 16
// token rows, with optional per-64-row sampling records.
//
// Replaces gemv_bf16_persist_p4 (crates/kernels/cu/gemv.cu:542-689: a persistent mma.sync GEMV over weights re-tiled on
// the host, one CTA walking 64-row quads, records written by the CTA that produced the quad).  Here the weight stays in
// its checkpoint layout (row-major bf16, no host re-tiling): TMA lands 128-row x 64-K boxes in shared memory in the
// tensor core's 128-byte-swizzled operand layout, tcgen05.mma kind::f16 multiplies them with the token rows ("swap-AB":
// the 128 vocabulary rows are the MMA's M, the 16 token rows its N), the whole K accumulates in tensor memory, and four
// epilogue warps store fp32 logits and build the records while the next row tile streams.  HBM-bound: 2 bytes per
// weight element (1.85 GB for 129280 x 7168).
//
// Sampling record of (token m, quad q = 64 vocabulary rows), 20 floats at spart[(m * n/64 + q) * 20], the layout the
// reference's sampler merges (cu/gemv.cu:651-688): [0] max of z, [1] sum of exp(z - max), [2] the 9th largest z,
// [3..10] the 8 largest z in descending order, [11..18] their vocabulary ids (int bits; ties go to the lower id),
// where z = logit / temperature for rows below sp_vloc and -inf otherwise, id = row + sp_off.
#include "internal.h"

namespace dsuf {

constexpr int KID_LMHEAD = 6;
constexpr int LH_NTOK = 16;                       // token columns of the MMA (rows beyond m are zero-filled by TMA)
constexpr int LH_KB = 64;                         // bf16 elements per 128-byte operand row
constexpr int LH_KPS = 2;                         // 64-K blocks per ring stage
constexpr int LH_A1 = 128 * 128;                  // one weight box: 128 rows x 128 bytes
constexpr int LH_B1 = LH_NTOK * 128;              // one token box
constexpr int LH_STAGE = LH_KPS * (LH_A1 + LH_B1);  // 36864
constexpr int LH_STAGES = 6;
constexpr int LH_SMEM = LH_STAGES * LH_STAGE + 1024;
constexpr int LH_THREADS = 192;                   // warp 0 producer, 1 MMA issuer, 2-5 epilogue
constexpr int LH_TM_COLS = 32;                    // two accumulators of 16 columns

struct LmHeadArgs {
    CUtensorMap tm_w, tm_x;
    float* out;           // [m][ldo] fp32
    int ldo, m, n, k;
    float alpha;
    float* spart;         // sampling records or null
    float inv_temp;
    int sp_vloc, sp_off;
    DevStatus* status;
};

// kind::f16 instruction descriptor: fp32 accumulator (bit 4), bf16 A and B (1 at bits 7 and 10), both K-major, N / 8 at
// bit 17, M / 16 at bit 24.
DSUF_DEV uint32_t lh_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(LH_NTOK / 8) << 17) | ((uint32_t)(128 / 16) << 24);
}
DSUF_DEV void lh_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        "  .reg .pred keep_d;\n"
        "  setp.ne.u32 keep_d, %4, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, keep_d;\n"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

__global__ void __launch_bounds__(LH_THREADS, 1) lm_head_kernel(const __grid_constant__ LmHeadArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* ring = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    __shared__ __align__(8) uint64_t full_bar[LH_STAGES], empty_bar[LH_STAGES], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t s_tmem;
    __shared__ float s_z[LH_NTOK][128];   // the tile's z values, for the records
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int RT = (a.n + 127) / 128, KS = (a.k + LH_KB * LH_KPS - 1) / (LH_KB * LH_KPS);   // row tiles, ring stages per tile
    bool dead = false;

    if (warp == 1) {
        tmem_alloc(&s_tmem, LH_TM_COLS);
        tmem_relinquish();
    }
    if (tid == 0) {
        for (int s = 0; s < LH_STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tfull_bar[b], 1);
            mbar_init(&tempty_bar[b], 4);
        }
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s_tmem;
    pdl_wait();
    pdl_launch_dependents();

    // row tiles are dealt round-robin: CTA c takes tiles c, c + grid, ...
    if (warp == 0) {
        // ---------------- producer: weight and token boxes of every stage ----------------
        if (lane == 0) {
            prefetch_tmap(&a.tm_w);
            prefetch_tmap(&a.tm_x);
        }
        const uint64_t pol_w = policy_evict_first(), pol_x = policy_evict_last();
        int s = 0;
        uint32_t ph = 0;
        long long n = 0;
        for (int rt = blockIdx.x; rt < RT; rt += gridDim.x) {
            for (int ks = 0; ks < KS; ++ks, ++n) {
                if (n >= LH_STAGES && !dead && !mbar_wait(&empty_bar[s], ph ^ 1, a.status, KID_LMHEAD, 1)) dead = true;
                if (warp_elect()) {
                    uint8_t* st = ring + s * LH_STAGE;
                    // (a box that starts beyond K or beyond the last row is zero-filled and still counts its full size)
                    mbar_expect_tx(&full_bar[s], LH_STAGE);
#pragma unroll
                    for (int kb = 0; kb < LH_KPS; ++kb) {
                        const int kbyte = (ks * LH_KPS + kb) * 128;
                        tma_2d(st + kb * LH_A1, &a.tm_w, kbyte, rt * 128, &full_bar[s], pol_w);
                        tma_2d(st + LH_KPS * LH_A1 + kb * LH_B1, &a.tm_x, kbyte, 0, &full_bar[s], pol_x);
                    }
                }
                __syncwarp();
                if (++s == LH_STAGES) { s = 0; ph ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer: the whole warp runs the loop, one elected lane issues ----------------
        const uint32_t idesc = lh_idesc();
        const uint32_t tmu = warp_uniform(tm);
        const uint64_t ad0 = warp_uniform(tc_smem_desc(ring, 16, 1024, TC_SWIZZLE_128B));
        const uint64_t bd0 = warp_uniform(tc_smem_desc(ring + LH_KPS * LH_A1, 16, 1024, TC_SWIZZLE_128B));
        int s = 0, item = 0;
        uint32_t ph = 0;
        for (int rt = blockIdx.x; rt < RT; rt += gridDim.x, ++item) {
            const int ab = item & 1;
            if (item >= 2 && !dead && !mbar_wait(&tempty_bar[ab], ((item >> 1) - 1) & 1, a.status, KID_LMHEAD, 2)) dead = true;
            tc_fence_after();
            for (int ks = 0; ks < KS; ++ks) {
                if (!dead && !mbar_wait(&full_bar[s], ph, a.status, KID_LMHEAD, 3)) dead = true;
                tc_fence_after();
                if (warp_elect()) {
                    const uint64_t so = (uint64_t)((s * LH_STAGE) >> 4);
#pragma unroll
                    for (int kb = 0; kb < LH_KPS; ++kb) {
#pragma unroll
                        for (int kc = 0; kc < 4; ++kc) {   // four K = 16 steps of 32 bytes inside a 128-byte row
                            const uint64_t ad = ad0 + so + (uint64_t)((kb * LH_A1 + kc * 32) >> 4);
                            const uint64_t bd = bd0 + so + (uint64_t)((kb * LH_B1 + kc * 32) >> 4);
                            lh_mma(tmu + ab * LH_NTOK, ad, bd, idesc, (ks | kb | kc) != 0);
                        }
                    }
                    tc_commit(&empty_bar[s]);   // the stage is free once these MMAs have read it
                }
                __syncwarp();
                if (++s == LH_STAGES) { s = 0; ph ^= 1; }
            }
            if (warp_elect()) tc_commit(&tfull_bar[ab]);
            __syncwarp();
        }
    } else {
        // ---------------- epilogue: 4 warps = 128 vocabulary rows of the tile ----------------
        const int ew = warp - 2;             // 0..3
        const int q4 = warp & 3;             // the tensor-memory lane quarter this warp may read
        const int r = q4 * 32 + lane;        // row inside the tile
        int item = 0;
        for (int rt = blockIdx.x; rt < RT; rt += gridDim.x, ++item) {
            const int ab = item & 1;
            if (!dead && !mbar_wait(&tfull_bar[ab], (item >> 1) & 1, a.status, KID_LMHEAD, 4)) dead = true;
            tc_fence_after();
            float v[LH_NTOK];
            tmem_ld<LH_NTOK>(tm + ((uint32_t)(q4 * 32) << 16) + ab * LH_NTOK, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[ab]);
            const int row = rt * 128 + r;
#pragma unroll
            for (int m = 0; m < LH_NTOK; ++m) {
                const float logit = v[m] * a.alpha;
                if (m < a.m && row < a.n) a.out[(size_t)m * a.ldo + row] = logit;
                if (a.spart) s_z[m][r] = row < a.sp_vloc && row < a.n ? logit * a.inv_temp : -INFINITY;
            }
            if (a.spart) {
                named_bar_sync(1, 128);
                // (token, half tile) pairs dealt to the four warps; a lane holds two of the quad's 64 values
                const int nq = a.n / 64;
                for (int p = ew; p < a.m * 2; p += 4) {
                    const int m = p >> 1, h = p & 1, q = rt * 2 + h;
                    if (q >= nq) continue;
                    const float z0 = s_z[m][h * 64 + lane], z1 = s_z[m][h * 64 + 32 + lane];
                    // one 64-bit word per candidate: the value mapped to an unsigned that orders like the float, then
                    // the complement of the id, so the largest word is the best value and, among equals, the lowest id
                    unsigned long long c[2];
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float z = e ? z1 : z0;
                        const unsigned bits = __float_as_uint(z);
                        const unsigned ordered = (bits >> 31) ? ~bits : (bits | 0x80000000u);
                        const unsigned id = (unsigned)(q * 64 + lane + 32 * e + a.sp_off);
                        c[e] = ((unsigned long long)ordered << 32) | (0xffffffffu - id);
                    }
                    float* rec = a.spart + ((size_t)m * nq + q) * 20;
                    float zmax = -INFINITY;
                    for (int k = 0; k < 9; ++k) {
                        const unsigned long long mine = c[0] > c[1] ? c[0] : c[1];
                        const unsigned hi = (unsigned)(mine >> 32);
                        const unsigned top_hi = __reduce_max_sync(0xffffffffu, hi);
                        const unsigned top_lo = __reduce_max_sync(0xffffffffu, hi == top_hi ? (unsigned)mine : 0u);
                        const unsigned long long best = ((unsigned long long)top_hi << 32) | top_lo;
                        const float bz = __uint_as_float((top_hi & 0x80000000u) ? (top_hi & 0x7fffffffu) : ~top_hi);
                        if (k == 0) zmax = bz;
                        if (lane == 0) {
                            if (k < 8) {
                                rec[3 + k] = bz;
                                rec[11 + k] = __int_as_float((int)(0xffffffffu - top_lo));
                            } else {
                                rec[2] = bz;
                            }
                        }
                        if (c[0] == best) c[0] = 0ull;   // retired: below every real candidate (-inf maps above 0)
                        if (c[1] == best) c[1] = 0ull;
                    }
                    float se = (z0 == -INFINITY ? 0.f : expf(z0 - zmax)) + (z1 == -INFINITY ? 0.f : expf(z1 - zmax));
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) se += __shfl_xor_sync(0xffffffffu, se, o);
                    if (lane == 0) {
                        rec[0] = zmax;
                        rec[1] = se;
                    }
                }
                named_bar_sync(1, 128);   // s_z is rewritten by the next tile
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 1) tmem_dealloc(tm, LH_TM_COLS);
}

static int encode_bf16_rows(dsuf_ctx* ctx, CUtensorMap* tm, const void* base, int k, long long ld_elems, long long rows, int box_rows) {
    cuuint64_t dims[2] = {(cuuint64_t)k * 2, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld_elems * 2};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1u, 1u};
    CUresult r = ctx->encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, DSUF_E_BADARG, "cuTensorMapEncodeTiled(lm head) failed: %d", (int)r);
    return DSUF_OK;
}

int lm_head_setup(dsuf_ctx* ctx) {
    cudaError_t e = cudaFuncSetAttribute(lm_head_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LH_SMEM);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(lm_head)");
    return DSUF_OK;
}

}  // namespace dsuf

using namespace dsuf;

extern "C" int32_t dsuf_lm_head_bf16(dsuf_ctx* ctx, void* stream, uint64_t w, int32_t n, int32_t k, uint64_t x, int32_t ldx, int32_t m,
                                     float alpha, uint64_t out, int32_t ldo, const dsuf_sampling_opts* sp) {
    if (!ctx) return DSUF_E_BADARG;
    if (m == 0) return DSUF_OK;   // an empty batch: nothing to launch (and no pointer to look at)
    DSUF_REQUIRE(ctx, w && x && out && (w & 15) == 0 && (x & 15) == 0 && (out & 3) == 0, "lm_head: null or misaligned pointer");
    DSUF_REQUIRE(ctx, n > 0 && k > 0 && k % 8 == 0 && ldx >= k && ldx % 8 == 0, "lm_head: k and ldx must be multiples of 8, ldx >= k");
    DSUF_REQUIRE(ctx, m > 0 && m <= LH_NTOK && ldo >= n, "lm_head: 0..%d token rows, ldo >= n", LH_NTOK);
    LmHeadArgs a;
    memset(&a, 0, sizeof(a));
    int rc = encode_bf16_rows(ctx, &a.tm_w, (const void*)w, k, k, n, 128);
    if (rc) return rc;
    rc = encode_bf16_rows(ctx, &a.tm_x, (const void*)x, k, ldx, m, LH_NTOK);
    if (rc) return rc;
    a.out = (float*)out;
    a.ldo = ldo; a.m = m; a.n = n; a.k = k;
    a.alpha = alpha;
    a.status = ctx->dev_status;
    if (sp && sp->records) {
        DSUF_REQUIRE(ctx, n % 64 == 0 && sp->temperature > 0.f && (sp->records & 3) == 0, "lm_head: records need n %% 64 == 0 and a temperature > 0");
        a.spart = (float*)sp->records;
        a.inv_temp = 1.0f / sp->temperature;
        a.sp_vloc = sp->valid_rows > 0 ? sp->valid_rows : n;
        a.sp_off = sp->id_offset;
    }
    const int rt = (n + 127) / 128;
    const int grid = rt < ctx->sm_count ? rt : ctx->sm_count;
    return launch(ctx, (cudaStream_t)stream, lm_head_kernel, dim3(grid), dim3(LH_THREADS), (size_t)LH_SMEM, a);
}
