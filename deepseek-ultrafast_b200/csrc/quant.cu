// FP8 (e4m3) activation quantization, stand-alone and fused with the routed-token scatter.
//
// Replaces tc_quant_rows (crates/kernels/cu/tcgemm.cu:300-340, with its optional RMS pre-normalisation and
// tc_row_sumsq, :341-355), the per-CTA quant_blocks8 staging of the decode
// GEMVs (cu/quantblocks.cuh:7-57) and moe_gather_quant (cu/tcmoe.cu:88-133).  Activations are quantized ONCE per
// token by this kernel; every GEMM consumer reads the codes.
//   MX geometry: 1x32 blocks, scale 2^ceil(log2(max(amax,1e-4)/448)) stored as UE8M0, exact reciprocal by
//                exponent flip (bit-identical to the reference).
//   DS geometry: 1x128 blocks, fp32 scale = amax/448 (1 for an all-zero block), code = rne(x / scale) with IEEE
//                division.
// HBM-bound: reads 2 B and writes ~1.03 B (x fan-out for the scatter form) per element; 16-byte loads,
// 8-byte stores, amax by warp shuffles.
#include "internal.h"
#include "quant_core.cuh"

namespace dsuf {

struct QuantArgs {
    const bf16* x;        // [rows_in][ldx]
    int ldx, rows_in, k;
    uint8_t* q;           // [rows_out][k]
    void* scales;         // MX: u8 [rows_out][k/32], DS: f32 [rows_out][k/128]
    const int* pair_row;  // scatter form: destination rows of token t are pair_row[t*fanout + j] (<0: skipped)
    int fanout;           // 0: plain (row r -> row r)
    const bf16* norm_w;   // RMS pre-normalisation weights [k], or null
    const float* sumsq;   // pre-normalisation: sum of squares of every input row (row_sumsq_kernel)
    float eps;
    int approx_rsqrt;     // pre-normalisation: 1 = the reference's rsqrtf (approximate instruction), 0 = correctly rounded 1/sqrt
};

template <int MODE>
__global__ void __launch_bounds__(256) act_quant_kernel(const QuantArgs a) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int row = blockIdx.x;
    const int k0 = (blockIdx.y * 256 + threadIdx.x) * 8;
    const bool live = k0 < a.k;
    float v[8];
    if (live) {
        const uint4 raw = *(const uint4*)(a.x + (size_t)row * a.ldx + k0);
        const bf16* h = (const bf16*)&raw;
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(h[e]);
        if (a.norm_w) {
            // tc_quant_rows with pw (cu/tcgemm.cu:316-320): v = bf16(w * (x * rs)), every product rounded on its own.
            // rs by correctly rounded sqrt and division by default (the reference's rsqrtf is a 2-ulp approximation).
            // With approx_rsqrt the same instruction is used and the codes are the reference kernel's on the same GPU.
            const float ms = __fadd_rn(__fdiv_rn(a.sumsq[row], (float)a.k), a.eps);
            const float rs = a.approx_rsqrt ? rsqrtf(ms) : __fdiv_rn(1.0f, __fsqrt_rn(ms));
            const uint4 wraw = *(const uint4*)(a.norm_w + k0);
            const bf16* hw = (const bf16*)&wraw;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[e] = bf16_round(__fmul_rn(__bfloat162float(hw[e]), __fmul_rn(v[e], rs)));
        }
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = 0.f;
    }
    constexpr int LANES = MODE == DSUF_MODE_MX ? 4 : 16;  // lanes sharing one scale block
    float sc;
    uint2 out;
    quant8<MODE>(v, out, sc);
    if (!live) return;
    const bool writes_scale = (threadIdx.x & (LANES - 1)) == 0;
    const int nfan = a.fanout > 0 ? a.fanout : 1;
    for (int j = 0; j < nfan; ++j) {
        const int dst = a.fanout > 0 ? a.pair_row[(size_t)row * a.fanout + j] : row;
        if (dst < 0) continue;
        *(uint2*)(a.q + (size_t)dst * a.k + k0) = out;
        if (writes_scale) {
            if (MODE == DSUF_MODE_MX) {
                const int kb = k0 >> 5;
                const uint8_t b = (uint8_t)(__float_as_uint(sc) >> 23);
                ((uint8_t*)a.scales)[(size_t)dst * (a.k >> 5) + kb] = b;
            } else {
                ((float*)a.scales)[(size_t)dst * (a.k >> 7) + (k0 >> 7)] = sc;
            }
        }
    }
}

// Large inputs (thousands of rows, no scatter, no pre-normalisation): one CTA per row, one whole 32-element block per
// thread -- four independent 16-byte loads in flight per thread and, in the MX geometry, no shuffle at all (a DS scale
// block is four neighbouring threads).  Same arithmetic as quant8, so codes and scales are bit-identical to the kernel
// above.
template <int MODE>
__global__ void __launch_bounds__(256) act_quant_rows_kernel(const bf16* x, int ldx, int k, uint8_t* q, void* scales) {
    pdl_wait();
    pdl_launch_dependents();  // dependents still wait for this grid to finish; only their prologues overlap
    const int row = blockIdx.x, nkb = k >> 5;
    // (k % 128 == 0: the four threads of a DS block are live or dead together, and all in one warp)
    for (int kb0 = 0; kb0 < nkb; kb0 += 256) {
        const int kb = kb0 + threadIdx.x;
        const bool live = kb < nkb;
        float v[32];
        if (live) {
            const bf16* xr = x + (size_t)row * ldx + kb * 32;
            uint4 raw[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) raw[j] = *(const uint4*)(xr + 8 * j);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bf16* h = (const bf16*)&raw[j];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[8 * j + e] = __bfloat162float(h[e]);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
        }
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
        uint32_t w[8];
        if (MODE == DSUF_MODE_MX) {
            const float sc = round_scale_pow2(fmaxf(amax, 1e-4f), 1.0f / 448.0f);
            const float inv = __uint_as_float(0x7f000000u - __float_as_uint(sc));
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = f32x4_to_e4m3x4(v[4 * j] * inv, v[4 * j + 1] * inv, v[4 * j + 2] * inv, v[4 * j + 3] * inv);
            if (live) ((uint8_t*)scales)[(size_t)row * nkb + kb] = (uint8_t)(__float_as_uint(sc) >> 23);
        } else {
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const float sc = amax == 0.f ? 1.0f : __fdiv_rn(amax, 448.0f);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                w[j] = f32x4_to_e4m3x4(__fdiv_rn(v[4 * j], sc), __fdiv_rn(v[4 * j + 1], sc), __fdiv_rn(v[4 * j + 2], sc), __fdiv_rn(v[4 * j + 3], sc));
            if (live && (threadIdx.x & 3) == 0) ((float*)scales)[(size_t)row * (nkb >> 2) + (kb >> 2)] = sc;
        }
        if (live) {
            uint4* o = (uint4*)(q + (size_t)row * k + kb * 32);
            o[0] = make_uint4(w[0], w[1], w[2], w[3]);
            o[1] = make_uint4(w[4], w[5], w[6], w[7]);
        }
    }
}

// tc_row_sumsq (cu/tcgemm.cu:341-355), same summation order: one warp per row, lane l takes k = 8 l + 256 i + e.
__global__ void __launch_bounds__(256) row_sumsq_kernel(const bf16* x, int ldx, int m, int k, float* out) {
    pdl_wait();
    pdl_launch_dependents();
    const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= m) return;
    float ss = 0.f;
    for (int kk = lane * 8; kk < k; kk += 256) {
        const uint4 raw = *(const uint4*)(x + (size_t)row * ldx + kk);
        const bf16* h = (const bf16*)&raw;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float v = __bfloat162float(h[e]);
            ss = __fmaf_rn(v, v, ss);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
    if (lane == 0) out[row] = ss;
}

int launch_row_sumsq(dsuf_ctx* ctx, cudaStream_t stream, const void* x, int ldx, int m, int k, float* out) {
    if (m == 0) return DSUF_OK;
    return launch(ctx, stream, row_sumsq_kernel, dim3((m + 7) / 8), dim3(256), 0, (const bf16*)x, ldx, m, k, out);
}

int launch_act_quant(dsuf_ctx* ctx, cudaStream_t stream, int mode, const void* x, int ldx, int rows_in, int k, void* q,
                     void* scales, const int* pair_row, int fanout, const void* norm_w, const float* sumsq, float eps) {
    QuantArgs a{(const bf16*)x, ldx, rows_in, k, (uint8_t*)q, scales, pair_row, fanout, (const bf16*)norm_w, sumsq, eps, ctx->prenorm_approx};
    if (rows_in == 0) return DSUF_OK;
    // (rows of at least 6144 elements keep three quarters of the CTA's 256 threads busy; the 2048-wide SwiGLU output of
    // the expert layer does not: there the kernel above is several times faster)
    if (rows_in >= 1024 && k >= 6144 && !pair_row && !norm_w && ((uintptr_t)q & 15) == 0 && k % 128 == 0) {
        if (mode == DSUF_MODE_MX)
            return launch(ctx, stream, act_quant_rows_kernel<DSUF_MODE_MX>, dim3(rows_in), dim3(256), 0, (const bf16*)x, ldx, k, (uint8_t*)q, scales);
        return launch(ctx, stream, act_quant_rows_kernel<DSUF_MODE_DS>, dim3(rows_in), dim3(256), 0, (const bf16*)x, ldx, k, (uint8_t*)q, scales);
    }
    dim3 grid(rows_in, (k + 2047) / 2048);
    if (mode == DSUF_MODE_MX)
        return launch(ctx, stream, act_quant_kernel<DSUF_MODE_MX>, grid, dim3(256), 0, a);
    return launch(ctx, stream, act_quant_kernel<DSUF_MODE_DS>, grid, dim3(256), 0, a);
}

}  // namespace dsuf
