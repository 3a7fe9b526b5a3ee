// The quantizer's inner step, shared by the stand-alone / scatter kernel (quant.cu) and the fused decode front end
// (moe_aux.cu): eight consecutive bf16-valued floats per thread, the block's amax by warp shuffles.
#pragma once
#include "common.cuh"
#include "../../include/dsuf_qmm.h"

namespace dsuf {

// MODE MX: 1x32 blocks (4 lanes), scale 2^ceil(log2(max(amax, 1e-4) / 448)), exact reciprocal by exponent flip
//          (crates/kernels/cu/quantblocks.cuh:7-57, cu/tcgemm.cu:325-338);
// MODE DS: 1x128 blocks (16 lanes), fp32 scale amax / 448 (1 for an all-zero block), code = rne(x / scale), IEEE division.
// Every lane of the warp must call (lanes without data pass zeros).  `sc` is the block's scale in every lane of the block.
template <int MODE>
DSUF_DEV void quant8(const float (&v)[8], uint2& codes, float& sc) {
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    constexpr int LANES = MODE == DSUF_MODE_MX ? 4 : 16;
#pragma unroll
    for (int o = 1; o < LANES; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (MODE == DSUF_MODE_MX) {
        sc = round_scale_pow2(fmaxf(amax, 1e-4f), 1.0f / 448.0f);
        const float inv = __uint_as_float(0x7f000000u - __float_as_uint(sc));
        codes.x = f32x4_to_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        codes.y = f32x4_to_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
    } else {
        sc = amax == 0.f ? 1.0f : __fdiv_rn(amax, 448.0f);
        codes.x = f32x4_to_e4m3x4(__fdiv_rn(v[0], sc), __fdiv_rn(v[1], sc), __fdiv_rn(v[2], sc), __fdiv_rn(v[3], sc));
        codes.y = f32x4_to_e4m3x4(__fdiv_rn(v[4], sc), __fdiv_rn(v[5], sc), __fdiv_rn(v[6], sc), __fdiv_rn(v[7], sc));
    }
}

}  // namespace dsuf
