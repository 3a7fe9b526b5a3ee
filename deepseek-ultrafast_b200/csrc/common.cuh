// Device-side building blocks shared by every kernel of the library: mbarrier / TMA / PDL wrappers with
// bounded waits, FP8/FP4 codec helpers that mirror the reference's host codecs
// (crates/model/src/formats.rs:4-90, crates/kernels/cu/common.cuh:51-84), and the legacy tensor-core MMA used
// by the HBM-bound decode kernels.  sm_100a only.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define DSUF_DEV __device__ __forceinline__

namespace dsuf {

// Device status word layout (written by a kernel whose bounded wait expired, read by dsuf_status_poll).
struct DevStatus {
    int code;     // 0 = ok, otherwise DSUF_DEVERR_*
    int kernel;   // kernel id
    int cta;      // blockIdx.x of the reporter
    int where;    // site id inside the kernel
};
enum { DEVERR_NONE = 0, DEVERR_WAIT_TIMEOUT = 1, DEVERR_BAD_PLAN = 2 };

// Every spin in this library gives up after this many clock64 ticks (~2 s at 2 GHz) and reports instead of hanging.
constexpr long long WAIT_BUDGET_TICKS = 4000000000ll;

DSUF_DEV void report(DevStatus* st, int code, int kernel, int where) {
    if (st && atomicCAS(&st->code, 0, code) == 0) {
        st->kernel = kernel;
        st->cta = (int)blockIdx.x;
        st->where = where;
    }
}

DSUF_DEV uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- programmatic dependent launch ----
DSUF_DEV void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
DSUF_DEV void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- mbarrier ----
DSUF_DEV void mbar_init(uint64_t* b, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count) : "memory");
}
DSUF_DEV void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
DSUF_DEV void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
DSUF_DEV void mbar_arrive(uint64_t* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
DSUF_DEV bool mbar_try_wait(uint64_t* b, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(smem_u32(b)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (after recording the site) when the phase did not complete within the budget.
// Callers carry on with finite loops so the kernel still terminates.
DSUF_DEV bool mbar_wait(uint64_t* b, uint32_t parity, DevStatus* st, int kernel, int where) {
    if (mbar_try_wait(b, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(b, parity)) return true;
        if (clock64() - t0 > WAIT_BUDGET_TICKS) {
            report(st, DEVERR_WAIT_TIMEOUT, kernel, where);
            return false;
        }
    }
}

// ---- bulk / tensor copies (global -> this CTA's shared memory, completion on an mbarrier) ----
DSUF_DEV uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
DSUF_DEV uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// src and dst 16-byte aligned, bytes a multiple of 16.
DSUF_DEV void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Innermost coordinate times element size must be a multiple of 16 bytes (callers only pass multiples of 128).
DSUF_DEV void tma_2d(void* dst, const void* tmap, int c0, int c1, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(c0), "r"(c1), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
DSUF_DEV void tma_3d(void* dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(
            smem_u32(dst)),
        "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
DSUF_DEV void prefetch_tmap(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

DSUF_DEV bool elect_one() {
    uint32_t pred;
    asm volatile("{ .reg .pred e; elect.sync _|e, 0xffffffff; selp.u32 %0, 1, 0, e; }" : "=r"(pred));
    return pred != 0;
}
DSUF_DEV void named_bar_sync(int id, int nthreads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory"); }

// ---- codecs ----
DSUF_DEV float e8m0_to_f32(uint32_t b) { return __uint_as_float((b & 0xffu) << 23); }

// 2^ceil(log2(amax * qmax_inv)) through the exponent bits (crates/model/src/formats.rs:86-90).
DSUF_DEV float round_scale_pow2(float amax, float qmax_inv) {
    const uint32_t bits = __float_as_uint(amax * qmax_inv);
    const int e = (int)((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) != 0 ? 1 : 0);
    return __uint_as_float((uint32_t)(e + 127) << 23);
}
// Two fp32 -> packed e4m3x2, round-to-nearest-even, saturating at 448, NaN -> 0x7f; `lo` lands in the low byte.
DSUF_DEV uint16_t f32x2_to_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}
DSUF_DEV uint32_t f32x4_to_e4m3x4(float a, float b, float c, float d) {
    return (uint32_t)f32x2_to_e4m3x2(a, b) | ((uint32_t)f32x2_to_e4m3x2(c, d) << 16);
}
// Eight packed e2m1 nibbles -> two words of e4m3 bytes holding value * 2^-6 exactly: the 3 magnitude bits of a
// nibble dropped into e4m3's low exponent bits and top mantissa bit decode (subnormals included) to e2m1 / 64.
// `even` receives elements 0,2,4,6 (low nibbles), `odd` elements 1,3,5,7.
DSUF_DEV void e2m1x8_to_e4m3(uint32_t w, uint32_t& even, uint32_t& odd) {
    even = ((w << 4) & 0x80808080u) | ((w << 2) & 0x1c1c1c1cu);
    odd = (w & 0x80808080u) | ((w >> 2) & 0x1c1c1c1cu);
}
constexpr float E2M1_UNSCALE = 64.0f;

// D(16x8,f32) += A(16x32,e4m3,row) * B(32x8,e4m3,col)
DSUF_DEV void mma_e4m3(float* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

DSUF_DEV float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

// Row permutation inside an 8-row group that makes 8-byte shared loads from 128-byte swizzled rows conflict free:
// fragment row g reads tile row ROWMAP(g).
DSUF_DEV int rowmap8(int g) { return ((g & 3) << 1) | (g >> 2); }

}  // namespace dsuf
