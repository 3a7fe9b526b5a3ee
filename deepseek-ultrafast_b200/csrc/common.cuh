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
// 4-byte asynchronous copy (LDGSTS) and its completion hook: the mbarrier receives one arrival from this thread
// once all of the thread's earlier cp.async copies have landed (the arrival must be part of the barrier's count).
DSUF_DEV void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
DSUF_DEV void cp_async_arrive_noinc(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
DSUF_DEV void bulk_g2s_nh(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)), "l"(src),
                 "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
DSUF_DEV void tma_2d_nh(void* dst, const void* tmap, int c0, int c1, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(dst)),
                 "l"(tmap), "r"(c0), "r"(c1), "r"(smem_u32(bar))
                 : "memory");
}
DSUF_DEV void tma_3d_nh(void* dst, const void* tmap, int c0, int c1, int c2, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
                 "l"(tmap), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
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
// Warp-uniform broadcasts: tcgen05 / TMA instructions take their descriptors from uniform registers; values the
// compiler cannot prove uniform cost a register-file round trip per operand on every issue.
DSUF_DEV uint32_t uni32(uint32_t v) { return __shfl_sync(0xffffffffu, v, 0); }
DSUF_DEV uint64_t uni64(uint64_t v) { return ((uint64_t)uni32((uint32_t)(v >> 32)) << 32) | uni32((uint32_t)v); }
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


// ---- tcgen05 (5th-generation tensor cores: operands in shared memory, accumulators in tensor memory) ----
DSUF_DEV void tmem_alloc(uint32_t* slot_in_smem, uint32_t ncols) {   // whole warp; ncols a power of two >= 32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot_in_smem)), "r"(ncols) : "memory");
}
DSUF_DEV void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
DSUF_DEV void tmem_dealloc(uint32_t taddr, uint32_t ncols) {          // whole warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
DSUF_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
DSUF_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
DSUF_DEV void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// The mbarrier receives one arrival when every tcgen05 operation issued so far by this thread has completed.
DSUF_DEV void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 512-byte scale-factor atom (32 rows x 16 bytes) from shared memory to 4 tensor-memory columns, all 4 lane quarters.
DSUF_DEV void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem] with UE8M0 block scales from tensor memory; one K=32 step of 8-bit containers.
DSUF_DEV void tc_mma_mx(uint32_t d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p; }" ::"r"(d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
        : "memory");
}
// Shared-memory matrix descriptor: start address, leading / stride byte offsets (16-byte units), descriptor
// version 1 (bit 46), layout type (2 = 128-byte swizzle, 0 = none).
DSUF_DEV uint64_t tc_smem_desc(const void* p, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    uint64_t d = (uint64_t)((smem_u32(p) & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(layout & 7) << 61;
    return d;
}
// Instruction descriptor of kind::mxf8f6f4 with M = 128: N>>3 at bit 17, UE8M0 scale type (bit 23), M>>4 at bit 24,
// A format at bits 7-9 (0 = e4m3, 5 = e2m1), B format e4m3; scale-factor byte selectors (bits 4-5 for B, 29-30 for A)
// are OR-ed in per K step.
DSUF_DEV uint32_t tc_idesc_mx(int n, bool a_is_e2m1) {
    return ((uint32_t)(n >> 3) << 17) | (1u << 23) | ((128u >> 4) << 24) | (a_is_e2m1 ? (5u << 7) : 0u);
}
DSUF_DEV uint32_t tc_idesc_sf(uint32_t idesc, uint32_t kc) { return idesc | (kc << 29) | (kc << 4); }

// Accumulator read-back: this warp's 32 lanes x NCOL consecutive fp32 columns.
template <int NCOL>
DSUF_DEV void tmem_ld(uint32_t taddr, float* v);
template <>
DSUF_DEV void tmem_ld<8>(uint32_t taddr, float* v) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}
template <>
DSUF_DEV void tmem_ld<16>(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
template <>
DSUF_DEV void tmem_ld<32>(uint32_t taddr, float* v) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

}  // namespace dsuf
