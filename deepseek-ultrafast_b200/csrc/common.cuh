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
enum { DEVERR_NONE = 0, DEVERR_WAIT_TIMEOUT = 1, DEVERR_BAD_PLAN = 2, DEVERR_EPOCH_DRIFT = 3 };

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

// ---- warp-level helpers ----
// True in exactly one lane of a converged warp (the hardware picks it); the others skip the guarded statement.
DSUF_DEV bool warp_elect() {
    uint32_t chosen = 0;
    asm volatile(
        "{\n"
        "  .reg .pred is_leader;\n"
        "  elect.sync _|is_leader, %1;\n"
        "  @is_leader mov.u32 %0, 1;\n"
        "}\n"
        : "+r"(chosen)
        : "r"(0xffffffffu));
    return chosen != 0;
}
// Lane 0's value in every lane.  tcgen05 / TMA instructions read descriptors and addresses from uniform registers;
// handing the compiler a value it can prove warp-uniform saves a register-file round trip per operand per issue.
template <typename T>
DSUF_DEV T warp_uniform(T v) {
    static_assert(sizeof(T) == 4 || sizeof(T) == 8, "32- or 64-bit values");
    if constexpr (sizeof(T) == 4) {
        return (T)__shfl_sync(0xffffffffu, (uint32_t)v, 0);
    } else {
        const uint32_t lo = __shfl_sync(0xffffffffu, (uint32_t)((uint64_t)v & 0xffffffffu), 0);
        const uint32_t hi = __shfl_sync(0xffffffffu, (uint32_t)((uint64_t)v >> 32), 0);
        return (T)(((uint64_t)hi << 32) | lo);
    }
}
// ---- thread-block clusters ----
DSUF_DEV uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
DSUF_DEV uint32_t cluster_num_ctas() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
    return r;
}
// Hardware barrier over every thread of every CTA of the cluster; shared-memory writes made before it are visible to
// the other CTAs' distributed-shared-memory reads after it.  Whole warps must call it together.
DSUF_DEV void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;" : : : "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" : : : "memory");
}
// One fp32 from the same shared-memory location of CTA `rank` of this cluster.
DSUF_DEV float ld_cluster_f32(const float* my_smem_ptr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
DSUF_DEV uint32_t ld_cluster_u32(const void* my_smem_ptr, uint32_t rank) {
    uint32_t remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(my_smem_ptr)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
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

// Packed fp32 arithmetic (two lanes per instruction, each rounded like the scalar fma.rn / mul.rn): halves the
// instruction count of the per-tile fp32 promotion.  The 64-bit operands are register pairs; the packing moves cost
// nothing when the allocator keeps the halves adjacent (accumulators and tensor-memory read-backs come in such pairs).
DSUF_DEV unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
DSUF_DEV void fma_f32x2(float& d0, float& d1, float a0, float a1, float b0, float b1) {
    unsigned long long d = pack_f32x2(d0, d1);
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(pack_f32x2(a0, a1)), "l"(pack_f32x2(b0, b1)));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
DSUF_DEV void mul_f32x2(float& d0, float& d1, float b0, float b1) {
    unsigned long long d = pack_f32x2(d0, d1);
    asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(d) : "l"(pack_f32x2(b0, b1)));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d0), "=f"(d1) : "l"(d));
}
DSUF_DEV float bf16_round(float v) { return __bfloat162float(__float2bfloat16(v)); }

// Row permutation inside an 8-row group that makes 8-byte shared loads from 128-byte swizzled rows conflict free:
// fragment row g reads tile row ROWMAP(g).
DSUF_DEV int rowmap8(int g) { return ((g & 3) << 1) | (g >> 2); }


// ---- tcgen05: operands in shared memory, accumulators and block scales in tensor memory ----
// Every wrapper is the single-CTA form (cta_group::1).  Tensor-memory addresses are (lane << 16) | column.

// Allocation: a whole warp asks for `ncols` columns (a power of two, at least 32); the base address is written to
// `result_in_smem`.  The same warp must give the columns back before the CTA exits.
DSUF_DEV void tmem_alloc(uint32_t* result_in_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" : : "r"(smem_u32(result_in_smem)), "r"(ncols) : "memory");
}
DSUF_DEV void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" : : : "memory"); }
DSUF_DEV void tmem_dealloc(uint32_t base, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" : : "r"(base), "r"(ncols) : "memory");
}

// Ordering of tensor-core work against barriers / thread synchronisation, and of generic-proxy shared-memory writes
// against the asynchronous proxy (TMA, tcgen05 operand reads).
DSUF_DEV void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" : : : "memory"); }
DSUF_DEV void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" : : : "memory"); }
DSUF_DEV void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" : : : "memory"); }

// One arrival on `bar` once all tcgen05 operations this thread has issued so far are complete.
DSUF_DEV void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" : : "r"(smem_u32(bar)) : "memory");
}

// Shared-memory operand descriptor.  Fields, low to high: start address, leading-dimension byte offset, stride byte
// offset (each in 16-byte units, 14 bits), the constant 0b001 at bit 46 that sm_100 descriptors carry, and the swizzle
// mode in the top three bits.
enum : uint32_t { TC_SWIZZLE_NONE = 0, TC_SWIZZLE_128B = 2 };
DSUF_DEV uint64_t tc_smem_desc(const void* smem_ptr, uint32_t leading_bytes, uint32_t stride_bytes, uint32_t swizzle) {
    auto units16 = [](uint32_t bytes) -> uint64_t { return (uint64_t)((bytes >> 4) & 0x3fffu); };
    return units16(smem_u32(smem_ptr)) | (units16(leading_bytes) << 16) | (units16(stride_bytes) << 32) | (1ull << 46) |
           ((uint64_t)(swizzle & 7u) << 61);
}

// Instruction descriptor of kind::mxf8f6f4 with block scaling, M = 128 rows of A, `n` columns of B (a multiple of 8).
// Bit positions: A element type at 7 (0 = e4m3, 5 = e2m1), B element type at 10 (e4m3 = 0), N / 8 at 17, the scale type
// at 23 (1 = UE8M0), M / 16 at 24.  The byte of each 4-byte scale word that a K = 32 step uses is chosen per step by
// tc_idesc_sf (B's selector at bit 4, A's at bit 29).
struct TcIdesc {
    static constexpr uint32_t A_TYPE_SHIFT = 7, N_SHIFT = 17, SCALE_UE8M0 = 1u << 23, M_SHIFT = 24, SFB_SEL_SHIFT = 4, SFA_SEL_SHIFT = 29;
    static constexpr uint32_t TYPE_E2M1 = 5;
};
DSUF_DEV uint32_t tc_idesc_mx(int n, bool a_is_e2m1) {
    uint32_t d = TcIdesc::SCALE_UE8M0 | ((uint32_t)(128 / 16) << TcIdesc::M_SHIFT) | ((uint32_t)(n / 8) << TcIdesc::N_SHIFT);
    if (a_is_e2m1) d |= TcIdesc::TYPE_E2M1 << TcIdesc::A_TYPE_SHIFT;
    return d;
}
DSUF_DEV uint32_t tc_idesc_sf(uint32_t idesc, uint32_t k_step) {
    return idesc | (k_step << TcIdesc::SFA_SEL_SHIFT) | (k_step << TcIdesc::SFB_SEL_SHIFT);
}

// Copies one 512-byte scale atom (32 rows x 16 bytes in shared memory) into 4 tensor-memory columns, replicated to the
// four 32-lane quarters.
DSUF_DEV void tc_cp_sf(uint32_t tmem_cols, uint64_t atom_desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" : : "r"(tmem_cols), "l"(atom_desc) : "memory");
}

// One K = 32 step on 8-bit containers: D[tmem] = (accumulate ? D : 0) + (A * scale_a) (B * scale_b), scales read from
// tensor memory.  Issued by a single thread.
DSUF_DEV void tc_mma_mx(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                        uint32_t accumulate) {
    asm volatile(
        "{\n"
        "  .reg .pred keep_d;\n"
        "  setp.ne.u32 keep_d, %6, 0;\n"
        "  tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%4], [%5], keep_d;\n"
        "}\n"
        :
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(sfa_tmem), "r"(sfb_tmem), "r"(accumulate)
        : "memory");
}

// Accumulator read-back.  A warp reads its own 32 lanes (lane quarter = warp index % 4) x NCOL consecutive fp32
// columns; thread i of the warp receives lane i's values.  The destination registers are written as floats directly
// (the instruction moves untyped 32-bit words).
#define DSUF_TM_F4(v, i) "=f"(v[i]), "=f"(v[(i) + 1]), "=f"(v[(i) + 2]), "=f"(v[(i) + 3])
#define DSUF_TM_F8(v, i) DSUF_TM_F4(v, i), DSUF_TM_F4(v, (i) + 4)
#define DSUF_TM_F16(v, i) DSUF_TM_F8(v, i), DSUF_TM_F8(v, (i) + 8)
DSUF_DEV void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" : : : "memory"); }
template <int NCOL>
DSUF_DEV void tmem_ld_issue(uint32_t taddr, float* v) {
    static_assert(NCOL == 8 || NCOL == 16 || NCOL == 32, "columns per load");
    if constexpr (NCOL == 8) {
        asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                     : DSUF_TM_F8(v, 0)
                     : "r"(taddr)
                     : "memory");
    } else if constexpr (NCOL == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
            : DSUF_TM_F16(v, 0)
            : "r"(taddr)
            : "memory");
    } else {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : DSUF_TM_F16(v, 0), DSUF_TM_F16(v, 16)
            : "r"(taddr)
            : "memory");
    }
}
// Load and wait for the data to be in registers.
template <int NCOL>
DSUF_DEV void tmem_ld(uint32_t taddr, float* v) {
    tmem_ld_issue<NCOL>(taddr, v);
    tmem_wait_ld();
}

}  // namespace dsuf
