// dsuf_probe_tensor_rate: what the tensor cores of this GPU deliver to the instruction the GEMMs of this library
// use (tcgen05.mma kind::mxf8f6f4.block_scale, M = 128, K = 32 of 8-bit containers) when nothing else limits it:
// operands already in shared memory, scales already in tensor memory, one CTA per SM issuing back to back into two
// alternating accumulators.  The benchmark divides a GEMM kernel's FLOP/s by this figure (next to the vendor's nominal
// peak), because no measured FP8 / FP4 tensor peak exists for the box otherwise.  A measurement aid without a
// counterpart in the reference.
#include "internal.h"

namespace dsuf {

constexpr int KID_PROBE = 6;
constexpr int PROBE_SMEM = 16384 + 32768 + 512 + 1024;  // A tile, B tile (up to 256 rows), one scale atom, alignment slack

__global__ void __launch_bounds__(128, 1) tensor_rate_kernel(int n_cols, int a_is_e2m1, int iters, DevStatus* status) {
    extern __shared__ uint8_t probe_smem[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t s_tmem;
    uint8_t* base = probe_smem + ((1024u - (smem_u32(probe_smem) & 1023u)) & 1023u);
    const int warp = threadIdx.x >> 5;
    // e4m3 1.0 in every operand byte (an e2m1 container decodes it as a small number: the values do not matter);
    // scale bytes of 2^-71, all finite
    for (int i = threadIdx.x; i < (16384 + 32768 + 512) / 4; i += blockDim.x) ((uint32_t*)base)[i] = 0x38383838u;
    if (warp == 0) {
        tmem_alloc(&s_tmem, 512);
        tmem_relinquish();
    }
    if (threadIdx.x == 0) {
        mbar_init(&done_bar, 1);
        mbar_fence_init();
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tm = s_tmem;
    if (warp == 1) {
        const uint32_t tmu = warp_uniform(tm);
        const uint64_t ad = warp_uniform(tc_smem_desc(base, 16, 1024, TC_SWIZZLE_128B));
        const uint64_t bd = warp_uniform(tc_smem_desc(base + 16384, 16, 1024, TC_SWIZZLE_128B));
        const uint64_t sfd = warp_uniform(tc_smem_desc(base + 16384 + 32768, 512, 128, TC_SWIZZLE_NONE));
        const uint32_t idesc = tc_idesc_mx(n_cols, a_is_e2m1 != 0);
        if (warp_elect()) {
            // scale columns 480..487; accumulators below them: two that alternate where both fit, else one
            tc_cp_sf(tmu + 480, sfd);
            tc_cp_sf(tmu + 484, sfd);
            const uint32_t second = 2 * n_cols <= 448 ? (uint32_t)n_cols : 0u;
            for (int i = 0; i < iters; ++i)
                tc_mma_mx(tmu + (i & 1) * second, ad + (uint64_t)((i & 3) * 2), bd + (uint64_t)((i & 3) * 2), tc_idesc_sf(idesc, i & 3),
                          tmu + 480, tmu + 484, 1u);
            tc_commit(&done_bar);
        }
        __syncwarp();
        mbar_wait(&done_bar, 0, status, KID_PROBE, 1);   // bounded: gives up and reports after the library's wait budget
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 0) tmem_dealloc(tm, 512);
}

}  // namespace dsuf

using namespace dsuf;

extern "C" int32_t dsuf_probe_tensor_rate(dsuf_ctx* ctx, void* stream, int32_t n_cols, int32_t a_is_e2m1, int32_t iters,
                                          double* flop_per_launch) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, n_cols >= 16 && n_cols <= 256 && n_cols % 16 == 0, "probe: n_cols must be a multiple of 16 in 16..256, got %d", n_cols);
    DSUF_REQUIRE(ctx, iters >= 1 && iters <= (1 << 22), "probe: iters out of range");
    cudaError_t e = cudaFuncSetAttribute(tensor_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PROBE_SMEM);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(probe)");
    if (flop_per_launch) *flop_per_launch = 2.0 * 128.0 * n_cols * 32.0 * iters * ctx->sm_count;
    return launch(ctx, (cudaStream_t)stream, tensor_rate_kernel, dim3(ctx->sm_count), dim3(128), (size_t)PROBE_SMEM, (int)n_cols,
                  (int)a_is_e2m1, (int)iters, ctx->dev_status);
}
