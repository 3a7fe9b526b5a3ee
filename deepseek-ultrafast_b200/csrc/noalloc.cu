// dsuf_gemm_fp8_static: the decode FP8 GEMV for callers that cannot allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the GEMV: an engine whose whole
// device budget was carved into one arena at start-up (the reference does exactly that, crates/engine/src/weights.rs:16-57,
// and has nothing left to hand out), a plugin loaded into a process whose allocator is owned by someone else, or code that
// runs where an allocation would synchronise the device.  dsuf_gemm_fp8 asks them for a workspace; this variant brings its
// own: the stream-K partial sums and arrival counters live in a fixed array in the library's device image.
//
// Consequences, all documented in include/dsuf_qmm.h:
//   * the array exists once per GPU that loads the library (about 10 MB, until the process exits);
//   * its size is fixed: weights with more than NOALLOC_MAX_ROW_TILES row tiles, or GPUs with more than
//     NOALLOC_MAX_CTAS SMs, are rejected with an error instead of overrunning it;
//   * every call uses the same array, so two calls that overlap on the GPU (different streams) race; calls must be
//     stream-ordered.  The arrival counters must start at zero: they are cleared on the stream before every launch,
//     whatever the previous call left behind.  The partial sums are fully rewritten before they are read.
//   * the first call on a device looks the array's address up (cudaGetSymbolAddress) and remembers it; make that
//     first call before any stream capture begins.  With lazy module loading (the CUDA default) that look-up is also
//     the moment the driver places this file's device image, array included, in device memory: a caller that is about
//     to hand all remaining device memory to its own arena makes one small call first.
#include <mutex>

#include "internal.h"

namespace {

constexpr int NOALLOC_MAX_CTAS = 160;         // one partial slot pair per CTA of the persistent grid
constexpr int NOALLOC_MAX_ROW_TILES = 1024;   // weights up to 131072 rows
constexpr size_t NOALLOC_PARTIAL_BYTES = (size_t)NOALLOC_MAX_CTAS * 2 * 64 * 128 * sizeof(float);
constexpr size_t NOALLOC_BYTES = NOALLOC_PARTIAL_BYTES + NOALLOC_MAX_ROW_TILES * sizeof(int);

// In host code this name is only a handle for the runtime, not a device address: it is never passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[NOALLOC_BYTES];

constexpr int MAX_DEVICES = 64;
std::mutex g_mu;
void* g_scratch_addr[MAX_DEVICES];  // device address of g_static_scratch on each device, looked up once

int scratch_for_current_device(dsuf_ctx* ctx, void** out) {
    const int dev = ctx->device;
    if (dev < 0 || dev >= MAX_DEVICES) return dsuf::fail(ctx, DSUF_E_BADARG, "gemm_fp8_static: device index %d out of range", dev);
    // every call: the launch below goes to the current device, and the address only means something there
    int cur = -1;
    cudaError_t e = cudaGetDevice(&cur);
    if (e != cudaSuccess) return dsuf::cuda_fail(ctx, e, "cudaGetDevice");
    if (cur != dev) return dsuf::fail(ctx, DSUF_E_BADARG, "gemm_fp8_static: device %d must be current (current is %d)", dev, cur);
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_scratch_addr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return dsuf::cuda_fail(ctx, e, "cudaGetSymbolAddress(static scratch)");
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return DSUF_OK;
}

}  // namespace

extern "C" int32_t dsuf_gemm_fp8_static(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m,
                                        uint64_t out, int32_t ldo, float alpha) {
    if (!ctx || !w) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, (xq & 15) == 0, "gemm_fp8_static: xq must be 16-byte aligned");
    DSUF_REQUIRE(ctx, w->rt <= NOALLOC_MAX_ROW_TILES,
                 "gemm_fp8_static: weight has %d row tiles, the built-in scratch holds %d (n <= %d); use dsuf_gemm_fp8 with a workspace",
                 w->rt, NOALLOC_MAX_ROW_TILES, NOALLOC_MAX_ROW_TILES * 128);
    DSUF_REQUIRE(ctx, ctx->sm_count <= NOALLOC_MAX_CTAS,
                 "gemm_fp8_static: %d SMs exceed the built-in scratch (%d CTAs); use dsuf_gemm_fp8 with a workspace", ctx->sm_count,
                 NOALLOC_MAX_CTAS);
    void* base = nullptr;
    int rc = scratch_for_current_device(ctx, &base);
    if (rc) return rc;
    int* counters = (int*)((unsigned char*)base + NOALLOC_PARTIAL_BYTES);
    // the array keeps whatever the last call left: the arrival counters have to start from zero
    cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)w->rt * sizeof(int), (cudaStream_t)stream);
    if (e != cudaSuccess) return dsuf::cuda_fail(ctx, e, "cudaMemsetAsync(static counters)");
    return dsuf::launch_stream_dense(ctx, (cudaStream_t)stream, w, (const void*)xq, (const void*)xs, m, (void*)out, ldo, alpha, base,
                                     counters);
}
