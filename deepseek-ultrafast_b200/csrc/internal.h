// Host-side internals of libdsuf_qmm: context, error plumbing, the kernel launch helper and the prototypes of
// the per-file launchers.  Nothing here is part of the exported C ABI (see include/dsuf_qmm.h).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "../../include/dsuf_qmm.h"
#include "common.cuh"

typedef __nv_bfloat16 bf16;

typedef CUresult (*dsuf_encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                         const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                         CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct dsuf_ctx {
    int device;
    int sm_count;
    int smem_optin;
    int use_pdl;                   // launch with programmatic stream serialization
    int use_tc;                    // decode shapes on the tcgen05 streaming kernel (1) or the mma.sync one (0)
    int use_pairs;                 // decode expert GEMMs: two tile records per ring stage where K allows (default on)
    int use_kslices;               // dense decode GEMV: cluster K-split where it pays (default on)
    int prenorm_approx;            // RMS pre-normalisation with the approximate rsqrt instruction, as the reference's kernels
    int clock_khz;                 // SM clock rate the wait budgets are converted with
    long long xchg_wait_ticks;     // clock64 budget of the peer-exchange kernels' waits (dsuf_ctx_set_wait_budget_us)
    dsuf::DevStatus* dev_status;   // device word written by a kernel whose bounded wait expired
    dsuf_encode_tiled_fn encode_tiled;
    // activation tensor maps already encoded, by (base, row bytes, rows, box rows): a layer calls with the same buffers
    // step after step, so the driver call is paid once per buffer, not once per launch (a context serves one host thread)
    struct XMapEntry { const void* base; int k_bytes; long long rows; int box_rows; CUtensorMap tm; };
    XMapEntry xmaps[32];
    unsigned xmap_next;
    char err[512];
};

struct dsuf_weight {
    dsuf_weight_desc d;
    CUtensorMap tm_stream;   // tile records as bytes for the streaming (decode) kernels
    CUtensorMap tm_tc;       // tile records for the tcgen05 kernels (FP4: 4-bit elements unpacked by TMA)
    int rt, kt;              // row tiles per matrix, K tiles per row
    int rec_bytes, codes_bytes;
    long long tiles_total;
};

namespace dsuf {

inline int fail(dsuf_ctx* ctx, int code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
    }
    return code;
}

inline int cuda_fail(dsuf_ctx* ctx, cudaError_t e, const char* what) {
    return fail(ctx, (int)e > 0 ? (int)e : DSUF_E_BADARG, "%s: %s", what, cudaGetErrorString(e));
}

#define DSUF_REQUIRE(ctx, cond, ...) \
    do { if (!(cond)) return ::dsuf::fail(ctx, DSUF_E_BADARG, __VA_ARGS__); } while (0)

// One launch path for every kernel: asynchronous on the caller's stream, optional PDL attribute, no
// allocation and no synchronisation (safe inside stream capture).
// `cluster_x` > 1 launches thread-block clusters of that many CTAs along x (the grid must be a multiple of it).
template <typename... KArgs, typename... Args>
int launch_cluster(dsuf_ctx* ctx, cudaStream_t stream, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int cluster_x,
                   Args&&... args) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    memset(attr, 0, sizeof(attr));
    unsigned n = 0;
    if (ctx->use_pdl) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "kernel launch");
    return DSUF_OK;
}

template <typename... KArgs, typename... Args>
int launch(dsuf_ctx* ctx, cudaStream_t stream, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    return launch_cluster(ctx, stream, kernel, grid, block, smem, 1, std::forward<Args>(args)...);
}

// per-file launchers
int launch_act_quant(dsuf_ctx* ctx, cudaStream_t stream, int mode, const void* x, int ldx, int rows_in, int k, void* q,
                     void* scales, const int* pair_row, int fanout, const void* norm_w = nullptr,
                     const float* sumsq = nullptr, float eps = 0.f);
int launch_row_sumsq(dsuf_ctx* ctx, cudaStream_t stream, const void* x, int ldx, int m, int k, float* out);
int launch_stream_dense(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_weight* w, const void* xq, const void* xs, int m,
                        void* out, int ldo, float alpha, void* workspace, int* counters_at = nullptr, const dsuf_gemm_opts* opts = nullptr);
int launch_stream_moe(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_weight* w, int epi, int act_mode, const dsuf_moe_plan* plan,
                      const void* xq, const void* xs, float swiglu_limit, void* out, int ldo);
int launch_route(dsuf_ctx* ctx, cudaStream_t stream, int score_fn, const float* scores, const float* bias, int t, int n_exp,
                 int topk, float route_scale, int* ids, float* w);
int launch_front(dsuf_ctx* ctx, cudaStream_t stream, int score_fn, const float* scores, const float* bias, int t, int n_exp_all,
                 int topk, float route_scale, int* ids, float* w, int e_lo, const dsuf_moe_plan* plan, int mode, const void* x, int ldx,
                 int h, void* xq, void* xs);
int launch_plan(dsuf_ctx* ctx, cudaStream_t stream, const int* ids, const float* w, int e_lo, const dsuf_moe_plan* plan);
int launch_unpermute(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_moe_plan* plan, const float* yrows, const void* shared,
                     int t, int topk, int h, void* out, int ldo);
int launch_unpermute_quant(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_moe_plan* plan, const float* yrows, const void* shared,
                           int t, int topk, int h, void* out, int ldo, int mode, void* q_out, void* s_out);
int stream_setup(dsuf_ctx* ctx);
int lm_head_setup(dsuf_ctx* ctx);
int encode_x_map(dsuf_ctx* ctx, CUtensorMap* tm, const void* base, int k_bytes, long long rows, int box_rows);

}  // namespace dsuf
