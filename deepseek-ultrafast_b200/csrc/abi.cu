// The exported C ABI (include/dsuf_qmm.h): context, weight descriptors, argument validation, dispatch.
// Every hot entry validates its launch contract on the host and returns an error code (the reference does the
// same with ensure!, crates/engine/src/ops.rs:342-354); none allocates or synchronises.
#include "internal.h"
#include "stream_gemv.cuh"

namespace dsuf {
size_t stream_workspace_bytes();
}
using namespace dsuf;

extern "C" {

int32_t dsuf_ctx_create(int32_t device, dsuf_ctx** out) {
    if (!out) return DSUF_E_BADARG;
    *out = nullptr;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return (int32_t)e;
    dsuf_ctx* ctx = new dsuf_ctx();
    memset(ctx, 0, sizeof(*ctx));
    ctx->device = device;
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) { delete ctx; return (int32_t)e; }
    if (prop.major != 10) {
        // sm_100a kernels only: fail loudly instead of falling back to anything else
        delete ctx;
        return DSUF_E_UNSUPPORTED;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->smem_optin = (int)prop.sharedMemPerBlockOptin;
    ctx->clock_khz = prop.clockRate > 0 ? prop.clockRate : 1965000;
    ctx->xchg_wait_ticks = WAIT_BUDGET_TICKS;
    ctx->use_kslices = 1;
    ctx->use_pairs = 1;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
    if (e != cudaSuccess || !fn || qres != cudaDriverEntryPointSuccess) { delete ctx; return e != cudaSuccess ? (int32_t)e : DSUF_E_UNSUPPORTED; }
    ctx->encode_tiled = (dsuf_encode_tiled_fn)fn;
    e = cudaMalloc(&ctx->dev_status, sizeof(DevStatus));
    if (e != cudaSuccess) { delete ctx; return (int32_t)e; }
    cudaMemset(ctx->dev_status, 0, sizeof(DevStatus));
    int rc = stream_setup(ctx);
    if (!rc) rc = lm_head_setup(ctx);
    if (rc) { cudaFree(ctx->dev_status); delete ctx; return rc; }
    *out = ctx;
    return DSUF_OK;
}

int32_t dsuf_ctx_destroy(dsuf_ctx* ctx) {
    if (!ctx) return DSUF_OK;
    cudaFree(ctx->dev_status);
    delete ctx;
    return DSUF_OK;
}

int32_t dsuf_last_error(dsuf_ctx* ctx, char* buf, size_t len) {
    if (!ctx || !buf || !len) return DSUF_E_BADARG;
    strncpy(buf, ctx->err, len - 1);
    buf[len - 1] = 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_pdl(dsuf_ctx* ctx, int32_t enabled) {
    if (!ctx) return DSUF_E_BADARG;
    ctx->use_pdl = enabled ? 1 : 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_decode_path(dsuf_ctx* ctx, int32_t tcgen05) {
    if (!ctx) return DSUF_E_BADARG;
    ctx->use_tc = tcgen05 ? 1 : 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_stage_pairs(dsuf_ctx* ctx, int32_t enabled) {
    if (!ctx) return DSUF_E_BADARG;
    ctx->use_pairs = enabled ? 1 : 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_dense_ksplit(dsuf_ctx* ctx, int32_t enabled) {
    if (!ctx) return DSUF_E_BADARG;
    ctx->use_kslices = enabled ? 1 : 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_prenorm_rsqrt(dsuf_ctx* ctx, int32_t approximate) {
    if (!ctx) return DSUF_E_BADARG;
    ctx->prenorm_approx = approximate ? 1 : 0;
    return DSUF_OK;
}

int32_t dsuf_ctx_set_wait_budget_us(dsuf_ctx* ctx, int64_t microseconds) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, microseconds >= 1 && microseconds <= 10000000, "wait budget must be 1 us .. 10 s, got %lld", (long long)microseconds);
    ctx->xchg_wait_ticks = (long long)microseconds * ctx->clock_khz / 1000;
    return DSUF_OK;
}

int32_t dsuf_sm_count(dsuf_ctx* ctx) { return ctx ? ctx->sm_count : 0; }

int32_t dsuf_status_poll(dsuf_ctx* ctx, void* stream, dsuf_dev_status* out) {
    if (!ctx || !out) return DSUF_E_BADARG;
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaStreamSynchronize");
    DevStatus h;
    e = cudaMemcpy(&h, ctx->dev_status, sizeof(h), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "status read");
    out->code = h.code; out->kernel = h.kernel; out->cta = h.cta; out->where = h.where;
    if (h.code) {
        cudaMemset(ctx->dev_status, 0, sizeof(DevStatus));
        return fail(ctx, DSUF_E_TIMEOUT, "device status %d from kernel %d cta %d site %d", h.code, h.kernel, h.cta, h.where);
    }
    return DSUF_OK;
}

int32_t dsuf_weight_create(dsuf_ctx* ctx, const dsuf_weight_desc* d, dsuf_weight** out) {
    if (!ctx || !d || !out) return DSUF_E_BADARG;
    *out = nullptr;
    DSUF_REQUIRE(ctx, d->fmt == DSUF_FMT_FP8 || d->fmt == DSUF_FMT_FP4, "weight: unknown fmt %d", d->fmt);
    DSUF_REQUIRE(ctx, d->n > 0 && d->k > 0 && d->k % 128 == 0, "weight: k (%d) must be a positive multiple of 128", d->k);
    DSUF_REQUIRE(ctx, d->n_experts >= 1, "weight: n_experts must be >= 1");
    DSUF_REQUIRE(ctx, d->tiles && (d->tiles & 15) == 0, "weight: tiles pointer must be 16-byte aligned");
    DSUF_REQUIRE(ctx, !(d->fmt == DSUF_FMT_FP8 && d->mode == DSUF_MODE_DS) || d->scales_ds, "weight: FP8 DS needs scales_ds");
    dsuf_weight* w = new dsuf_weight();
    memset(w, 0, sizeof(*w));
    w->d = *d;
    w->rt = (d->n + 127) / 128;
    w->kt = d->k / 128;
    w->codes_bytes = d->fmt == DSUF_FMT_FP4 ? 8192 : 16384;
    w->rec_bytes = w->codes_bytes + ((d->fmt == DSUF_FMT_FP4 || d->mode == DSUF_MODE_MX) ? 512 : 0);
    w->tiles_total = (long long)d->n_experts * w->rt * w->kt;
    if (w->tiles_total >= (1ll << 31)) { delete w; return fail(ctx, DSUF_E_BADARG, "weight: too many tiles"); }
    const cuuint32_t row_bytes = d->fmt == DSUF_FMT_FP4 ? 64u : 128u;
    cuuint64_t dims[3] = {row_bytes, 128, (cuuint64_t)w->tiles_total};
    cuuint64_t strides[2] = {row_bytes, (cuuint64_t)w->rec_bytes};
    cuuint32_t box[3] = {row_bytes, 128, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = ctx->encode_tiled(&w->tm_stream, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)d->tiles, dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                                   d->fmt == DSUF_FMT_FP4 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { delete w; return fail(ctx, DSUF_E_BADARG, "cuTensorMapEncodeTiled(weight stream) failed: %d", (int)r); }
    if (d->fmt == DSUF_FMT_FP4) {
        // same bytes seen as 4-bit elements: TMA widens every 16 packed codes (8 bytes) to 16 bytes of shared memory
        cuuint64_t edims[3] = {128, 128, (cuuint64_t)w->tiles_total};
        cuuint32_t ebox[3] = {128, 128, 1};
        r = ctx->encode_tiled(&w->tm_tc, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, (void*)d->tiles, edims, strides, ebox, es,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { delete w; return fail(ctx, DSUF_E_BADARG, "cuTensorMapEncodeTiled(weight fp4 unpack) failed: %d", (int)r); }
    } else {
        w->tm_tc = w->tm_stream;
    }
    *out = w;
    return DSUF_OK;
}

int32_t dsuf_weight_destroy(dsuf_weight* w) {
    delete w;
    return DSUF_OK;
}

int32_t dsuf_act_quant_fp8(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t m, int32_t k,
                           uint64_t q_out, uint64_t scale_out) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "act_quant: unknown mode %d", mode);
    DSUF_REQUIRE(ctx, m >= 0 && k > 0 && k % 128 == 0, "act_quant: k (%d) must be a positive multiple of 128", k);
    DSUF_REQUIRE(ctx, ldx >= k && ldx % 8 == 0, "act_quant: ldx (%d) must be >= k and a multiple of 8", ldx);
    if (m == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, x && q_out && scale_out, "act_quant: null pointer");
    DSUF_REQUIRE(ctx, (x & 15) == 0 && (q_out & 7) == 0, "act_quant: x must be 16-byte and q_out 8-byte aligned");
    return launch_act_quant(ctx, (cudaStream_t)stream, mode, (const void*)x, ldx, m, k, (void*)q_out, (void*)scale_out, nullptr, 0);
}

int32_t dsuf_row_sumsq(dsuf_ctx* ctx, void* stream, uint64_t x, int32_t ldx, int32_t m, int32_t k, uint64_t sumsq_out) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, m >= 0 && k > 0 && k % 8 == 0, "row_sumsq: k (%d) must be a positive multiple of 8", k);
    DSUF_REQUIRE(ctx, ldx >= k && ldx % 8 == 0, "row_sumsq: ldx (%d) must be >= k and a multiple of 8", ldx);
    if (m == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, x && sumsq_out && (x & 15) == 0, "row_sumsq: null or misaligned pointer");
    return launch_row_sumsq(ctx, (cudaStream_t)stream, (const void*)x, ldx, m, k, (float*)sumsq_out);
}

int32_t dsuf_act_quant_fp8_prenorm(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t m, int32_t k,
                                   uint64_t norm_w, uint64_t sumsq, float eps, uint64_t q_out, uint64_t scale_out) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "act_quant_prenorm: unknown mode %d", mode);
    DSUF_REQUIRE(ctx, m >= 0 && k > 0 && k % 128 == 0, "act_quant_prenorm: k (%d) must be a positive multiple of 128", k);
    DSUF_REQUIRE(ctx, ldx >= k && ldx % 8 == 0, "act_quant_prenorm: ldx (%d) must be >= k and a multiple of 8", ldx);
    if (m == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, x && q_out && scale_out && norm_w && sumsq, "act_quant_prenorm: null pointer");
    DSUF_REQUIRE(ctx, (x & 15) == 0 && (norm_w & 15) == 0 && (q_out & 7) == 0, "act_quant_prenorm: x and norm_w must be 16-byte, q_out 8-byte aligned");
    return launch_act_quant(ctx, (cudaStream_t)stream, mode, (const void*)x, ldx, m, k, (void*)q_out, (void*)scale_out, nullptr, 0,
                            (const void*)norm_w, (const float*)sumsq, eps);
}

size_t dsuf_gemm_workspace_bytes(dsuf_ctx*) { return stream_workspace_bytes(); }

int32_t dsuf_workspace_init(dsuf_ctx* ctx, void* stream, uint64_t workspace, size_t bytes) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, workspace && bytes >= stream_workspace_bytes(), "workspace_init: need %zu bytes", stream_workspace_bytes());
    cudaError_t e = cudaMemsetAsync((void*)workspace, 0, stream_workspace_bytes(), (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaMemsetAsync(workspace)");
    return DSUF_OK;
}

int32_t dsuf_gemm_fp8(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m, uint64_t out,
                      int32_t ldo, float alpha, uint64_t workspace) {
    if (!ctx || !w) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, (xq & 15) == 0, "dsuf_gemm_fp8: xq must be 16-byte aligned");
    return launch_stream_dense(ctx, (cudaStream_t)stream, w, (const void*)xq, (const void*)xs, m, (void*)out, ldo, alpha, (void*)workspace);
}

int32_t dsuf_gemm_fp8_ex(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m, uint64_t out,
                         int32_t ldo, const dsuf_gemm_opts* opts, uint64_t workspace) {
    if (!ctx || !w || !opts) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, (xq & 15) == 0, "dsuf_gemm_fp8_ex: xq must be 16-byte aligned");
    return launch_stream_dense(ctx, (cudaStream_t)stream, w, (const void*)xq, (const void*)xs, m, (void*)out, ldo, opts->alpha,
                               (void*)workspace, nullptr, opts);
}

int32_t dsuf_moe_route(dsuf_ctx* ctx, void* stream, int32_t score_fn, uint64_t scores, uint64_t bias, int32_t t,
                       int32_t n_exp, int32_t topk, float route_scale, uint64_t ids_out, uint64_t w_out) {
    if (!ctx) return DSUF_E_BADARG;
    DSUF_REQUIRE(ctx, n_exp >= 1 && n_exp <= 512, "moe_route: n_exp (%d) must be in 1..512", n_exp);
    DSUF_REQUIRE(ctx, topk >= 1 && topk <= 16 && topk <= n_exp, "moe_route: topk (%d) must be in 1..min(16, n_exp)", topk);
    DSUF_REQUIRE(ctx, score_fn >= 0 && score_fn <= 2, "moe_route: unknown score_fn %d", score_fn);
    DSUF_REQUIRE(ctx, t >= 0 && scores && ids_out && w_out, "moe_route: null pointer");
    return launch_route(ctx, (cudaStream_t)stream, score_fn, (const float*)scores, (const float*)bias, t, n_exp, topk, route_scale,
                        (int*)ids_out, (float*)w_out);
}

size_t dsuf_moe_plan_scratch_ints(int32_t p, int32_t n_exp) {
    const size_t nblk = ((size_t)(p > 0 ? p : 0) + 1023) / 1024;
    return (nblk + 1) * (size_t)n_exp + (size_t)(p > 0 ? p : 0) + 16;
}

static int check_plan(dsuf_ctx* ctx, const dsuf_moe_plan* p) {
    DSUF_REQUIRE(ctx, p, "plan: null");
    DSUF_REQUIRE(ctx, p->p >= 0 && p->n_exp >= 1 && p->n_exp <= 512, "plan: n_exp (%d) must be in 1..512", p->n_exp);
    DSUF_REQUIRE(ctx, p->tile_rows == 8 || p->tile_rows == 16 || p->tile_rows == 128, "plan: tile_rows must be 8, 16 or 128");
    DSUF_REQUIRE(ctx, p->max_tiles >= p->p / p->tile_rows + p->n_exp, "plan: max_tiles %d < p/tile_rows + n_exp", p->max_tiles);
    DSUF_REQUIRE(ctx, p->expert_off && p->row_pair && p->pair_row && p->row_w && p->tiles && p->ntiles && p->scratch, "plan: null buffer");
    DSUF_REQUIRE(ctx, (p->tiles & 15) == 0, "plan: tiles must be 16-byte aligned");
    return DSUF_OK;
}

int32_t dsuf_moe_permute_plan(dsuf_ctx* ctx, void* stream, uint64_t ids, uint64_t w, int32_t e_lo, const dsuf_moe_plan* plan) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, plan->p == 0 || (ids && w), "permute_plan: null pointer");
    return launch_plan(ctx, (cudaStream_t)stream, (const int*)ids, (const float*)w, e_lo, plan);
}

int32_t dsuf_moe_gather_quant(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t t, int32_t h,
                              int32_t topk, const dsuf_moe_plan* plan, uint64_t xq_out, uint64_t xs_out) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "gather_quant: unknown mode %d", mode);
    DSUF_REQUIRE(ctx, h > 0 && h % 128 == 0 && ldx >= h && ldx % 8 == 0, "gather_quant: h (%d) must be a multiple of 128, ldx a multiple of 8", h);
    DSUF_REQUIRE(ctx, topk >= 1 && (long long)t * topk == plan->p, "gather_quant: t*topk != plan.p");
    if (t == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, x && xq_out && xs_out && (x & 15) == 0 && (xq_out & 15) == 0, "gather_quant: null or misaligned pointer");
    return launch_act_quant(ctx, (cudaStream_t)stream, mode, (const void*)x, ldx, t, h, (void*)xq_out, (void*)xs_out,
                            (const int*)plan->pair_row, topk);
}

int32_t dsuf_moe_route_plan_gather(dsuf_ctx* ctx, void* stream, int32_t score_fn, uint64_t scores, uint64_t bias, int32_t t,
                                   int32_t n_exp_all, int32_t topk, float route_scale, uint64_t ids_out, uint64_t w_out, int32_t e_lo,
                                   const dsuf_moe_plan* plan, int32_t mode, uint64_t x, int32_t ldx, int32_t h, uint64_t xq_out,
                                   uint64_t xs_out) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, n_exp_all >= 1 && n_exp_all <= 512, "route_plan_gather: n_exp_all (%d) must be in 1..512", n_exp_all);
    DSUF_REQUIRE(ctx, topk >= 1 && topk <= 16 && topk <= n_exp_all, "route_plan_gather: topk (%d) must be in 1..min(16, n_exp_all)", topk);
    DSUF_REQUIRE(ctx, score_fn >= 0 && score_fn <= 2, "route_plan_gather: unknown score_fn %d", score_fn);
    DSUF_REQUIRE(ctx, t >= 0 && (long long)t * topk == plan->p, "route_plan_gather: t*topk != plan.p");
    DSUF_REQUIRE(ctx, plan->p <= 1024, "route_plan_gather: at most 1024 (token, expert) pairs per call, got %d: use the separate entries", plan->p);
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "route_plan_gather: unknown mode %d", mode);
    DSUF_REQUIRE(ctx, h > 0 && h % 128 == 0 && ldx >= h && ldx % 8 == 0, "route_plan_gather: h (%d) must be a multiple of 128, ldx a multiple of 8", h);
    if (t == 0) return launch_plan(ctx, (cudaStream_t)stream, nullptr, nullptr, e_lo, plan);
    DSUF_REQUIRE(ctx, scores && ids_out && w_out && x && xq_out && xs_out && (x & 15) == 0 && (xq_out & 15) == 0,
                 "route_plan_gather: null or misaligned pointer");
    return launch_front(ctx, (cudaStream_t)stream, score_fn, (const float*)scores, (const float*)bias, t, n_exp_all, topk, route_scale,
                        (int*)ids_out, (float*)w_out, e_lo, plan, mode, (const void*)x, ldx, h, (void*)xq_out, (void*)xs_out);
}

int32_t dsuf_moe_gather_quant_prenorm(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t t, int32_t h,
                                      int32_t topk, const dsuf_moe_plan* plan, uint64_t norm_w, uint64_t sumsq, float eps,
                                      uint64_t xq_out, uint64_t xs_out) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "gather_quant_prenorm: unknown mode %d", mode);
    DSUF_REQUIRE(ctx, h > 0 && h % 128 == 0 && ldx >= h && ldx % 8 == 0, "gather_quant_prenorm: h (%d) must be a multiple of 128, ldx a multiple of 8", h);
    DSUF_REQUIRE(ctx, topk >= 1 && (long long)t * topk == plan->p, "gather_quant_prenorm: t*topk != plan.p");
    if (t == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, x && xq_out && xs_out && norm_w && sumsq && (x & 15) == 0 && (xq_out & 15) == 0 && (norm_w & 15) == 0,
                 "gather_quant_prenorm: null or misaligned pointer");
    return launch_act_quant(ctx, (cudaStream_t)stream, mode, (const void*)x, ldx, t, h, (void*)xq_out, (void*)xs_out,
                            (const int*)plan->pair_row, topk, (const void*)norm_w, (const float*)sumsq, eps);
}

int32_t dsuf_moe_w13_swiglu(dsuf_ctx* ctx, void* stream, const dsuf_weight* w13, int32_t act_mode, const dsuf_moe_plan* plan,
                            uint64_t xq, uint64_t xs, float swiglu_limit, uint64_t act_out) {
    if (!ctx || !w13) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    if (plan->p == 0) return DSUF_OK;   /* an empty batch launches nothing, like route / quant / unpermute */
    DSUF_REQUIRE(ctx, (xq & 15) == 0, "moe_w13: xq must be 16-byte aligned");
    return launch_stream_moe(ctx, (cudaStream_t)stream, w13, EPI_W13, act_mode, plan, (const void*)xq, (const void*)xs, swiglu_limit,
                             (void*)act_out, w13->d.n / 2);
}

int32_t dsuf_moe_w2(dsuf_ctx* ctx, void* stream, const dsuf_weight* w2, int32_t act_mode, const dsuf_moe_plan* plan, uint64_t act_q,
                    uint64_t act_s, uint64_t yrows_out) {
    if (!ctx || !w2) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    if (plan->p == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, (act_q & 15) == 0, "moe_w2: act_q must be 16-byte aligned");
    return launch_stream_moe(ctx, (cudaStream_t)stream, w2, EPI_W2, act_mode, plan, (const void*)act_q, (const void*)act_s, 0.f,
                             (void*)yrows_out, w2->d.n);
}

int32_t dsuf_moe_unpermute(dsuf_ctx* ctx, void* stream, const dsuf_moe_plan* plan, uint64_t yrows, uint64_t shared, int32_t t,
                           int32_t topk, int32_t h, uint64_t out, int32_t ldo) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, topk >= 1 && topk <= 16 && (long long)t * topk == plan->p, "unpermute: t*topk != plan.p");
    DSUF_REQUIRE(ctx, h > 0 && h % 4 == 0 && ldo >= h && ldo % 4 == 0, "unpermute: h and ldo must be multiples of 4");
    if (t == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, yrows && out && (yrows & 15) == 0 && (out & 7) == 0, "unpermute: null or misaligned pointer");
    return launch_unpermute(ctx, (cudaStream_t)stream, plan, (const float*)yrows, (const void*)shared, t, topk, h, (void*)out, ldo);
}

int32_t dsuf_moe_unpermute_quant(dsuf_ctx* ctx, void* stream, const dsuf_moe_plan* plan, uint64_t yrows, uint64_t shared, int32_t t,
                                 int32_t topk, int32_t h, uint64_t out, int32_t ldo, int32_t mode, uint64_t xq, uint64_t xs) {
    if (!ctx) return DSUF_E_BADARG;
    int rc = check_plan(ctx, plan);
    if (rc) return rc;
    DSUF_REQUIRE(ctx, topk >= 1 && topk <= 16 && (long long)t * topk == plan->p, "unpermute_quant: t*topk != plan.p");
    DSUF_REQUIRE(ctx, mode == DSUF_MODE_MX || mode == DSUF_MODE_DS, "unpermute_quant: mode");
    DSUF_REQUIRE(ctx, h > 0 && h % 128 == 0 && ldo >= h && ldo % 8 == 0, "unpermute_quant: h must be a multiple of 128, ldo of 8");
    if (t == 0) return DSUF_OK;
    DSUF_REQUIRE(ctx, yrows && out && xq && xs && (yrows & 15) == 0 && (out & 15) == 0 && (shared & 15) == 0 && (xq & 7) == 0 && (xs & 3) == 0,
                 "unpermute_quant: null or misaligned pointer");
    return launch_unpermute_quant(ctx, (cudaStream_t)stream, plan, (const float*)yrows, (const void*)shared, t, topk, h, (void*)out, ldo, mode,
                                  (void*)xq, (void*)xs);
}

}  // extern "C"
