// Host launchers of the streaming (decode-shape) kernels: geometry checks, TMA descriptors for the activation
// rows, instantiation table.  Launch contracts mirror ops::gemv (crates/engine/src/ops.rs:331-474: shape
// preconditions returned as errors, never UB) and ops::moe_gemv (ops.rs:482-634).
#include <stdlib.h>
#include "internal.h"
#include "stream_gemv.cuh"
#include "tc_stream.cuh"
#include "tc_prefill.cuh"

namespace dsuf {

constexpr int WS_MAX_CTAS = 256;
constexpr int WS_MAX_ROW_TILES = 8192;
constexpr size_t WS_PARTIAL_BYTES = (size_t)WS_MAX_CTAS * 2 * 64 * 128 * sizeof(float);  // [cta][head/tail][<=64 tokens][128 rows]
constexpr size_t WS_BYTES = WS_PARTIAL_BYTES + WS_MAX_ROW_TILES * sizeof(int);

int encode_x_map(dsuf_ctx* ctx, CUtensorMap* tm, const void* base, int k_bytes, long long rows, int box_rows) {
    for (const auto& e : ctx->xmaps)
        if (e.base == base && e.k_bytes == k_bytes && e.rows == rows && e.box_rows == box_rows) {
            *tm = e.tm;
            return DSUF_OK;
        }
    cuuint64_t dims[2] = {(cuuint64_t)k_bytes, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k_bytes};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t es[2] = {1u, 1u};
    CUresult r = ctx->encode_tiled(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, es,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(ctx, DSUF_E_BADARG, "cuTensorMapEncodeTiled(activations) failed: %d", (int)r);
    auto& slot = ctx->xmaps[ctx->xmap_next++ % (sizeof(ctx->xmaps) / sizeof(ctx->xmaps[0]))];
    slot.base = base; slot.k_bytes = k_bytes; slot.rows = rows; slot.box_rows = box_rows; slot.tm = *tm;
    return DSUF_OK;
}

template <int FMT, int WMX, int AMX, int N, int EPI, int PAIR = 1>
static int set_attr_tc(dsuf_ctx* ctx) {
    cudaError_t e = cudaFuncSetAttribute(tc_stream_kernel<FMT, WMX, AMX, N, EPI, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         TcCfg<N, PAIR>::SMEM);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(tc_stream)");
    return DSUF_OK;
}

template <int FMT, int WMX, int AMX, int NT8, int EPI>
static int set_attr(dsuf_ctx* ctx) {
    cudaError_t e = cudaFuncSetAttribute(stream_gemv_kernel<FMT, WMX, AMX, NT8, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         StreamCfg<FMT>::SMEM);
    if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(stream_gemv)");
    return DSUF_OK;
}

int stream_setup(dsuf_ctx* ctx) {
    int rc = 0;
#define SA(...) if ((rc = set_attr<__VA_ARGS__>(ctx))) return rc
    SA(FMT_FP8, 0, 0, 1, EPI_DENSE); SA(FMT_FP8, 0, 0, 2, EPI_DENSE);
    SA(FMT_FP8, 1, 1, 1, EPI_DENSE); SA(FMT_FP8, 1, 1, 2, EPI_DENSE);
    SA(FMT_FP4, 1, 0, 1, EPI_W13); SA(FMT_FP4, 1, 0, 2, EPI_W13);
    SA(FMT_FP4, 1, 1, 1, EPI_W13); SA(FMT_FP4, 1, 1, 2, EPI_W13);
    SA(FMT_FP4, 1, 0, 1, EPI_W2); SA(FMT_FP4, 1, 0, 2, EPI_W2);
    SA(FMT_FP4, 1, 1, 1, EPI_W2); SA(FMT_FP4, 1, 1, 2, EPI_W2);
#undef SA
#define ST(...) if ((rc = set_attr_tc<__VA_ARGS__>(ctx))) return rc
    ST(FMT_FP8, 0, 0, 8, EPI_DENSE); ST(FMT_FP8, 0, 0, 16, EPI_DENSE); ST(FMT_FP8, 0, 0, 32, EPI_DENSE); ST(FMT_FP8, 0, 0, 64, EPI_DENSE);
    ST(FMT_FP8, 1, 1, 8, EPI_DENSE); ST(FMT_FP8, 1, 1, 16, EPI_DENSE); ST(FMT_FP8, 1, 1, 32, EPI_DENSE); ST(FMT_FP8, 1, 1, 64, EPI_DENSE);
    ST(FMT_FP4, 1, 0, 8, EPI_W13); ST(FMT_FP4, 1, 0, 16, EPI_W13); ST(FMT_FP4, 1, 0, 128, EPI_W13);
    ST(FMT_FP4, 1, 1, 8, EPI_W13); ST(FMT_FP4, 1, 1, 16, EPI_W13); ST(FMT_FP4, 1, 1, 128, EPI_W13);
    ST(FMT_FP4, 1, 0, 8, EPI_W2); ST(FMT_FP4, 1, 0, 16, EPI_W2); ST(FMT_FP4, 1, 0, 128, EPI_W2);
    ST(FMT_FP4, 1, 1, 8, EPI_W2); ST(FMT_FP4, 1, 1, 16, EPI_W2); ST(FMT_FP4, 1, 1, 128, EPI_W2);
    // two tile records per ring stage (weights with an even number of K tiles)
    ST(FMT_FP4, 1, 0, 8, EPI_W13, 2); ST(FMT_FP4, 1, 0, 16, EPI_W13, 2); ST(FMT_FP4, 1, 1, 8, EPI_W13, 2); ST(FMT_FP4, 1, 1, 16, EPI_W13, 2);
    ST(FMT_FP4, 1, 0, 8, EPI_W2, 2); ST(FMT_FP4, 1, 0, 16, EPI_W2, 2); ST(FMT_FP4, 1, 1, 8, EPI_W2, 2); ST(FMT_FP4, 1, 1, 16, EPI_W2, 2);
    ST(FMT_FP8, 0, 0, 8, EPI_DENSE, 2); ST(FMT_FP8, 0, 0, 16, EPI_DENSE, 2); ST(FMT_FP8, 0, 0, 32, EPI_DENSE, 2); ST(FMT_FP8, 0, 0, 64, EPI_DENSE, 2);
    ST(FMT_FP8, 1, 1, 8, EPI_DENSE, 2); ST(FMT_FP8, 1, 1, 16, EPI_DENSE, 2); ST(FMT_FP8, 1, 1, 32, EPI_DENSE, 2); ST(FMT_FP8, 1, 1, 64, EPI_DENSE, 2);
#undef ST
    // 128-token steps, except the dense DS GEMM, which walks a slot in two 64-token halves (measured: 1.51 against
    // 1.79 ms on 7168 x 7168 x 16384 tokens; for the FP4 expert GEMMs with DS scales the halves are 12 - 19 % slower)
    for (const void* f : {(const void*)tc_prefill_kernel<EPI_W13, 1>, (const void*)tc_prefill_kernel<EPI_W2, 1>,
                          (const void*)tc_prefill_kernel<EPI_W13, 0>, (const void*)tc_prefill_kernel<EPI_W2, 0>,
                          (const void*)tc_prefill_kernel<EPI_DENSE, 1, FMT_FP8, 1>}) {
        cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, TcpCfg::SMEM);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(tc_prefill)");
    }
    for (const void* f : {(const void*)tc_prefill_kernel<EPI_DENSE, 0, FMT_FP8, 0, 64>}) {
        cudaError_t e = cudaFuncSetAttribute(f, cudaFuncAttributeMaxDynamicSharedMemorySize, TcpCfgT<64>::SMEM);
        if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFuncSetAttribute(tc_prefill, 64-token steps)");
    }
    return DSUF_OK;
}

static void fill_common(dsuf_ctx* ctx, StreamArgs& a, const dsuf_weight* w) {
    memset(&a, 0, sizeof(a));
    a.tm_w = w->tm_stream;
    a.wtiles = (const uint8_t*)w->d.tiles;
    a.wscale_ds = (const float*)w->d.scales_ds;
    a.status = ctx->dev_status;
    a.RT = w->rt;
    a.KT = w->kt;
    a.rec_bytes = w->rec_bytes;
    a.codes_bytes = w->codes_bytes;
    a.n_rows = w->d.n;
    a.alpha = 1.0f;
}

int launch_stream_dense(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_weight* w, const void* xq, const void* xs, int m,
                        void* out, int ldo, float alpha, void* workspace, int* counters_at, const dsuf_gemm_opts* opts) {
    DSUF_REQUIRE(ctx, w->d.fmt == DSUF_FMT_FP8 && w->d.n_experts == 1, "dsuf_gemm_fp8: weight is not a dense FP8 weight");
    const int n_first = (opts && opts->epilogue == DSUF_EPI_SWIGLU) ? w->d.n / 2 : (opts && opts->n_split > 0) ? opts->n_split : w->d.n;   // columns of `out`
    DSUF_REQUIRE(ctx, ldo >= n_first, "dsuf_gemm_fp8: ldo %d < %d output columns", ldo, n_first);
    DSUF_REQUIRE(ctx, xq && xs && out, "dsuf_gemm_fp8: null pointer");
    DSUF_REQUIRE(ctx, !w->d.gate_up || (opts && opts->epilogue == DSUF_EPI_SWIGLU),
                 "dsuf_gemm_fp8: a gate/up-interleaved weight is only meaningful with the SwiGLU epilogue (dsuf_gemm_fp8_ex)");
    StreamArgs a;
    fill_common(ctx, a, w);
    if (opts) {
        DSUF_REQUIRE(ctx, opts->n_split >= 0 && opts->n_split < w->d.n, "dsuf_gemm_fp8_ex: n_split (%d) must be in 0..n-1", opts->n_split);
        DSUF_REQUIRE(ctx, opts->n_split == 0 || (opts->out2 && opts->ldo2 >= w->d.n - opts->n_split),
                     "dsuf_gemm_fp8_ex: n_split needs out2 with ldo2 >= n - n_split");
        DSUF_REQUIRE(ctx, opts->epilogue == DSUF_EPI_STORE || opts->epilogue == DSUF_EPI_SWIGLU || opts->epilogue == DSUF_EPI_SQRT_SOFTPLUS ||
                              opts->epilogue == DSUF_EPI_ACCUMULATE,
                     "dsuf_gemm_fp8_ex: unknown epilogue %d", opts->epilogue);
        if (opts->epilogue == DSUF_EPI_SWIGLU) {
            DSUF_REQUIRE(ctx, w->d.gate_up && w->d.mode == DSUF_MODE_MX, "dsuf_gemm_fp8_ex: the SwiGLU epilogue needs an MX weight packed with dsuf_pack_fp8_weight_gate_up");
            DSUF_REQUIRE(ctx, ctx->use_tc, "dsuf_gemm_fp8_ex: the SwiGLU epilogue runs on the tcgen05 path only");
            DSUF_REQUIRE(ctx, opts->alpha == 1.0f && !opts->out_f32 && opts->n_split == 0, "dsuf_gemm_fp8_ex: the SwiGLU epilogue takes alpha = 1, bf16 output, no split");
            DSUF_REQUIRE(ctx, ldo >= w->d.n / 2, "dsuf_gemm_fp8_ex: ldo %d < n / 2 = %d activation columns", ldo, w->d.n / 2);
            a.swiglu = 1;
            a.swiglu_limit = opts->swiglu_limit;
        }
        a.ssp = opts->epilogue == DSUF_EPI_SQRT_SOFTPLUS ? 1 : 0;
        if (opts->rope_cos) {
            DSUF_REQUIRE(ctx, ctx->use_tc && opts->epilogue == DSUF_EPI_STORE && !opts->out_f32, "dsuf_gemm_fp8_ex: the fused rotary embedding needs the tcgen05 path, the store epilogue and bf16 output");
            DSUF_REQUIRE(ctx, opts->rope_sin && opts->rope_pos && (opts->rope_cos & 3) == 0 && (opts->rope_sin & 3) == 0 && (opts->rope_pos & 3) == 0,
                         "dsuf_gemm_fp8_ex: rope tables / position null or misaligned");
            DSUF_REQUIRE(ctx, opts->rope_head >= 2 && opts->rope_head % 2 == 0 && opts->rope_off >= 0 && opts->rope_off % 2 == 0 &&
                              opts->rope_off < opts->rope_head && opts->rope_head - opts->rope_off <= 64 && w->d.n % 2 == 0 && opts->n_split % 2 == 0,
                         "dsuf_gemm_fp8_ex: rope_head / rope_off must be even, 0 <= rope_off < rope_head, at most 64 rotated rows per head");
            a.rope_cos = (const float*)opts->rope_cos;
            a.rope_sin = (const float*)opts->rope_sin;
            a.rope_pos = (const int*)opts->rope_pos;
            a.rope_head = opts->rope_head;
            a.rope_off = opts->rope_off;
        }
        a.accumulate = opts->epilogue == DSUF_EPI_ACCUMULATE ? 1 : 0;
        a.out_f32 = (opts->out_f32 || a.ssp || a.accumulate) ? 1 : 0;
        a.n_split = opts->n_split;
        a.out2 = (void*)opts->out2;
        a.ldo2 = opts->ldo2;
        alpha = opts->alpha;
    }
    if (ctx->use_tc && m > 64) {
        // prefill-size M: 128-token tiles x pairs of weight row tiles (tc_prefill.cuh); needs no workspace
        const bool ds = w->d.mode != DSUF_MODE_MX;
        int rc = encode_x_map(ctx, &a.tm_x, xq, w->d.k, m, ds ? 64 : 128);
        if (rc) return rc;
        a.tm_w = w->tm_tc;
        a.xscale = xs;
        a.out = out;
        a.m = m;
        a.x_rows = m;
        a.ldo = ldo;
        a.alpha = alpha;
        const int grid = ctx->sm_count;
        if (!ds)
            return launch(ctx, stream, tc_prefill_kernel<EPI_DENSE, 1, FMT_FP8, 1>, dim3(grid), dim3(TcpCfg::THREADS), (size_t)TcpCfg::SMEM, a);
        return launch(ctx, stream, tc_prefill_kernel<EPI_DENSE, 0, FMT_FP8, 0, 64>, dim3(grid), dim3(TcpCfgT<64>::THREADS),
                      (size_t)TcpCfgT<64>::SMEM, a);
    }
    const int m_max = ctx->use_tc ? 64 : 16;
    DSUF_REQUIRE(ctx, m >= 1 && m <= m_max, "dsuf_gemm_fp8: the mma.sync decode path takes 1..%d token rows per call, got %d", m_max, m);
    DSUF_REQUIRE(ctx, w->rt <= WS_MAX_ROW_TILES, "dsuf_gemm_fp8: too many row tiles (%d)", w->rt);
    DSUF_REQUIRE(ctx, workspace, "dsuf_gemm_fp8: null workspace");
    const int nt8 = m <= 8 ? 1 : 2;
    const int ntok = m <= 8 ? 8 : m <= 16 ? 16 : m <= 32 ? 32 : 64;
    int rc = encode_x_map(ctx, &a.tm_x, xq, w->d.k, m, ntok);
    if (rc) return rc;
    a.xscale = xs;
    a.out = out;
    a.partial = (float*)workspace;
    a.counters = counters_at ? counters_at : (int*)((uint8_t*)workspace + WS_PARTIAL_BYTES);
    a.m = m;
    a.x_rows = m;
    a.ldo = ldo;
    a.alpha = alpha;
    // the tcgen05 kernel streams two K tiles per ring step where the tile count is even: everything below counts steps
    const int pair = (ctx->use_tc && ctx->use_pairs && (w->kt & 1) == 0) ? 2 : 1;
    const int kt = w->kt / pair;
    const long long tot = (long long)w->rt * kt;
    int grid = ctx->sm_count < WS_MAX_CTAS ? ctx->sm_count : WS_MAX_CTAS;
    if (tot < grid) grid = (int)tot;
    // Stream-K balances to one tile but pays a partial-sum exchange per split row tile (a few microseconds on a kernel
    // of tens); whole row tiles per CTA are preferred when they need no more tile-steps than that.
    // the stream-K exchange of partial sums through global memory (fence, counter, re-read by the last CTA of a row tile)
    // measured 5-6 us on kernels of 12-16: as much as ten ring steps of two tiles
    const long long fix = 20 / pair;
    const long long steps_streamk = (tot + grid - 1) / grid + fix, steps_whole = (long long)((w->rt + grid - 1) / grid) * kt;
    a.whole_items = steps_whole <= steps_streamk ? 1 : 0;
    const bool mx = w->d.mode == DSUF_MODE_MX;
    int cluster = 1;
    if (ctx->use_tc && ctx->use_kslices) {
        // Weights with few row tiles: one row tile per cluster, K cut into 1, 2, 4 or 8 slices that are summed through
        // distributed shared memory (~1 us) instead of through global partials.  Cost in ring steps of a CTA's stream;
        // taken when better than the other two decompositions.
        const long long steps_other = a.whole_items ? steps_whole : steps_streamk;
        long long best = steps_other;
        for (int cs : {1, 2, 4, 8}) {
            // (clusters of 8 fit twice into a GPC of 16-20 SMs at one CTA per SM: 16 of them at most run at once)
            if ((long long)w->rt * cs > (cs == 8 ? 128 : grid) || kt < cs) continue;
            const long long steps = (kt + cs - 1) / cs + (cs > 1 ? (pair == 2 ? 2 : 3) : 0);
            if (steps < best) { best = steps; cluster = cs; a.kslices = cs; }
        }
        if (a.kslices) grid = w->rt * a.kslices;
    }
    if (ctx->use_tc) {
        a.tm_w = w->tm_tc;
#define GT(WMX, AMX, NN) (pair == 2 ? launch_cluster(ctx, stream, tc_stream_kernel<FMT_FP8, WMX, AMX, NN, EPI_DENSE, 2>, dim3(grid), dim3(TcCfg<NN, 2>::THREADS), (size_t)TcCfg<NN, 2>::SMEM, cluster, a) \
                                 : launch_cluster(ctx, stream, tc_stream_kernel<FMT_FP8, WMX, AMX, NN, EPI_DENSE>, dim3(grid), dim3(TcCfg<NN>::THREADS), (size_t)TcCfg<NN>::SMEM, cluster, a))
        if (mx) return ntok == 8 ? GT(1, 1, 8) : ntok == 16 ? GT(1, 1, 16) : ntok == 32 ? GT(1, 1, 32) : GT(1, 1, 64);
        return ntok == 8 ? GT(0, 0, 8) : ntok == 16 ? GT(0, 0, 16) : ntok == 32 ? GT(0, 0, 32) : GT(0, 0, 64);
#undef GT
    }
    const size_t smem = StreamCfg<FMT_FP8>::SMEM;
#define GO(WMX, AMX, NT) launch(ctx, stream, stream_gemv_kernel<FMT_FP8, WMX, AMX, NT, EPI_DENSE>, dim3(grid), dim3(STREAM_THREADS), smem, a)
    if (mx) return nt8 == 1 ? GO(1, 1, 1) : GO(1, 1, 2);
    return nt8 == 1 ? GO(0, 0, 1) : GO(0, 0, 2);
#undef GO
}

int launch_stream_moe(dsuf_ctx* ctx, cudaStream_t stream, const dsuf_weight* w, int epi, int act_mode, const dsuf_moe_plan* plan,
                      const void* xq, const void* xs, float swiglu_limit, void* out, int ldo) {
    DSUF_REQUIRE(ctx, w->d.fmt == DSUF_FMT_FP4, "grouped streaming GEMM: weight is not FP4");
    DSUF_REQUIRE(ctx, plan->tile_rows == 8 || plan->tile_rows == 16 || (plan->tile_rows == 128 && ctx->use_tc),
                 "grouped GEMM: plan tile_rows must be 8 or 16 (any decode path) or 128 (tcgen05 path)");
    DSUF_REQUIRE(ctx, xq && xs && out, "grouped streaming GEMM: null pointer");
    DSUF_REQUIRE(ctx, epi != EPI_W13 || w->d.gate_up, "dsuf_moe_w13_swiglu: weight was not packed with gate_up=1");
    if (plan->p == 0) return DSUF_OK;  // an empty batch: nothing to launch (route, quant and unpermute return OK as well)
    StreamArgs a;
    fill_common(ctx, a, w);
    const int nt8 = plan->tile_rows / 8;
    const bool prefill_pairs = ctx->use_tc && plan->tile_rows == 128;
    int rc = encode_x_map(ctx, &a.tm_x, xq, w->d.k, plan->p, plan->tile_rows);
    if (rc) return rc;
    a.xscale = xs;
    a.slots = (const int4*)plan->tiles;
    a.nslots = (const int*)plan->ntiles;
    a.row_w = (const float*)plan->row_w;
    a.out = out;
    a.x_rows = plan->p;
    a.ldo = ldo;
    a.swiglu_limit = swiglu_limit;
    const int grid = ctx->sm_count;
    const bool amx = act_mode == DSUF_MODE_MX;
    if (ctx->use_tc) {
        a.tm_w = w->tm_tc;
#define GT(AMX, NN, EPI) launch(ctx, stream, tc_stream_kernel<FMT_FP4, 1, AMX, NN, EPI>, dim3(grid), dim3(TcCfg<NN>::THREADS), (size_t)TcCfg<NN>::SMEM, a)
        const int tr = plan->tile_rows;
        if (prefill_pairs) {
            // prefill-size token tiles: two row tiles per step, two issuers
#define GP(EPI, AMX) launch(ctx, stream, tc_prefill_kernel<EPI, AMX>, dim3(grid), dim3(TcpCfg::THREADS), (size_t)TcpCfg::SMEM, a)
            if (epi == EPI_W13) return amx ? GP(EPI_W13, 1) : GP(EPI_W13, 0);
            return amx ? GP(EPI_W2, 1) : GP(EPI_W2, 0);
#undef GP
        }
        if (tr <= 16 && (w->kt & 1) == 0 && ctx->use_pairs) {
            // decode slots: two tile records per ring stage, half the pipeline hand-offs per byte streamed
#define GT2(AMX, NN, EPI) launch(ctx, stream, tc_stream_kernel<FMT_FP4, 1, AMX, NN, EPI, 2>, dim3(grid), dim3(TcCfg<NN, 2>::THREADS), (size_t)TcCfg<NN, 2>::SMEM, a)
            if (epi == EPI_W13) {
                if (amx) return tr == 8 ? GT2(1, 8, EPI_W13) : GT2(1, 16, EPI_W13);
                return tr == 8 ? GT2(0, 8, EPI_W13) : GT2(0, 16, EPI_W13);
            }
            if (amx) return tr == 8 ? GT2(1, 8, EPI_W2) : GT2(1, 16, EPI_W2);
            return tr == 8 ? GT2(0, 8, EPI_W2) : GT2(0, 16, EPI_W2);
#undef GT2
        }
        if (epi == EPI_W13) {
            if (amx) return tr == 8 ? GT(1, 8, EPI_W13) : tr == 16 ? GT(1, 16, EPI_W13) : GT(1, 128, EPI_W13);
            return tr == 8 ? GT(0, 8, EPI_W13) : tr == 16 ? GT(0, 16, EPI_W13) : GT(0, 128, EPI_W13);
        }
        if (amx) return tr == 8 ? GT(1, 8, EPI_W2) : tr == 16 ? GT(1, 16, EPI_W2) : GT(1, 128, EPI_W2);
        return tr == 8 ? GT(0, 8, EPI_W2) : tr == 16 ? GT(0, 16, EPI_W2) : GT(0, 128, EPI_W2);
#undef GT
    }
    const size_t smem = StreamCfg<FMT_FP4>::SMEM;
#define GO(AMX, NT, EPI) launch(ctx, stream, stream_gemv_kernel<FMT_FP4, 1, AMX, NT, EPI>, dim3(grid), dim3(STREAM_THREADS), smem, a)
    if (epi == EPI_W13) {
        if (amx) return nt8 == 1 ? GO(1, 1, EPI_W13) : GO(1, 2, EPI_W13);
        return nt8 == 1 ? GO(0, 1, EPI_W13) : GO(0, 2, EPI_W13);
    }
    if (amx) return nt8 == 1 ? GO(1, 1, EPI_W2) : GO(1, 2, EPI_W2);
    return nt8 == 1 ? GO(0, 1, EPI_W2) : GO(0, 2, EPI_W2);
#undef GO
}

size_t stream_workspace_bytes() { return WS_BYTES; }

}  // namespace dsuf
