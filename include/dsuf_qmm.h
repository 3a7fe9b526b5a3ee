/*
 * dsuf_qmm.h -- C ABI of libdsuf_qmm, the B200 (sm_100a) implementation of deepseek-ultrafast's quantized
 * matrix-product path: FP8 activation quantization, FP8 block-scaled GEMV/GEMM, grouped MXFP4 expert GEMMs
 * (gate/up + SwiGLU, down) and the routed-token permute / unpermute around them.
 *
 * The reference has no C ABI: crates/engine/src/ops.rs fills #[repr(C)] parameter structs and launches cubin
 * kernels by name through crates/cuda/src/lib.rs:630-664.  Each entry point below names the reference
 * interface it stands in for, so crates/engine keeps its call surface and only the bodies of those functions
 * turn into FFI calls.
 *
 * Conventions (mirroring crates/cuda + crates/engine):
 *   - uint64_t arguments are device pointers; `stream` is a CUstream / cudaStream_t passed as void*.
 *   - every function returns int32_t: 0 ok, >0 a CUDA error code, <0 a DSUF_E_* code; dsuf_last_error() gives
 *     the message.  Preconditions are validated on the host and reported -- never undefined behaviour.
 *   - hot calls are asynchronous on the caller's stream, allocate nothing, never synchronise and may be
 *     recorded into a CUDA graph; functions marked (load-time) may allocate or synchronise.
 *   - the caller owns all device memory, including scratch; sizes come from the *_bytes() queries.
 *   - one context per device, used from the thread that has that device current; no global mutable state.
 *   - bf16 data is raw uint16 bit patterns; FP8 codes are e4m3 bytes; FP4 codes are e2m1, two per byte,
 *     low nibble = even k; UE8M0 scales are exponent bytes (2^(b-127)).
 */
#ifndef DSUF_QMM_H
#define DSUF_QMM_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { DSUF_OK = 0, DSUF_E_BADARG = -1, DSUF_E_UNSUPPORTED = -2, DSUF_E_TIMEOUT = -3, DSUF_E_NCCL = -4, DSUF_E_NOMEM = -5 };

/* Scale geometries.  MX = what the reference implements (1x32 activations, 32x32 FP8 weights, power-of-two
 * UE8M0 scales: crates/kernels/cu/quantblocks.cuh:7-57, crates/model/src/formats.rs:59-84).
 * DS = 1x128 activations / 128x128 FP8 weights with fp32 scales amax/448. */
enum { DSUF_MODE_MX = 0, DSUF_MODE_DS = 1 };
enum { DSUF_FMT_FP8 = 0, DSUF_FMT_FP4 = 1 };               /* WFmt, crates/engine/src/ops.rs:6-39 */
enum { DSUF_SCORE_IDENTITY = 0, DSUF_SCORE_SOFTMAX = 1, DSUF_SCORE_SQRT_SOFTPLUS = 2 };

typedef struct dsuf_ctx dsuf_ctx;
typedef struct dsuf_weight dsuf_weight;

typedef struct {
    int32_t code;   /* 0 = no device-side error; 1 = a bounded wait expired; 2 = inconsistent plan; 3 = the ranks of a peer
                       exchange no longer count the same calls (a peer's flag is more than one call ahead) */
    int32_t kernel; /* kernel id */
    int32_t cta;
    int32_t where;
} dsuf_dev_status;

/* ---- context (load-time).  Stands in for Device::new + ops::hw() (crates/cuda/src/lib.rs:52-138,
 * crates/engine/src/ops.rs:205-232): binds to the device's primary context, queries SM count and the
 * shared-memory opt-in, raises the kernels' dynamic shared-memory limits. ---- */
int32_t dsuf_ctx_create(int32_t device, dsuf_ctx** out);
int32_t dsuf_ctx_destroy(dsuf_ctx* ctx);
/* Copies the message of the last failing call on this context into buf (NUL-terminated). */
int32_t dsuf_last_error(dsuf_ctx* ctx, char* buf, size_t len);
/* Enables (1) or disables (0) programmatic dependent launch on every kernel of this context
 * (Launch{pdl}, crates/cuda/src/lib.rs:633-638).  Default 0. */
int32_t dsuf_ctx_set_pdl(dsuf_ctx* ctx, int32_t enabled);
/* Decode-shape kernels: 1 = tcgen05 streaming kernel (TMA-unpacked FP4, block scales in tensor memory),
 * 0 = mma.sync streaming kernel (the counterpart of the reference's cu/gemv.cu family).  Both compute the same
 * function; the choice mirrors the reference's runtime switch between gemv and tc_gemv (model.rs:1523-1530). */
int32_t dsuf_ctx_set_decode_path(dsuf_ctx* ctx, int32_t tcgen05);
/* Decode-shape expert GEMMs on the tcgen05 path: 1 (default) streams two 128-K tile records per ring stage where the
 * weight has an even number of K tiles (half the barrier hand-offs per byte), 0 one per stage.  Both are deterministic;
 * they add the per-tile fp32 partial sums in a different order. */
int32_t dsuf_ctx_set_stage_pairs(dsuf_ctx* ctx, int32_t enabled);
/* Decode-shape dense GEMV on the tcgen05 path: 1 (default) lets weights with few row tiles run as one row tile per
 * thread-block cluster with K cut into slices summed through distributed shared memory -- the counterpart of the cluster
 * K-split of ops::gemv / ops::tc_gemv (ops.rs:298-328, 1105-1107) -- where that beats stream-K with global partial sums;
 * 0 keeps stream-K / whole row tiles only.  The results of the two are both deterministic but differ in summation order. */
int32_t dsuf_ctx_set_dense_ksplit(dsuf_ctx* ctx, int32_t enabled);
/* (synchronises `stream`) Reads and clears the device status word.  The reference's device waits are unbounded
 * spins with no error reporting (cu/comm.cu:217-224); here every wait is bounded and reports through this. */
int32_t dsuf_status_poll(dsuf_ctx* ctx, void* stream, dsuf_dev_status* out);
int32_t dsuf_sm_count(dsuf_ctx* ctx);
/* How long the peer-exchange kernels (dsuf_ep_allreduce_bf16, dsuf_ep_combine_bf16) wait for a peer's announcement
 * before they give up, record code 1 in the status word and return with an incomplete sum: 1 us .. 10 s, default
 * about 2 s.  Set it to what the deployment's worst rank-to-rank skew allows.  The reference's waits never give up
 * (cu/comm.cu:217-224). */
int32_t dsuf_ctx_set_wait_budget_us(dsuf_ctx* ctx, int64_t microseconds);

/* ---- host-side weight formats (load-time, no GPU).  Replace crates/model/src/formats.rs + packing.rs. ---- */

/* quant_fp8_b32 twin (formats.rs:59-84) for MX; 128x128 fp32 amax/448 for DS.
 * w bf16 [n][k] -> codes [n][k], scales MX: u8 [n/32][k/32], DS: f32 [n/128][k/128]. */
int32_t dsuf_quant_fp8_weight_host(int32_t mode, const uint16_t* w, int32_t n, int32_t k, uint8_t* codes, void* scales);
/* Synthetic MXFP4 quantizer following the reference's FP4 rule (cu/kv_fp4.cu:25-32):
 * w bf16 [n][k] -> codes [n][k/2], scales u8 [n][k/32]. */
int32_t dsuf_quant_fp4_weight_host(const uint16_t* w, int32_t n, int32_t k, uint8_t* codes, uint8_t* scales);

/* Packed image = contiguous 128-row x 128-K tile records ordered [row tile][k tile], replacing tile_fp8 /
 * tile_fp4 / tile_sf_blocks (formats.rs:96-228) and expert_shard (packing.rs:174-254).  One image feeds both the
 * streaming decode kernels and the tcgen05 prefill kernels.
 *   FP8 MX: 16384 B codes + 512 B scale atom;  FP8 DS: 16384 B codes (scales stay a separate f32 [n/128][k/128]);
 *   FP4   :  8192 B codes + 512 B scale atom.
 * n is padded up to a multiple of 128 with zero rows; k must be a multiple of 128. */
size_t dsuf_packed_bytes(int32_t fmt, int32_t mode, int32_t n, int32_t k);
int32_t dsuf_pack_fp8_weight(int32_t mode, const uint8_t* codes, const void* scales, int32_t n, int32_t k, uint8_t* out);
/* The FP8 shared expert's gate/up weight (the w1 / w3 merge of Loader::layer, weights.rs:447-470, tile_fp8_k64 in
 * crates/model/src/formats.rs:120-143): MX codes [2*inter][k] with gate rows first, then up rows, and their 32x32 UE8M0
 * scales, packed with the same 8 + 8 gate / up row interleave as the FP4 experts, for dsuf_gemm_fp8_ex with the SwiGLU
 * epilogue (set dsuf_weight_desc.gate_up).  n % 64 == 0. */
int32_t dsuf_pack_fp8_weight_gate_up(const uint8_t* codes, const uint8_t* scales, int32_t n, int32_t k, uint8_t* out);
/* gate_up != 0: codes/scales are [2*inter][k] with gate rows first, then up rows (n = 2*inter); rows are
 * interleaved per 16-row group as 8 gate + the 8 matching up rows (the reference interleaves 32+32 per
 * 64-row quad, packing.rs:237-241) so the SwiGLU epilogue finds both halves in one thread. */
int32_t dsuf_pack_fp4_weight(const uint8_t* codes, const uint8_t* scales, int32_t n, int32_t k, int32_t gate_up, uint8_t* out);

/* ---- checkpoint-facing loaders (load-time, host only).  Replace Checkpoint (crates/model/src/st.rs:17-106), Loader::fp8
 * (crates/engine/src/weights.rs:254-276) and the expert part of Loader::layer (weights.rs:421-446). ---- */
typedef struct dsuf_ckpt dsuf_ckpt;
typedef struct {
    char dtype[16];        /* the safetensors dtype string: "F8_E4M3", "BF16", "F32", ... */
    int32_t rank;
    int64_t shape[8];
    const void* data;      /* inside the read-only mapping of the file; valid until dsuf_ckpt_close */
    size_t nbytes;
} dsuf_tensor_info;
/* Maps one .safetensors file, or every *.safetensors file of a directory in name order (Checkpoint::open, st.rs:24-31),
 * and indexes the tensors.  *out is set even when the call fails, so that dsuf_ckpt_last_error can be read; close it. */
int32_t dsuf_ckpt_open(const char* path, dsuf_ckpt** out);
int32_t dsuf_ckpt_close(dsuf_ckpt* c);
int32_t dsuf_ckpt_last_error(dsuf_ckpt* c, char* buf, size_t len);
int64_t dsuf_ckpt_count(dsuf_ckpt* c);
int32_t dsuf_ckpt_tensor(dsuf_ckpt* c, const char* name, dsuf_tensor_info* out);
/* Loader::fp8: `{name}.weight` F8_E4M3 [n][k] + `{name}.scale` UE8M0 [n/32][k/32] -> MX tile records of rows [r0, r1)
 * (multiples of 32; the records pad rows up to a multiple of 128), dsuf_packed_bytes(FP8, MX, r1 - r0, k) bytes at
 * tiles_out.  One image serves both the decode and the prefill kernels (the reference keeps a fragment-tiled and a
 * row-major copy, weights.rs:181-214). */
int32_t dsuf_ckpt_load_fp8_dense(dsuf_ckpt* c, const char* name, int32_t n, int32_t k, int32_t r0, int32_t r1, uint8_t* tiles_out);
/* Experts e0 .. e1-1 of `{prefix}.ffn.experts.{e}.{w1,w3,w2}.{weight,scale}` (FP4 codes two per byte + UE8M0 per 1x32;
 * w1 = gate [inter][dim], w3 = up [inter][dim], w2 = down [dim][inter]) -> tile records: w13_out receives
 * (e1 - e0) x dsuf_packed_bytes(FP4, MX, 2 inter, dim) bytes with gate / up rows interleaved for the SwiGLU epilogue,
 * w2_out (e1 - e0) x dsuf_packed_bytes(FP4, MX, dim, inter).  dim and inter multiples of 128. */
int32_t dsuf_ckpt_load_fp4_experts(dsuf_ckpt* c, const char* prefix, int32_t e0, int32_t e1, int32_t dim, int32_t inter, uint8_t* w13_out,
                                   uint8_t* w2_out);

/* Weight descriptor = Weight{fmt,w,s,n,k} / Experts (ops.rs:6-39, weights.rs:82-92). */
typedef struct {
    int32_t fmt;             /* DSUF_FMT_* */
    int32_t mode;            /* FP8: DSUF_MODE_*; FP4: ignored (always UE8M0 per 1x32) */
    int32_t n, k;            /* rows and K of one matrix */
    int32_t n_experts;       /* 1 for a dense weight */
    int32_t gate_up;         /* rows packed with dsuf_pack_fp4_weight(gate_up=1) */
    uint64_t tiles;          /* device: n_experts packed images back to back */
    uint64_t scales_ds;      /* device: FP8 DS only, f32 [n_pad/128][k/128] */
} dsuf_weight_desc;
/* (load-time) Builds the TMA descriptors for a packed weight (tensor_map_u8_sw128 / tensor_map_fp4_unpack_*,
 * crates/cuda/src/lib.rs:694-808, built by Loader::tc_copy, weights.rs:181-214). */
int32_t dsuf_weight_create(dsuf_ctx* ctx, const dsuf_weight_desc* desc, dsuf_weight** out);
int32_t dsuf_weight_destroy(dsuf_weight* w);

/* ---- hot calls ---- */

/* tc_quant_rows (cu/tcgemm.cu:300-340) and the in-GEMV quant_blocks8 staging (cu/quantblocks.cuh:7-57).
 * x bf16 [m][ldx] -> q [m][k]; scales MX: u8 [m][k/32], DS: f32 [m][k/128].  k % 128 == 0, ldx % 8 == 0. */
int32_t dsuf_act_quant_fp8(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t m, int32_t k,
                           uint64_t q_out, uint64_t scale_out);

/* tc_row_sumsq (cu/tcgemm.cu:341-355): sumsq_out[r] = sum_k x[r][k]^2 in fp32, in the reference's summation order
 * (one warp per row, lane l takes k = 8 l + 256 i + e, xor butterfly).  k % 8 == 0. */
int32_t dsuf_row_sumsq(dsuf_ctx* ctx, void* stream, uint64_t x, int32_t ldx, int32_t m, int32_t k, uint64_t sumsq_out);

/* tc_quant_rows with RMS pre-normalisation (TqParams.pw / norm_part / eps, cu/tcgemm.cu:286-340; launched by
 * Rank::gemm_tc, model.rs:1328-1345): quantizes v = bf16(norm_w[k] * (x[r][k] * rs[r])) with
 * rs = 1 / sqrt(sumsq[r] / k + eps) instead of x.  norm_w bf16 [k], sumsq f32 [m] (dsuf_row_sumsq, or a producer
 * kernel's own partial sums added up by the caller).  By default rs is evaluated with correctly rounded sqrt and
 * division; the reference uses the approximate rsqrtf instruction, so its codes can differ where a product sits on a
 * rounding boundary (dsuf_ctx_set_prenorm_rsqrt selects the reference's instruction). */
int32_t dsuf_act_quant_fp8_prenorm(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t m, int32_t k,
                                   uint64_t norm_w, uint64_t sumsq, float eps, uint64_t q_out, uint64_t scale_out);
/* How the pre-normalising quantizers (dsuf_act_quant_fp8_prenorm, dsuf_moe_gather_quant_prenorm) evaluate 1/sqrt:
 * 0 (default) correctly rounded, which a CPU can reproduce bit for bit; 1 the GPU's approximate rsqrt instruction, which
 * is what the reference's kernels execute (cu/tcgemm.cu:305, cu/tcmoe.cu:97) -- with it the codes and scales equal the
 * reference kernels' on the same GPU (about 1 code in 10^4 differs otherwise). */
int32_t dsuf_ctx_set_prenorm_rsqrt(dsuf_ctx* ctx, int32_t approximate);

/* Scratch of dsuf_gemm_fp8: stream-K partial sums and arrival counters.  Must be zeroed once with
 * dsuf_workspace_init before first use; the kernels leave it zeroed.  Calls sharing one workspace must be
 * stream-ordered. */
size_t dsuf_gemm_workspace_bytes(dsuf_ctx* ctx);
int32_t dsuf_workspace_init(dsuf_ctx* ctx, void* stream, uint64_t workspace, size_t bytes);

/* ops::gemv (ops.rs:331-474), ops::tc_gemv (ops.rs:1118-1163) and Rank::gemm_tc (model.rs:1328-1370) in one call:
 * out[m][n] (bf16, row stride ldo) = alpha * W . dequant(xq, xs).  Activations come pre-quantized from
 * dsuf_act_quant_fp8 in the weight's geometry.  Token rows per call: 1..16 on the mma.sync decode path; on the
 * tcgen05 path 1..64 take the weight-streaming kernel (one pass over W, uses the workspace) and any m > 64 takes the
 * prefill kernel (128-token tiles x pairs of 128-row weight tiles; the workspace is not touched and may be 0). */
int32_t dsuf_gemm_fp8(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m, uint64_t out,
                      int32_t ldo, float alpha, uint64_t workspace);

/* GemvOpts (crates/engine/src/ops.rs:165-193), the part that concerns the Store epilogue of a dense projection:
 *   alpha    the output scale
 *   out_f32  1 = fp32 output (out / out2 are float buffers) instead of bf16 (GemvOpts.out_f32; cu/gemv.cu:510-517)
 *   n_split  > 0 = weight rows [n_split, n) are written to out2 (row stride ldo2) at column row - n_split, rows
 *            [0, n_split) to out (GemvOpts.split: one launch for two projections merged along n, e.g. Loader::fp8_merged)
 * The Partial epilogue kind of the reference's dense GEMV (its K-split across launches; here the K reduction is inside the
 * launch) and the FP4 index-query branch of its fused RoPE (iq_head) are not offered. */
typedef struct {
    float alpha;
    int32_t out_f32;
    int32_t n_split;
    int32_t ldo2;
    uint64_t out2;
    int32_t epilogue;      /* DSUF_EPI_STORE, _SWIGLU, _SQRT_SOFTPLUS or _ACCUMULATE */
    float swiglu_limit;    /* SwiGLU: clamp as cu/gemv.cu:470-483 when > 0 */
    /* Fused rotary embedding (GemvOpts.rope, ops.rs:165-193; cu/gemv.cu:508-516), STORE epilogue, bf16 output, tcgen05
     * path: rope_cos / rope_sin f32 [positions][32], rope_pos a DEVICE int (token row m sits at position rope_pos[0] + m);
     * output rows r of the first output (r < n_split when split) with (r % rope_head) >= rope_off are rotated in
     * (even, odd) pairs.  rope_cos = 0: no rotation. */
    uint64_t rope_cos;
    uint64_t rope_sin;
    uint64_t rope_pos;
    int32_t rope_head;
    int32_t rope_off;
} dsuf_gemm_opts;
/* Epilogue::Store / Epilogue::SwiGlu (crates/engine/src/ops.rs:137-144).  SWIGLU: the weight holds gate and up rows
 * (packed by dsuf_pack_fp8_weight_gate_up, MX scales, tcgen05 path) and out receives bf16 [m][n/2] =
 * bf16(silu(bf16 gate) * bf16 up), the reference's shared-expert gate/up projection (gemm_tc with Epilogue::SwiGlu,
 * model.rs:3081-3084; cu/tcgemm.cu:89-110); alpha must be 1, out_f32 0, n_split 0.
 * SQRT_SOFTPLUS: the router-gate projection (ops::gemv with Epilogue::SqrtSoftplus, model.rs:3094; cu/gemv.cu:523):
 * fp32 out[m][n] = sqrt(softplus(alpha * dot)) (sqrt(x) itself above 20, cu/common.cuh:17-24), i.e. the scores
 * dsuf_moe_route_tokens takes with DSUF_SCORE_IDENTITY; out is always fp32 (out_f32 is implied), n_split works as for STORE.
 * ACCUMULATE: fp32 out[m][n] += alpha * dot -- what the reference's Epilogue::AtomicAdd is used for on dense weights
 * (several projections summed into one fp32 buffer, cu/gemv.cu:489-491), without atomics: every output element is written
 * by exactly one thread of the launch after the K reduction, so the sum is deterministic; out is fp32 (out_f32 implied). */
enum { DSUF_EPI_STORE = 0, DSUF_EPI_SWIGLU = 1, DSUF_EPI_SQRT_SOFTPLUS = 2, DSUF_EPI_ACCUMULATE = 3 };
/* dsuf_gemm_fp8 with options; same kernels, any number of token rows. */
int32_t dsuf_gemm_fp8_ex(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m, uint64_t out,
                         int32_t ldo, const dsuf_gemm_opts* opts, uint64_t workspace);

/* No counterpart in the reference.  Same function as dsuf_gemm_fp8 for callers that cannot allocate device memory
 * (an engine that spent its device budget on one start-up arena, a plugin without its own allocator, a caller for which
 * an allocation would synchronise the device): the stream-K scratch is a fixed array inside the library's device image
 * instead of a caller workspace.  Limits and rules:
 *   - about 10 MB per GPU that loads the library, held until the process exits;
 *   - weights of at most 131072 rows (1024 row tiles) on GPUs of at most 160 SMs; anything larger returns
 *     DSUF_E_BADARG with a message that says so;
 *   - all calls share the one array: calls that overlap on the GPU race, so keep them stream-ordered; its arrival
 *     counters are cleared on the stream before each launch, nothing else carries over between calls;
 *   - the first call on a device resolves the array's device address; make that call before any stream capture
 *     starts, and -- since the CUDA runtime may place the library's device image (the array included) in device memory
 *     only at that moment -- before the caller gives the rest of the device memory away.  The context's device must be
 *     current on every call.
 * Calls no cudaMalloc / cudaFree and no allocating library routine. */
int32_t dsuf_gemm_fp8_static(dsuf_ctx* ctx, void* stream, const dsuf_weight* w, uint64_t xq, uint64_t xs, int32_t m,
                             uint64_t out, int32_t ldo, float alpha);

/* No counterpart in the reference: a measurement aid for the roofline of the GEMM kernels.  Launches one CTA per SM that
 * issues `iters` tcgen05.mma (kind::mxf8f6f4.block_scale, M = 128, N = n_cols, K = 32; A e4m3 or e2m1) back to back on
 * operands that already sit in shared memory, and returns in *flop_per_launch the floating-point operations of the
 * launch; the caller times the launch with CUDA events.  FLOP / time is what the tensor cores of this GPU deliver to
 * that instruction at the clocks they hold: the measured ceiling the prefill kernels are compared with.
 * n_cols a multiple of 16 in 16..256. */
int32_t dsuf_probe_tensor_rate(dsuf_ctx* ctx, void* stream, int32_t n_cols, int32_t a_is_e2m1, int32_t iters,
                               double* flop_per_launch);

/* moe_route_tokens + route_token (cu/ops.cu:615-623, cu/route.cuh:3-56; RouteArgs ops.rs:124-135):
 * top-k of score+bias, ties to the lower id, weights = score / sum(selected scores) * route_scale.
 * scores f32 [t][n_exp] (logits when score_fn != IDENTITY), bias f32 [n_exp] or 0.
 * ids_out i32 [t][topk], w_out f32 [t][topk].  n_exp <= 512, topk <= 16. */
int32_t dsuf_moe_route(dsuf_ctx* ctx, void* stream, int32_t score_fn, uint64_t scores, uint64_t bias, int32_t t,
                       int32_t n_exp, int32_t topk, float route_scale, uint64_t ids_out, uint64_t w_out);

/* Permute plan = MpParams outputs (ops.rs:1478-1491) of moe_perm (cu/tcmoe.cu:19-69) and, with tile_rows = 8 or
 * 16, the decode MoePlan slots (cu/gemv.cu:9-17,715-776).  All buffers caller-allocated. */
typedef struct {
    uint64_t expert_off; /* i32 [n_exp+1]  first permuted row of each local expert */
    uint64_t row_pair;   /* i32 [p]        pair index (token*topk + j) of each permuted row */
    uint64_t pair_row;   /* i32 [p]        permuted row of each pair, -1 when its expert is not local */
    uint64_t row_w;      /* f32 [p]        routing weight of each permuted row */
    uint64_t tiles;      /* i32x4 [max_tiles] (local expert, first row, rows <= tile_rows, 0) */
    uint64_t ntiles;     /* i32 [2]        number of tiles, number of permuted rows */
    uint64_t scratch;    /* i32 [dsuf_moe_plan_scratch_ints(p, n_exp)] */
    int32_t p;           /* pairs = tokens * topk */
    int32_t n_exp;       /* local experts */
    int32_t tile_rows;   /* 8 / 16 (decode streaming) or 128 (tcgen05 prefill) */
    int32_t max_tiles;   /* capacity of tiles[]: p / tile_rows + n_exp is always enough */
} dsuf_moe_plan;
size_t dsuf_moe_plan_scratch_ints(int32_t p, int32_t n_exp);
/* Counting sort of the pairs by expert; rows of one expert are in ascending pair order (the reference's order
 * inside an expert depends on atomicAdd timing, cu/tcmoe.cu:62).  Pairs whose expert is outside
 * [e_lo, e_lo + n_exp) are dropped (expert-parallel shard). */
int32_t dsuf_moe_permute_plan(dsuf_ctx* ctx, void* stream, uint64_t ids, uint64_t w, int32_t e_lo, const dsuf_moe_plan* plan);

/* moe_gather_quant (cu/tcmoe.cu:88-133, MqParams ops.rs:1495-1509): quantize each token row once and write it
 * to all of its permuted rows.  x bf16 [t][ldx] -> xq [p][h], xs MX u8 [p][h/32] / DS f32 [p][h/128]. */
int32_t dsuf_moe_gather_quant(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t t, int32_t h,
                              int32_t topk, const dsuf_moe_plan* plan, uint64_t xq_out, uint64_t xs_out);

/* Decode front end in one launch: dsuf_moe_route + dsuf_moe_permute_plan + dsuf_moe_gather_quant for at most 1024
 * (token, expert) pairs, with the same outputs bit for bit.  The reference routes inside its decode MoE launch as well
 * (route_plan, cu/gemv.cu:715-776, RouteArgs in GemvParams); here the routing, the plan and the quantized permuted rows
 * are produced together and every later kernel only reads them.  scores f32 [t][n_exp_all] over ALL experts; the plan
 * keeps the pairs whose expert lies in [e_lo, e_lo + plan->n_exp). */
int32_t dsuf_moe_route_plan_gather(dsuf_ctx* ctx, void* stream, int32_t score_fn, uint64_t scores, uint64_t bias, int32_t t,
                                   int32_t n_exp_all, int32_t topk, float route_scale, uint64_t ids_out, uint64_t w_out, int32_t e_lo,
                                   const dsuf_moe_plan* plan, int32_t mode, uint64_t x, int32_t ldx, int32_t h, uint64_t xq_out,
                                   uint64_t xs_out);

/* The same with the RMS pre-normalisation of dsuf_act_quant_fp8_prenorm in front (moe_gather_quant with MqParams.pw,
 * cu/tcmoe.cu:88-133: every token row is normalised and quantised once, then written to its topk permuted rows).
 * norm_w bf16 [h], sumsq f32 [t] (dsuf_row_sumsq of x). */
int32_t dsuf_moe_gather_quant_prenorm(dsuf_ctx* ctx, void* stream, int32_t mode, uint64_t x, int32_t ldx, int32_t t, int32_t h,
                                      int32_t topk, const dsuf_moe_plan* plan, uint64_t norm_w, uint64_t sumsq, float eps,
                                      uint64_t xq_out, uint64_t xs_out);

/* Grouped gate/up GEMM + SwiGLU: moe_fp4_swiglu (cu/gemv.cu:1016-1692 via ops::moe_gemv, ops.rs:482-634) for
 * decode plans, tc_moe_w13 (cu/tcmoe.cu:184-588, TmParams ops.rs:1513-1534) for 128-row plans.
 * act_out bf16 [p][inter] indexed by permuted row:
 * bf16(silu(bf16 gate) * bf16 up * routing weight), optional clamp as cu/gemv.cu:470-483. */
int32_t dsuf_moe_w13_swiglu(dsuf_ctx* ctx, void* stream, const dsuf_weight* w13, int32_t act_mode, const dsuf_moe_plan* plan,
                            uint64_t xq, uint64_t xs, float swiglu_limit, uint64_t act_out);
/* Grouped down GEMM: moe_fp4_store / moe_w2 / tc_moe_w2.  act_q [p][inter] + act_s from dsuf_act_quant_fp8 over
 * act_out; yrows_out f32 [p][h] indexed by permuted row. */
int32_t dsuf_moe_w2(dsuf_ctx* ctx, void* stream, const dsuf_weight* w2, int32_t act_mode, const dsuf_moe_plan* plan,
                    uint64_t act_q, uint64_t act_s, uint64_t yrows_out);
/* Unpermute + combine, the nsum/src2 part of comm_push (cu/comm.cu:167-180):
 * out[t] = bf16(sum_j yrows[pair_row[t*topk+j]] (+ shared[t])), rows with pair_row < 0 skipped. */
int32_t dsuf_moe_unpermute(dsuf_ctx* ctx, void* stream, const dsuf_moe_plan* plan, uint64_t yrows, uint64_t shared, int32_t t,
                           int32_t topk, int32_t h, uint64_t out, int32_t ldo);
/* dsuf_moe_unpermute that also leaves its result quantized for the next projection: xq [t][h] FP8 codes and xs block
 * scales (mode MX: u8 [t][h/32], DS: f32 [t][h/128]) equal to dsuf_act_quant_fp8(mode, out) bit for bit -- the activation
 * staging the reference's next GEMV would run on these rows (quant_blocks8, cu/quantblocks.cuh:7-57) done by the producer.
 * h % 128 == 0, out and shared 16-byte aligned. */
int32_t dsuf_moe_unpermute_quant(dsuf_ctx* ctx, void* stream, const dsuf_moe_plan* plan, uint64_t yrows, uint64_t shared, int32_t t,
                                 int32_t topk, int32_t h, uint64_t out, int32_t ldo, int32_t mode, uint64_t xq, uint64_t xs);

/* ---- expert-parallel exchange over NVLink peer memory ----
 * One-shot all-reduce of bf16 rows: out[i] = bf16(sum over ranks r = 0..world-1, in that order, of peer_data[r][i]).
 * Replaces comm_push / comm_push2_body / nv_contrib (crates/kernels/cu/comm.cu:134-279, 355-375, 559-584).
 *   peer_data[r]   device address, valid on THIS GPU, of rank r's partial buffer (n_elems bf16); entry `rank` is this
 *                  rank's own buffer, which the producing kernels of this stream have already written
 *   peer_flags[r]  device address of rank r's flag block (dsuf_ep_flag_bytes(world) bytes, zeroed once at set-up)
 *   state          this rank's own 8 zero-initialised bytes of device memory (call counter), one per flag block
 *   out            local result buffer, distinct from every partial buffer
 * The caller maps the buffers (CUDA IPC / VMM; the Python mirror uses torch's symmetric memory).  Every rank must
 * make the same sequence of calls with the same flag blocks.  A partial buffer may be rewritten only after a LATER
 * call on this rank has returned on the stream (alternate two buffers, as the layer stack does).  Waits are
 * bounded: a missing peer ends in DSUF_DEVERR_WAIT_TIMEOUT in the status word, not in a hang.
 * world <= 8; n_elems % 8 == 0.  Safe to capture in a CUDA graph (the epoch lives in `state`). */
size_t dsuf_ep_flag_bytes(int32_t world);
int32_t dsuf_ep_allreduce_bf16(dsuf_ctx* ctx, void* stream, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                               int32_t world, int64_t n_elems, uint64_t state, uint64_t out);

/* All-gather of column slices over the same buffers, flags and hand-shake: rank r has written columns
 * [r * cols / world, (r + 1) * cols / world) of every row of ITS buffer peer_data[r] (bf16 [rows][cols]); out [rows][cols]
 * receives every slice from its owner.  This is the exchange after a tensor-parallel projection whose OUTPUT is sharded
 * (each rank computes complete dot products for its columns, so nothing is summed across ranks and the result equals the
 * unsharded projection bit for bit); each rank pulls (world - 1) / world of the rows' bytes instead of world - 1 times
 * all of them.  cols % (8 * world) == 0.  The reference, tensor-parallel over K, has no counterpart (cu/comm.cu sums). */
int32_t dsuf_ep_allgather_cols_bf16(dsuf_ctx* ctx, void* stream, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                                    int32_t world, int32_t rows, int32_t cols, uint64_t state, uint64_t out);

/* Combine fused with its exchange, one kernel: dsuf_moe_unpermute's sum of every token's top-k expert rows on this
 * rank (pair_row from the plan, yrows fp32 [rows][h] from dsuf_moe_w2, optional bf16 `shared` rows added by this rank:
 * pass them on ONE rank), written into this rank's partial buffer peer_data[rank], then dsuf_ep_allreduce_bf16's
 * hand-shake and rank-ordered sum into out [t][h] bf16 (dense rows).  Replaces the nsum / src2 sum plus push of
 * comm_push (cu/comm.cu:167-180) across ranks.  Same buffer, flag, state and sequencing rules as above; h % 8 == 0. */
int32_t dsuf_ep_combine_bf16(dsuf_ctx* ctx, void* stream, uint64_t pair_row, uint64_t yrows, uint64_t shared, int32_t t,
                             int32_t topk, int32_t h, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                             int32_t world, uint64_t state, uint64_t out);
/* dsuf_ep_combine_bf16 that also leaves the result quantized for the next projection: xq [t][h] FP8 codes and xs block
 * scales (mode MX: u8 [t][h/32], DS: f32 [t][h/128]) equal to dsuf_act_quant_fp8(mode, out) bit for bit, so the layer that
 * follows starts at its GEMM.  The counterpart of the activation staging the reference's decode GEMVs run on their input
 * (quant_blocks8, cu/quantblocks.cuh:7-57) moved into the producer.  xq = xs = 0: plain combine.  h % 128 == 0. */
int32_t dsuf_ep_combine_quant_bf16(dsuf_ctx* ctx, void* stream, uint64_t pair_row, uint64_t yrows, uint64_t shared, int32_t t,
                                   int32_t topk, int32_t h, const uint64_t* peer_data, const uint64_t* peer_flags, int32_t rank,
                                   int32_t world, uint64_t state, uint64_t out, int32_t mode, uint64_t xq, uint64_t xs);

/* ---- output head.  Replaces the persistent bf16 GEMV with sampling records, gemv_bf16_persist_p4
 * (crates/kernels/cu/gemv.cu:542-689; ops::gemv with GemvOpts {persist, samp_rec, out_f32}, ops.rs:165-193). ----
 * out fp32 [m][ldo] = alpha * x [m][ldx] (bf16) . w [n][k]^T (bf16, ROW-MAJOR as in the checkpoint: no host re-tiling,
 * where the reference streams weights re-tiled by tile_bf16), m <= 16, k % 8 == 0.  With `sp` and sp->records != 0 the
 * kernel also writes, per token and per quad of 64 vocabulary rows, the 20-float record the reference's sampler merges
 * (cu/gemv.cu:651-688): [0] max z, [1] sum exp(z - max), [2] the 9th largest z, [3..10] the 8 largest z (descending),
 * [11..18] their ids as int bits (ties: lower id first), [19] unused; z = logit / temperature for rows < valid_rows
 * (0: all n) and -inf above, id = row + id_offset (a vocabulary shard's first row).  records: float
 * [m][n / 64][20]; n % 64 == 0. */
typedef struct {
    uint64_t records;
    float temperature;
    int32_t valid_rows;
    int32_t id_offset;
} dsuf_sampling_opts;
int32_t dsuf_lm_head_bf16(dsuf_ctx* ctx, void* stream, uint64_t w, int32_t n, int32_t k, uint64_t x, int32_t ldx, int32_t m,
                          float alpha, uint64_t out, int32_t ldo, const dsuf_sampling_opts* sp);

#ifdef __cplusplus
}
#endif
#endif
