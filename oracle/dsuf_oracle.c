/*
 * dsuf_oracle.c -- CPU restatement of the quantized matrix-product path of
 * basetenlabs/deepseek-ultrafast.  TEST INFRASTRUCTURE ONLY: this file is the
 * checker for the CUDA library and the timed scalar CPU baseline.  Nothing in
 * the product library links, loads or calls it.
 *
 * Parity status: the codecs and the FP8 32x32 weight quantizer are pinned
 * against the reference's own known-answer tests (every-bf16 / midpoint sweep
 * of crates/model/src/formats.rs:235-248, the seeded round-trip bound of
 * formats.rs:250-272, the f16 staging contract and power-of-two commutation of
 * crates/engine/src/ops.rs:1671-1705).  The reference holds no golden GEMM or
 * MoE outputs; in the MX geometry the quantizers, the router, the permute
 * plan, the dense GEMV / GEMM outputs and the prefill expert GEMMs (gate/up +
 * SwiGLU + re-quantization, down) of this file are instead pinned by the
 * reference's own sm_100a kernels executed on the GPU (oracle/refkernels.py,
 * tests/test_ref_kernels.py).  The DS geometry is defined by the benchmark
 * configuration, not by reference source, and is pinned by formula only.
 *
 * Two quantization geometries are restated:
 *   MX  (what the reference source implements): activations 1x32 with a
 *       power-of-two scale 2^ceil(log2(amax/448)), amax floored at 1e-4
 *       (crates/kernels/cu/quantblocks.cuh:7-57, cu/tcgemm.cu:300-340);
 *       FP8 weights 32x32 with UE8M0 scales (formats.rs:59-84).
 *   DS  (what the benchmark configurations specify): activations 1x128 with
 *       fp32 scale = amax/448 (IEEE division; amax==0 -> scale 1), codes
 *       rne_e4m3(x/scale) with IEEE fp32 division; FP8 weights 128x128 with the
 *       same rule.  Accumulation: fp32, ascending k inside a 128-block, then
 *       acc += partial * sa * sw.
 * MXFP4 expert weights: e2m1 codes, two per byte, low nibble = even k, UE8M0
 * scale per 1x32 along K (crates/model/src/packing.rs:11-17); the synthetic
 * quantizer follows the reference's own FP4 rule (cu/kv_fp4.cu:25-32).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <float.h>

#define DSUFO_MODE_MX 0
#define DSUFO_MODE_DS 1

static inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
static inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }

float dsufo_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* round-to-nearest-even f32 -> bf16, NaN kept quiet (what `half::bf16::from_f32` and
 * the device `__float2bfloat16` both do). */
uint16_t dsufo_f32_to_bf16(float f) {
    uint32_t b = f32_bits(f);
    if ((b & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((b >> 16) | 0x40);
    b += 0x7fffu + ((b >> 16) & 1u);
    return (uint16_t)(b >> 16);
}
static inline float bf16r(float f) { return dsufo_bf16_to_f32(dsufo_f32_to_bf16(f)); }

/* ---- codecs: crates/model/src/formats.rs:4-57 ---- */
float dsufo_e4m3_to_f32(uint8_t b) {
    float s = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0xf;
    float m = (float)(b & 7);
    if (e == 0xf && (b & 7) == 7) return NAN;
    if (e == 0) return s * m / 8.0f * ldexpf(1.0f, -6);
    return s * (1.0f + m / 8.0f) * ldexpf(1.0f, e - 7);
}

float dsufo_e8m0_to_f32(uint8_t b) { return bits_f32((uint32_t)b << 23); }

/* nearest-value search, ties to the even code: formats.rs:18-35 */
uint8_t dsufo_f32_to_e4m3(float x) {
    if (isnan(x)) return 0x7f;
    uint8_t s = signbit(x) ? 0x80 : 0;
    float a = fminf(fabsf(x), 448.0f);
    uint8_t best = 0;
    float bd = INFINITY;
    for (int c = 0; c <= 0x7e; ++c) {
        float d = fabsf(dsufo_e4m3_to_f32((uint8_t)c) - a);
        if (d < bd || (d == bd && (c & 1) == 0)) { bd = d; best = (uint8_t)c; }
    }
    return s | best;
}

/* bit-trick encoder: formats.rs:37-57 */
uint8_t dsufo_f32_to_e4m3_fast(float x) {
    if (isnan(x)) return 0x7f;
    uint8_t s = signbit(x) ? 0x80 : 0;
    float a = fabsf(x);
    if (a >= 448.0f) return s | 0x7e;
    if (a < 0.015625f) {
        float q = a * 512.0f, f = floorf(q), d = q - f;
        uint32_t fi = (uint32_t)f;
        uint32_t m = (d > 0.5f || (d == 0.5f && (fi & 1))) ? fi + 1 : fi;
        return s | (uint8_t)m;
    }
    uint32_t b = f32_bits(a);
    uint32_t r = (b + 0x7ffffu + ((b >> 20) & 1u)) >> 20;
    int e = (int)(r >> 3) - 127 + 7;
    return s | (uint8_t)(e << 3) | (uint8_t)(r & 7);
}

/* e2m1: bit3 sign, magnitudes {0,.5,1,1.5,2,3,4,6}; encode = nearest, ties to the even code,
 * saturating at 6 (device twin: cvt.rn.satfinite.e2m1x2.f32, cu/rope.cuh:9-14). */
static const float E2M1_MAG[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
float dsufo_e2m1_to_f32(uint8_t c) { float v = E2M1_MAG[c & 7]; return (c & 8) ? -v : v; }
uint8_t dsufo_f32_to_e2m1(float x) {
    if (isnan(x)) return 0x7;
    uint8_t s = signbit(x) ? 8 : 0;
    float a = fminf(fabsf(x), 6.0f);
    int best = 0;
    float bd = INFINITY;
    for (int c = 0; c < 8; ++c) {
        float d = fabsf(E2M1_MAG[c] - a);
        if (d < bd || (d == bd && (c & 1) == 0)) { bd = d; best = c; }
    }
    return s | (uint8_t)best;
}

/* formats.rs:86-90, cu/common.cuh:80-84 */
float dsufo_round_scale_pow2(float amax, float qmax_inv) {
    uint32_t bits = f32_bits(amax * qmax_inv);
    int e = (int)((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) ? 1 : 0);
    return bits_f32((uint32_t)(e + 127) << 23);
}

/* ---- activation quantizer ----
 * MX: cu/tcgemm.cu:325-338 (amax floor 1e-4, pow2 scale, exact reciprocal by exponent flip).
 *     scales: UE8M0 bytes [m][k/32].
 * DS: 1x128, scale = amax/448 (1 when the block is all zero), code = rne(x/scale).
 *     scales: fp32 [m][k/128].
 * x is bf16 [m][ldx]; q is [m][k]. */
void dsufo_act_quant(int mode, const uint16_t* x, int ldx, int m, int k, uint8_t* q, void* scales) {
    const int blk = mode == DSUFO_MODE_MX ? 32 : 128;
    const int nkb = k / blk;
    for (int r = 0; r < m; ++r)
        for (int kb = 0; kb < nkb; ++kb) {
            const uint16_t* xr = x + (size_t)r * ldx + (size_t)kb * blk;
            float amax = 0.f;
            for (int j = 0; j < blk; ++j) amax = fmaxf(amax, fabsf(dsufo_bf16_to_f32(xr[j])));
            uint8_t* qo = q + (size_t)r * k + (size_t)kb * blk;
            if (mode == DSUFO_MODE_MX) {
                float sc = dsufo_round_scale_pow2(fmaxf(amax, 1e-4f), 1.0f / 448.0f);
                float inv = bits_f32(0x7f000000u - f32_bits(sc));
                for (int j = 0; j < blk; ++j) qo[j] = dsufo_f32_to_e4m3_fast(dsufo_bf16_to_f32(xr[j]) * inv);
                ((uint8_t*)scales)[(size_t)r * nkb + kb] = (uint8_t)((f32_bits(sc) >> 23) & 0xff);
            } else {
                float sc = amax == 0.f ? 1.0f : amax / 448.0f;
                for (int j = 0; j < blk; ++j) qo[j] = dsufo_f32_to_e4m3_fast(dsufo_bf16_to_f32(xr[j]) / sc);
                ((float*)scales)[(size_t)r * nkb + kb] = sc;
            }
        }
}

/* ---- RMS pre-normalisation in front of the activation quantizer ----
 * tc_row_sumsq (crates/kernels/cu/tcgemm.cu:341-355): one warp per row; lane l accumulates x[k]^2 for
 * k = 8 l + 256 i + e (e inner, fused multiply-add), then a 16, 8, 4, 2, 1 xor butterfly (cu/common.cuh:86-90).
 * The summation order is restated exactly, so the fp32 result is bit-identical to the CUDA path's. */
void dsufo_row_sumsq(const uint16_t* x, int ldx, int m, int k, float* out) {
    for (int r = 0; r < m; ++r) {
        float lane[32], tmp[32];
        for (int l = 0; l < 32; ++l) {
            float ss = 0.f;
            for (int kk = l * 8; kk < k; kk += 256)
                for (int e = 0; e < 8; ++e) {
                    const float v = dsufo_bf16_to_f32(x[(size_t)r * ldx + kk + e]);
                    ss = fmaf(v, v, ss);
                }
            lane[l] = ss;
        }
        for (int o = 16; o > 0; o >>= 1) {
            for (int l = 0; l < 32; ++l) tmp[l] = lane[l] + lane[l ^ o];
            memcpy(lane, tmp, sizeof(lane));
        }
        out[r] = lane[0];
    }
}

/* tc_quant_rows with pw != null (cu/tcgemm.cu:300-340): v = bf16(w * (x * rs)), rs = 1 / sqrt(sumsq / K + eps),
 * then the quantizer above.  The reference evaluates rs with rsqrtf, an approximate instruction (2 ulp); this
 * restatement and the CUDA path both use the correctly rounded square root and division, so they agree bit for bit
 * with each other and differ from the reference's rs by at most that approximation error. */
void dsufo_act_quant_prenorm(int mode, const uint16_t* x, int ldx, int m, int k, const uint16_t* norm_w, const float* sumsq,
                             float eps, uint8_t* q, void* scales) {
    const int blk = mode == DSUFO_MODE_MX ? 32 : 128;
    uint16_t* v = (uint16_t*)malloc(sizeof(uint16_t) * (size_t)k);
    for (int r = 0; r < m; ++r) {
        const float rs = 1.0f / sqrtf(sumsq[r] / (float)k + eps);
        for (int c = 0; c < k; ++c) {
            const float xr = dsufo_bf16_to_f32(x[(size_t)r * ldx + c]) * rs;
            v[c] = dsufo_f32_to_bf16(dsufo_bf16_to_f32(norm_w[c]) * xr);
        }
        dsufo_act_quant(mode, v, k, 1, k, q + (size_t)r * k,
                        (uint8_t*)scales + (size_t)r * (k / blk) * (mode == DSUFO_MODE_MX ? 1 : 4));
    }
    free(v);
}

/* ---- FP8 weight quantizers ----
 * MX: formats.rs:59-84 (32x32 blocks, amax floor 1e-30, inv = 1/s). scales u8 [n/32][k/32].
 * DS: 128x128 blocks, fp32 amax/448. scales f32 [n/128][k/128]. */
void dsufo_quant_fp8_weight(int mode, const uint16_t* w, int n, int k, uint8_t* q, void* scales) {
    const int blk = mode == DSUFO_MODE_MX ? 32 : 128;
    const int nb = n / blk, kb = k / blk;
#pragma omp parallel for collapse(2) schedule(static)
    for (int rb = 0; rb < nb; ++rb)
        for (int cb = 0; cb < kb; ++cb) {
            float amax = 0.f;
            for (int r = 0; r < blk; ++r)
                for (int c = 0; c < blk; ++c)
                    amax = fmaxf(amax, fabsf(dsufo_bf16_to_f32(w[(size_t)(rb * blk + r) * k + cb * blk + c])));
            float s, inv = 0.f;
            if (mode == DSUFO_MODE_MX) {
                s = dsufo_round_scale_pow2(fmaxf(amax, 1e-30f), 1.0f / 448.0f);
                inv = 1.0f / s;
                ((uint8_t*)scales)[(size_t)rb * kb + cb] = (uint8_t)(f32_bits(s) >> 23);
            } else {
                s = amax == 0.f ? 1.0f : amax / 448.0f;
                ((float*)scales)[(size_t)rb * kb + cb] = s;
            }
            for (int r = 0; r < blk; ++r)
                for (int c = 0; c < blk; ++c) {
                    size_t i = (size_t)(rb * blk + r) * k + cb * blk + c;
                    float v = dsufo_bf16_to_f32(w[i]);
                    q[i] = dsufo_f32_to_e4m3_fast(mode == DSUFO_MODE_MX ? v * inv : v / s);
                }
        }
}

/* MXFP4 weight quantizer (synthetic weights only; real checkpoints arrive quantized).
 * Rule of cu/kv_fp4.cu:25-32: scale = round_scale_pow2(max(amax, 6*FLT_MIN), 1/6),
 * code = rn_e2m1(clamp(x/scale, +-6)).  codes [n][k/2], low nibble = even k; scales u8 [n][k/32]. */
void dsufo_quant_fp4_weight(const uint16_t* w, int n, int k, uint8_t* codes, uint8_t* scales) {
    const int kb = k / 32;
#pragma omp parallel for schedule(static)
    for (int r = 0; r < n; ++r)
        for (int b = 0; b < kb; ++b) {
            const uint16_t* wr = w + (size_t)r * k + b * 32;
            float amax = 0.f;
            for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(dsufo_bf16_to_f32(wr[j])));
            float s = dsufo_round_scale_pow2(fmaxf(amax, 6.0f * FLT_MIN), 1.0f / 6.0f);
            float inv = 1.0f / s;
            scales[(size_t)r * kb + b] = (uint8_t)(f32_bits(s) >> 23);
            for (int j = 0; j < 32; j += 2) {
                uint8_t lo = dsufo_f32_to_e2m1(fminf(fmaxf(dsufo_bf16_to_f32(wr[j]) * inv, -6.f), 6.f));
                uint8_t hi = dsufo_f32_to_e2m1(fminf(fmaxf(dsufo_bf16_to_f32(wr[j + 1]) * inv, -6.f), 6.f));
                codes[(size_t)r * (k / 2) + b * 16 + j / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
}

/* ---- dequantize-then-matmul, FP8 weights ----
 * out[m][n] = alpha * sum_kb  sw[n/B][kb] * sa[m][kb'] * sum_{k in block} e4m3(w) * e4m3(x)
 * MX follows cu/gemv.cu:354-369 (32-K partial in fp32, then fmaf(partial, scale, acc)).
 * out_bf16 and out_f32 are both optional. */
static float E4M3_LUT[256];
static int lut_ready = 0;
static void init_lut(void) {
    if (lut_ready) return;
    for (int i = 0; i < 256; ++i) E4M3_LUT[i] = dsufo_e4m3_to_f32((uint8_t)i);
    lut_ready = 1;
}

void dsufo_gemm_fp8(int mode, const uint8_t* wq, const void* ws, int n, int k, const uint8_t* xq, const void* xs, int m,
                    float alpha, uint16_t* out_bf16, float* out_f32, int ldo) {
    init_lut();
    const int blk = mode == DSUFO_MODE_MX ? 32 : 128;
    const int nkb = k / blk;
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c)
        for (int r = 0; r < m; ++r) {
            float acc = 0.f;
            for (int kb = 0; kb < nkb; ++kb) {
                float part = 0.f;
                const uint8_t* wp = wq + (size_t)c * k + kb * blk;
                const uint8_t* xp = xq + (size_t)r * k + kb * blk;
                for (int j = 0; j < blk; ++j) part += E4M3_LUT[wp[j]] * E4M3_LUT[xp[j]];
                float sc;
                if (mode == DSUFO_MODE_MX)
                    sc = dsufo_e8m0_to_f32(((const uint8_t*)ws)[(size_t)(c / 32) * nkb + kb]) *
                         dsufo_e8m0_to_f32(((const uint8_t*)xs)[(size_t)r * nkb + kb]);
                else
                    sc = ((const float*)ws)[(size_t)(c / 128) * nkb + kb] * ((const float*)xs)[(size_t)r * nkb + kb];
                acc = fmaf(part, sc, acc);
            }
            acc *= alpha;
            if (out_bf16) out_bf16[(size_t)r * ldo + c] = dsufo_f32_to_bf16(acc);
            if (out_f32) out_f32[(size_t)r * ldo + c] = acc;
        }
}

/* ---- dequantize-then-matmul, MXFP4 weights x FP8 activations (cu/gemv.cu:370-396) ----
 * codes [n][k/2], wscale u8 [n][k/32]; activations in either geometry.
 * out_f32[m][ldo] = sum over 32-K blocks of  ws * sa * sum e2m1(w)*e4m3(x). */
void dsufo_gemm_fp4(int act_mode, const uint8_t* codes, const uint8_t* wscale, int n, int k, const uint8_t* xq,
                    const void* xs, int m, float* out_f32, int ldo) {
    init_lut();
    const int kb32 = k / 32;
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c)
        for (int r = 0; r < m; ++r) {
            float acc = 0.f;
            if (act_mode == DSUFO_MODE_MX) {
                for (int b = 0; b < kb32; ++b) {
                    float part = 0.f;
                    for (int j = 0; j < 32; ++j) {
                        uint8_t by = codes[(size_t)c * (k / 2) + b * 16 + j / 2];
                        part += dsufo_e2m1_to_f32((j & 1) ? (by >> 4) : (by & 15)) * E4M3_LUT[xq[(size_t)r * k + b * 32 + j]];
                    }
                    float sc = dsufo_e8m0_to_f32(wscale[(size_t)c * kb32 + b]) *
                               dsufo_e8m0_to_f32(((const uint8_t*)xs)[(size_t)r * kb32 + b]);
                    acc = fmaf(part, sc, acc);
                }
            } else {
                for (int B = 0; B < k / 128; ++B) {
                    float tile = 0.f;
                    for (int b = 4 * B; b < 4 * B + 4; ++b) {
                        float part = 0.f;
                        for (int j = 0; j < 32; ++j) {
                            uint8_t by = codes[(size_t)c * (k / 2) + b * 16 + j / 2];
                            part += dsufo_e2m1_to_f32((j & 1) ? (by >> 4) : (by & 15)) * E4M3_LUT[xq[(size_t)r * k + b * 32 + j]];
                        }
                        tile = fmaf(part, dsufo_e8m0_to_f32(wscale[(size_t)c * kb32 + b]), tile);
                    }
                    acc = fmaf(tile, ((const float*)xs)[(size_t)r * (k / 128) + B], acc);
                }
            }
            out_f32[(size_t)r * ldo + c] = acc;
        }
}

/* ---- router: cu/route.cuh:3-56 ----
 * score_fn 0: scores used as given; 1: softmax over the expert axis (benchmark configs);
 * 2: sqrt(softplus(x)) (cu/common.cuh:17-24).  Selection key = score + bias, ties -> lowest id;
 * weight = score / (sum of selected scores + 1e-20) when topk > 1, times route_scale. */
void dsufo_route(int score_fn, const float* scores, const float* bias, int t, int n_exp, int topk, float route_scale,
                 int32_t* ids, float* w) {
    float* sc = (float*)malloc(sizeof(float) * n_exp);
    float* key = (float*)malloc(sizeof(float) * n_exp);
    for (int m = 0; m < t; ++m) {
        const float* s = scores + (size_t)m * n_exp;
        if (score_fn == 1) {
            float mx = -INFINITY, sum = 0.f;
            for (int e = 0; e < n_exp; ++e) mx = fmaxf(mx, s[e]);
            for (int e = 0; e < n_exp; ++e) { sc[e] = expf(s[e] - mx); sum += sc[e]; }
            for (int e = 0; e < n_exp; ++e) sc[e] = sc[e] / sum;
        } else if (score_fn == 2) {
            for (int e = 0; e < n_exp; ++e) sc[e] = sqrtf(s[e] > 20.f ? s[e] : log1pf(expf(s[e])));
        } else {
            for (int e = 0; e < n_exp; ++e) sc[e] = s[e];
        }
        for (int e = 0; e < n_exp; ++e) key[e] = sc[e] + (bias ? bias[e] : 0.f);
        float wsum = 0.f;
        for (int j = 0; j < topk; ++j) {
            int bi = -1;
            for (int e = 0; e < n_exp; ++e)
                if (key[e] != -INFINITY && (bi < 0 || key[e] > key[bi])) bi = e;
            if (bi < 0) bi = 0;
            ids[(size_t)m * topk + j] = bi;
            w[(size_t)m * topk + j] = sc[bi];
            wsum += sc[bi];
            key[bi] = -INFINITY;
        }
        for (int j = 0; j < topk; ++j) {
            float v = w[(size_t)m * topk + j];
            if (topk > 1) v = v / (wsum + 1e-20f);
            w[(size_t)m * topk + j] = v * route_scale;
        }
    }
    free(sc);
    free(key);
}

/* ---- permute plan: cu/tcmoe.cu:19-69 ----
 * Counting sort of the P = t*topk (token, expert) pairs by expert.  The reference fills rows of one
 * expert in atomicAdd order (nondeterministic); here rows of an expert are in ascending pair index.
 * expert_off[n_exp+1], row_pair[P] (pair of permuted row), pair_row[P] (inverse),
 * tiles[4*i] = (expert, first_row, count<=tile_rows, 0), returns number of tiles. */
int dsufo_permute_plan(const int32_t* ids, int p, int n_exp, int tile_rows, int32_t* expert_off, int32_t* row_pair,
                       int32_t* pair_row, int32_t* tiles) {
    int32_t* cnt = (int32_t*)calloc(n_exp + 1, sizeof(int32_t));
    for (int i = 0; i < p; ++i) cnt[ids[i]]++;
    expert_off[0] = 0;
    for (int e = 0; e < n_exp; ++e) expert_off[e + 1] = expert_off[e] + cnt[e];
    memset(cnt, 0, sizeof(int32_t) * n_exp);
    for (int i = 0; i < p; ++i) {
        int e = ids[i], r = expert_off[e] + cnt[e]++;
        row_pair[r] = i;
        pair_row[i] = r;
    }
    int nt = 0;
    for (int e = 0; e < n_exp; ++e)
        for (int r0 = expert_off[e]; r0 < expert_off[e + 1]; r0 += tile_rows) {
            int c = expert_off[e + 1] - r0;
            if (tiles) { tiles[4 * nt] = e; tiles[4 * nt + 1] = r0; tiles[4 * nt + 2] = c < tile_rows ? c : tile_rows; tiles[4 * nt + 3] = 0; }
            ++nt;
        }
    free(cnt);
    return nt;
}

/* ---- whole routed-expert layer ----
 * x bf16 [t][h]; ids/w [t][topk]; w13 codes [n_exp][2*inter][h/2] (rows 0..inter-1 gate, inter..2*inter-1 up),
 * w13 scales [n_exp][2*inter][h/32]; w2 codes [n_exp][h][inter/2], scales [n_exp][h][inter/32].
 * Steps (cu/gemv.cu:470-483,1619-1640; cu/comm.cu:167-180):
 *   xq = act_quant(x[t]);  g = bf16(gate.xq), u = bf16(up.xq);
 *   if L > 0: u = clamp(u, +-L), g = min(g, L);  a = bf16(g/(1+exp(-g)) * u * w_route);
 *   aq = act_quant(a);  ypair[p] = w2 . aq  (fp32);  y[t] = bf16(sum_j ypair[t*topk+j] (+ shared[t])).
 * Optional outputs (may be NULL): act_bf16 [P][inter], ypair [P][h].
 * Only experts with id in [e_lo, e_hi) are evaluated (expert-parallel shard); other pairs add 0. */
void dsufo_moe_layer(int act_mode, const uint16_t* x, int t, int h, int inter, int topk, const int32_t* ids,
                     const float* w, const uint8_t* w13c, const uint8_t* w13s, const uint8_t* w2c, const uint8_t* w2s,
                     float swiglu_limit, const uint16_t* shared, int e_lo, int e_hi, uint16_t* y_bf16, float* y_f32,
                     uint16_t* act_bf16, float* ypair_out) {
    init_lut();
    const int blk = act_mode == DSUFO_MODE_MX ? 32 : 128;
    const int P = t * topk;
    uint8_t* xq = (uint8_t*)malloc((size_t)t * h);
    void* xs = malloc((size_t)t * (h / blk) * 4);
    dsufo_act_quant(act_mode, x, h, t, h, xq, xs);
    const size_t xs_el = act_mode == DSUFO_MODE_MX ? 1 : 4;
    float* ypair = (float*)calloc((size_t)P * h, sizeof(float));
#pragma omp parallel
    {
        float* gu = (float*)malloc(sizeof(float) * 2 * inter);
        uint16_t* a = (uint16_t*)malloc(sizeof(uint16_t) * inter);
        uint8_t* aq = (uint8_t*)malloc(inter);
        void* as = malloc((size_t)(inter / blk) * 4);
#pragma omp for schedule(dynamic, 1)
        for (int p = 0; p < P; ++p) {
            const int tok = p / topk, e = ids[p];
            if (e < e_lo || e >= e_hi) {
                if (act_bf16) memset(act_bf16 + (size_t)p * inter, 0, sizeof(uint16_t) * inter);
                continue;
            }
            dsufo_gemm_fp4(act_mode, w13c + (size_t)e * 2 * inter * (h / 2), w13s + (size_t)e * 2 * inter * (h / 32),
                           2 * inter, h, xq + (size_t)tok * h, (const uint8_t*)xs + (size_t)tok * (h / blk) * xs_el, 1, gu,
                           2 * inter);
            for (int i = 0; i < inter; ++i) {
                float g = bf16r(gu[i]), u = bf16r(gu[inter + i]);
                if (swiglu_limit > 0.f) { u = fminf(fmaxf(u, -swiglu_limit), swiglu_limit); g = fminf(g, swiglu_limit); }
                a[i] = dsufo_f32_to_bf16(g / (1.0f + expf(-g)) * u * w[p]);
            }
            if (act_bf16) memcpy(act_bf16 + (size_t)p * inter, a, sizeof(uint16_t) * inter);
            dsufo_act_quant(act_mode, a, inter, 1, inter, aq, as);
            dsufo_gemm_fp4(act_mode, w2c + (size_t)e * h * (inter / 2), w2s + (size_t)e * h * (inter / 32), h, inter, aq, as,
                           1, ypair + (size_t)p * h, h);
        }
        free(gu); free(a); free(aq); free(as);
    }
    for (int tok = 0; tok < t; ++tok)
        for (int c = 0; c < h; ++c) {
            float s = 0.f;
            for (int j = 0; j < topk; ++j) s += ypair[(size_t)(tok * topk + j) * h + c];
            if (shared) s += dsufo_bf16_to_f32(shared[(size_t)tok * h + c]);
            if (y_bf16) y_bf16[(size_t)tok * h + c] = dsufo_f32_to_bf16(s);
            if (y_f32) y_f32[(size_t)tok * h + c] = s;
        }
    if (ypair_out) memcpy(ypair_out, ypair, sizeof(float) * (size_t)P * h);
    free(xq); free(xs); free(ypair);
}

/* fp32 "dequantize then matmul" without any blocking of the accumulation: the looser reference that the
 * 1e-2 relative-Frobenius tolerance is stated against. w_deq [n][k], x_deq [m][k] already dequantized. */
void dsufo_matmul_f32(const float* w_deq, const float* x_deq, int n, int k, int m, float* out) {
#pragma omp parallel for schedule(static)
    for (int c = 0; c < n; ++c)
        for (int r = 0; r < m; ++r) {
            double acc = 0.0;
            for (int j = 0; j < k; ++j) acc += (double)w_deq[(size_t)c * k + j] * (double)x_deq[(size_t)r * k + j];
            out[(size_t)r * n + c] = (float)acc;
        }
}

int dsufo_num_threads(void) {
#ifdef _OPENMP
    extern int omp_get_max_threads(void);
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* The timed CPU baseline wants every host core even when the launcher exported OMP_NUM_THREADS=1 (torch.distributed.run
 * does): n <= 0 leaves the setting alone.  Returns the thread count in force. */
int dsufo_set_num_threads(int n) {
#ifdef _OPENMP
    extern void omp_set_num_threads(int);
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
    return dsufo_num_threads();
}

/* ---- known-answer sweeps restated from the reference's own unit tests ---- */

/* formats.rs:235-248: the bit-trick encoder equals the nearest-value search on every bf16 value, on two
 * perturbations of each, and on every midpoint between adjacent codes.  Returns the number of mismatches. */
int dsufo_kat_e4m3_sweep(void) {
    int bad = 0;
    for (uint32_t bits = 0; bits <= 0xffff; ++bits) {
        float x = dsufo_bf16_to_f32((uint16_t)bits);
        float v[3] = {x, bits_f32(f32_bits(x) + 0x8000u), bits_f32(f32_bits(x) + 0x4321u)};
        for (int i = 0; i < 3; ++i) bad += dsufo_f32_to_e4m3_fast(v[i]) != dsufo_f32_to_e4m3(v[i]);
    }
    for (int c = 0; c < 0x7e; ++c) {
        float mid = (dsufo_e4m3_to_f32((uint8_t)c) + dsufo_e4m3_to_f32((uint8_t)(c + 1))) / 2.0f;
        bad += dsufo_f32_to_e4m3_fast(mid) != dsufo_f32_to_e4m3(mid);
        bad += dsufo_f32_to_e4m3_fast(-mid) != dsufo_f32_to_e4m3(-mid);
    }
    return bad;
}

/* formats.rs:250-272: xorshift64 matrix (seed 0x9e3779b97f4a7c15, 64x96, every 97th value large),
 * quantized 32x32, dequantized error bound |x|/16 + sc*2^-10.  Writes the generated bf16 matrix to w
 * (64*96) when non-NULL; returns the number of violations. */
int dsufo_kat_fp8_b32_roundtrip(uint16_t* w_out, uint8_t* q_out, uint8_t* s_out) {
    enum { N = 64, K = 96 };
    static uint16_t w[N * K];
    static uint8_t q[N * K], s[(N / 32) * (K / 32)];
    uint64_t seed = 0x9e3779b97f4a7c15ull;
    for (int i = 0; i < N * K; ++i) {
        seed ^= seed << 13; seed ^= seed >> 7; seed ^= seed << 17;
        float v = ((float)(seed >> 40) / (float)(1ull << 24) - 0.5f) * (i % 97 == 0 ? 40.0f : 0.1f);
        w[i] = dsufo_f32_to_bf16(v);
    }
    dsufo_quant_fp8_weight(DSUFO_MODE_MX, w, N, K, q, s);
    int bad = 0;
    for (int r = 0; r < N; ++r)
        for (int c = 0; c < K; ++c) {
            float x = dsufo_bf16_to_f32(w[r * K + c]);
            float sc = dsufo_e8m0_to_f32(s[(r / 32) * (K / 32) + c / 32]);
            float y = dsufo_e4m3_to_f32(q[r * K + c]) * sc;
            bad += !(fabsf(x - y) <= fabsf(x) / 16.0f + sc * ldexpf(1.0f, -10));
        }
    if (w_out) memcpy(w_out, w, sizeof(w));
    if (q_out) memcpy(q_out, q, sizeof(q));
    if (s_out) memcpy(s_out, s, sizeof(s));
    return bad;
}
