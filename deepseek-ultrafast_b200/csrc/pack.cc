// Host-side weight formats of libdsuf_qmm (no GPU): quantizers for synthetic / bf16 checkpoints and the
// packers that lay quantized weights out as 128x128 tile records.
//
// Stands in for crates/model/src/formats.rs (f32_to_e4m3_fast :37-57, quant_fp8_b32 :59-84, round_scale_pow2
// :86-90, tile_fp8 :96-118, tile_fp4 :147-180, tile_sf_blocks :216-228) and crates/model/src/packing.rs
// (expert_shard gate/up interleave :224-241).  The reference keeps two images of every dense weight (an
// mma.sync fragment-ordered one and a row-major one for TMA); here one tile-record image serves both paths.
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <float.h>

#include <algorithm>
#include <thread>
#include <vector>

#include "../../include/dsuf_qmm.h"

namespace {

inline float bits_f32(uint32_t b) { float f; memcpy(&f, &b, 4); return f; }
inline uint32_t f32_bits(float f) { uint32_t b; memcpy(&b, &f, 4); return b; }
inline float bf16_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

// Round-to-nearest-even onto the e4m3 grid with saturation at 448 and NaN -> 0x7f: integer rounding of the
// fp32 bit pattern for normals, scaled integer rounding for the subnormal range.
uint8_t encode_e4m3(float x) {
    if (x != x) return 0x7f;
    const uint8_t sign = (f32_bits(x) >> 31) ? 0x80 : 0;
    const float a = fabsf(x);
    if (a >= 448.0f) return sign | 0x7e;
    if (a < 0.015625f) {                       // below 2^-6: multiples of 2^-9
        const float scaled = a * 512.0f;
        float fl = floorf(scaled);
        const float frac = scaled - fl;
        uint32_t m = (uint32_t)fl;
        if (frac > 0.5f || (frac == 0.5f && (m & 1u))) ++m;
        return sign | (uint8_t)m;
    }
    const uint32_t b = f32_bits(a);
    const uint32_t r = (b + 0x7ffffu + ((b >> 20) & 1u)) >> 20;  // keep 3 mantissa bits, ties to even
    const int e = (int)(r >> 3) - 127 + 7;
    return sign | (uint8_t)(e << 3) | (uint8_t)(r & 7u);
}

uint8_t encode_e2m1(float x) {
    static const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    if (x != x) return 7;
    const uint8_t sign = (f32_bits(x) >> 31) ? 8 : 0;
    const float a = std::min(fabsf(x), 6.0f);
    int best = 0;
    float bd = INFINITY;
    for (int c = 0; c < 8; ++c) {
        const float d = fabsf(mag[c] - a);
        if (d < bd || (d == bd && !(c & 1))) { bd = d; best = c; }
    }
    return sign | (uint8_t)best;
}

float pow2_scale(float amax, float qmax_inv) {
    const uint32_t bits = f32_bits(amax * qmax_inv);
    const int e = (int)((bits >> 23) & 0xff) - 127 + ((bits & 0x7fffffu) ? 1 : 0);
    return bits_f32((uint32_t)(e + 127) << 23);
}

template <class F>
void parallel_for(int n, F f) {
    unsigned hw = std::thread::hardware_concurrency();
    const int nt = std::max(1, std::min<int>(hw ? hw : 1, n));
    if (nt == 1) { for (int i = 0; i < n; ++i) f(i); return; }
    std::vector<std::thread> th;
    for (int t = 0; t < nt; ++t)
        th.emplace_back([=] { for (int i = t; i < n; i += nt) f(i); });
    for (auto& x : th) x.join();
}

}  // namespace

extern "C" {

int32_t dsuf_quant_fp8_weight_host(int32_t mode, const uint16_t* w, int32_t n, int32_t k, uint8_t* codes, void* scales) {
    const int blk = mode == DSUF_MODE_MX ? 32 : 128;
    if (!w || !codes || !scales || n <= 0 || k <= 0 || n % blk || k % blk) return DSUF_E_BADARG;
    const int nb = n / blk, kb = k / blk;
    parallel_for(nb, [=](int rb) {
        for (int cb = 0; cb < kb; ++cb) {
            float amax = 0.f;
            for (int r = 0; r < blk; ++r)
                for (int c = 0; c < blk; ++c) amax = std::max(amax, fabsf(bf16_f32(w[(size_t)(rb * blk + r) * k + cb * blk + c])));
            float s, inv = 0.f;
            if (mode == DSUF_MODE_MX) {
                s = pow2_scale(std::max(amax, 1e-30f), 1.0f / 448.0f);
                inv = 1.0f / s;
                ((uint8_t*)scales)[(size_t)rb * kb + cb] = (uint8_t)(f32_bits(s) >> 23);
            } else {
                s = amax == 0.f ? 1.0f : amax / 448.0f;
                ((float*)scales)[(size_t)rb * kb + cb] = s;
            }
            for (int r = 0; r < blk; ++r)
                for (int c = 0; c < blk; ++c) {
                    const size_t i = (size_t)(rb * blk + r) * k + cb * blk + c;
                    const float v = bf16_f32(w[i]);
                    codes[i] = encode_e4m3(mode == DSUF_MODE_MX ? v * inv : v / s);
                }
        }
    });
    return DSUF_OK;
}

int32_t dsuf_quant_fp4_weight_host(const uint16_t* w, int32_t n, int32_t k, uint8_t* codes, uint8_t* scales) {
    if (!w || !codes || !scales || n <= 0 || k <= 0 || k % 32) return DSUF_E_BADARG;
    const int kb = k / 32;
    parallel_for(n, [=](int r) {
        for (int b = 0; b < kb; ++b) {
            const uint16_t* wr = w + (size_t)r * k + b * 32;
            float amax = 0.f;
            for (int j = 0; j < 32; ++j) amax = std::max(amax, fabsf(bf16_f32(wr[j])));
            const float s = pow2_scale(std::max(amax, 6.0f * FLT_MIN), 1.0f / 6.0f);
            const float inv = 1.0f / s;
            scales[(size_t)r * kb + b] = (uint8_t)(f32_bits(s) >> 23);
            for (int j = 0; j < 32; j += 2) {
                const uint8_t lo = encode_e2m1(std::min(std::max(bf16_f32(wr[j]) * inv, -6.f), 6.f));
                const uint8_t hi = encode_e2m1(std::min(std::max(bf16_f32(wr[j + 1]) * inv, -6.f), 6.f));
                codes[(size_t)r * (k / 2) + b * 16 + j / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
    });
    return DSUF_OK;
}

size_t dsuf_packed_bytes(int32_t fmt, int32_t mode, int32_t n, int32_t k) {
    if (n <= 0 || k <= 0 || k % 128) return 0;
    const size_t rt = (size_t)(n + 127) / 128, kt = (size_t)k / 128;
    const size_t rec = fmt == DSUF_FMT_FP4 ? 8192 + 512 : (mode == DSUF_MODE_MX ? 16384 + 512 : 16384);
    return rt * kt * rec;
}

int32_t dsuf_pack_fp8_weight(int32_t mode, const uint8_t* codes, const void* scales, int32_t n, int32_t k, uint8_t* out) {
    if (!codes || !out || n <= 0 || k <= 0 || k % 128) return DSUF_E_BADARG;
    if (mode == DSUF_MODE_MX && (!scales || n % 32)) return DSUF_E_BADARG;
    const int rt = (n + 127) / 128, kt = k / 128;
    const size_t rec = mode == DSUF_MODE_MX ? 16384 + 512 : 16384;
    parallel_for(rt, [=](int t) {
        for (int c = 0; c < kt; ++c) {
            uint8_t* rec_p = out + ((size_t)t * kt + c) * rec;
            for (int r = 0; r < 128; ++r) {
                const int row = t * 128 + r;
                if (row < n) memcpy(rec_p + r * 128, codes + (size_t)row * k + c * 128, 128);
                else memset(rec_p + r * 128, 0, 128);
            }
            if (mode == DSUF_MODE_MX) {
                uint8_t* sf = rec_p + 16384;
                for (int r = 0; r < 128; ++r) {
                    const int row = t * 128 + r;
                    for (int b = 0; b < 4; ++b)
                        sf[(r % 32) * 16 + (r / 32) * 4 + b] =
                            row < n ? ((const uint8_t*)scales)[(size_t)(row / 32) * (k / 32) + c * 4 + b] : 127;
                }
            }
        }
    });
    return DSUF_OK;
}

int32_t dsuf_pack_fp8_weight_gate_up(const uint8_t* codes, const uint8_t* scales, int32_t n, int32_t k, uint8_t* out) {
    // FP8 MX weight [n = 2 inter][k], gate rows first, then up rows: the same 8 + 8 row interleave per 16-row group as the
    // FP4 expert packer, every row keeping the scales of the 32 x 32 block it came from
    if (!codes || !scales || !out || n <= 0 || k <= 0 || k % 128 || n % 64) return DSUF_E_BADARG;
    const int rt = (n + 127) / 128, kt = k / 128, inter = n / 2;
    const size_t rec = 16384 + 512;
    parallel_for(rt, [=](int t) {
        for (int c = 0; c < kt; ++c) {
            uint8_t* rec_p = out + ((size_t)t * kt + c) * rec;
            uint8_t* sf = rec_p + 16384;
            for (int r = 0; r < 128; ++r) {
                const int pr = t * 128 + r;
                if (pr < n) {
                    const int src = ((pr % 16) / 8 ? inter : 0) + (pr / 16) * 8 + pr % 8;
                    memcpy(rec_p + r * 128, codes + (size_t)src * k + c * 128, 128);
                    for (int b = 0; b < 4; ++b) sf[(r % 32) * 16 + (r / 32) * 4 + b] = scales[(size_t)(src / 32) * (k / 32) + c * 4 + b];
                } else {
                    memset(rec_p + r * 128, 0, 128);
                    for (int b = 0; b < 4; ++b) sf[(r % 32) * 16 + (r / 32) * 4 + b] = 127;
                }
            }
        }
    });
    return DSUF_OK;
}

int32_t dsuf_pack_fp4_weight(const uint8_t* codes, const uint8_t* scales, int32_t n, int32_t k, int32_t gate_up, uint8_t* out) {
    if (!codes || !scales || !out || n <= 0 || k <= 0 || k % 128) return DSUF_E_BADARG;
    if (gate_up && n % 16) return DSUF_E_BADARG;
    const int rt = (n + 127) / 128, kt = k / 128, inter = n / 2;
    const size_t rec = 8192 + 512;
    parallel_for(rt, [=](int t) {
        for (int c = 0; c < kt; ++c) {
            uint8_t* rec_p = out + ((size_t)t * kt + c) * rec;
            uint8_t* sf = rec_p + 8192;
            for (int r = 0; r < 128; ++r) {
                const int pr = t * 128 + r;
                int src = pr;
                if (gate_up && pr < n) src = ((pr % 16) / 8 ? inter : 0) + (pr / 16) * 8 + pr % 8;
                if (pr < n) {
                    memcpy(rec_p + r * 64, codes + (size_t)src * (k / 2) + c * 64, 64);
                    for (int b = 0; b < 4; ++b) sf[(r % 32) * 16 + (r / 32) * 4 + b] = scales[(size_t)src * (k / 32) + c * 4 + b];
                } else {
                    memset(rec_p + r * 64, 0, 64);
                    for (int b = 0; b < 4; ++b) sf[(r % 32) * 16 + (r / 32) * 4 + b] = 127;
                }
            }
        }
    });
    return DSUF_OK;
}

}  // extern "C"
