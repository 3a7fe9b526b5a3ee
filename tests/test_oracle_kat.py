"""The CPU oracle against the reference's own known-answer tests (restated; the Rust tests cannot run here).

Sources: crates/model/src/formats.rs:235-272 (codec sweep, seeded FP8 32x32 round trip),
crates/engine/src/ops.rs:1671-1705 (f16 staging contract, power-of-two scale commutation).
"""
import numpy as np

import oracle


def test_e4m3_fast_equals_search_on_every_bf16_and_midpoint():
    assert oracle.lib().dsufo_kat_e4m3_sweep() == 0


def test_e4m3_decode_table():
    lut = oracle.e4m3_lut()
    assert lut[0x7e] == 448.0 and lut[0xfe] == -448.0
    assert np.isnan(lut[0x7f]) and np.isnan(lut[0xff])
    assert lut[0x01] == 2.0 ** -9 and lut[0x08] == 2.0 ** -6 and lut[0x38] == 1.0
    L = oracle.lib()
    assert L.dsufo_f32_to_e4m3(float("nan")) == 0x7f
    assert L.dsufo_f32_to_e4m3_fast(1e9) == 0x7e and L.dsufo_f32_to_e4m3_fast(-1e9) == 0xfe
    # every finite code round-trips
    for c in range(256):
        if c & 0x7f == 0x7f:
            continue
        assert L.dsufo_f32_to_e4m3_fast(float(lut[c])) == (c if c != 0x80 else 0x80)


def test_ue8m0_and_round_scale_pow2():
    L = oracle.lib()
    assert L.dsufo_e8m0_to_f32(127) == 1.0 and L.dsufo_e8m0_to_f32(130) == 8.0
    # always a power of two >= amax/qmax
    rng = np.random.default_rng(0)
    for a in np.abs(rng.standard_normal(2000)).astype(np.float32) * 10:
        s = L.dsufo_round_scale_pow2(float(a), 1.0 / 448.0)
        m, _ = np.frexp(np.float32(s))
        assert m == 0.5
        assert s >= np.float32(a) * np.float32(1.0 / 448.0)
        assert s / 2 < np.float32(a) * np.float32(1.0 / 448.0) or s / 2 == 0
    assert L.dsufo_round_scale_pow2(448.0, 1.0 / 448.0) in (1.0, 2.0)


def test_quant_fp8_b32_roundtrip_seeded():
    assert oracle.lib().dsufo_kat_fp8_b32_roundtrip(None, None, None) == 0


def test_e2m1_codec():
    lut = oracle.e2m1_lut()
    assert list(lut[:8]) == [0, 0.5, 1, 1.5, 2, 3, 4, 6]
    assert list(lut[8:]) == [-0.0, -0.5, -1, -1.5, -2, -3, -4, -6]
    L = oracle.lib()
    for c in range(16):
        if c == 8:
            continue
        assert L.dsufo_f32_to_e2m1(float(lut[c])) == c
    assert L.dsufo_f32_to_e2m1(100.0) == 7 and L.dsufo_f32_to_e2m1(-100.0) == 15
    assert L.dsufo_f32_to_e2m1(2.5) == 4   # tie 2|3 -> even code (2.0)
    assert L.dsufo_f32_to_e2m1(0.25) == 0  # tie 0|0.5 -> even code (0)
    assert L.dsufo_f32_to_e2m1(5.0) == 6   # tie 4|6 -> even code (4.0)


def test_f16_staging_contract():
    """e4m3 x 2^k is exact in f16 for k in [-15, 7] (ops.rs:1671-1690)."""
    lut = oracle.e4m3_lut().astype(np.float64)
    for k in range(-15, 8):
        v = lut * 2.0 ** k
        ok = ~np.isnan(v)
        staged = (lut.astype(np.float32) * np.float32(2.0 ** k)).astype(np.float16).astype(np.float64)
        assert (staged[ok] == v[ok]).all(), k


def test_block_partial_scales_exactly():
    """A power-of-two scale commutes with a 16-term fp32 dot product (ops.rs:1692-1705)."""
    w = np.array([0.75, -1.5, 0.5, 6.0, -0.5, 1.0, 1.5, -6.0, 0.5, 0.5, -1.5, 4.0, 0.0, 2.0, -0.5, 3.0], np.float32)
    x = np.array([448.0, -0.0625, 1.0, -2.0, 0.125, 104.0, -7.5, 0.5, 0.25, -3.0, 9.0, 0.03125, 1.0, -1.0, 5.5, -0.25], np.float32)
    for k in range(-15, 8):
        sc = np.float32(2.0 ** k)
        a = b = np.float32(0)
        for i in range(16):
            a = np.float32(a + w[i] * x[i])
            b = np.float32(b + w[i] * np.float32(x[i] * sc))
        assert b == np.float32(a * sc)


def test_act_quant_mx_properties():
    rng = np.random.default_rng(1)
    x = oracle.f32_to_bf16(rng.standard_normal((5, 256)).astype(np.float32))
    x[0, :32] = 0          # all-zero block -> floor 1e-4
    q, s = oracle.act_quant(oracle.MODE_MX, x)
    assert s.dtype == np.uint8 and s.shape == (5, 8)
    deq = oracle.dequant_fp8(oracle.MODE_MX, q, s)
    xf = oracle.bf16_to_f32(x)
    sc = np.repeat((s.astype(np.uint32) << 23).view(np.float32), 32, axis=1)
    assert (np.abs(deq - xf) <= np.abs(xf) / 16 + sc * 2.0 ** -10).all()
    assert (q[0, :32] == 0).all()
    assert s[0, 0] == ((np.float32(2.0 ** -22).view(np.uint32)) >> 23)  # 2^ceil(log2(1e-4/448)) = 2^-22
    assert np.abs(oracle.e4m3_lut()[q]).max() <= 448


def test_act_quant_ds_properties():
    rng = np.random.default_rng(2)
    x = oracle.f32_to_bf16(rng.standard_normal((3, 384)).astype(np.float32))
    x[1, 128:256] = 0
    q, s = oracle.act_quant(oracle.MODE_DS, x)
    assert s.dtype == np.float32 and s.shape == (3, 3)
    xf = oracle.bf16_to_f32(x)
    amax = np.abs(xf).reshape(3, 3, 128).max(axis=2)
    want = np.where(amax == 0, np.float32(1), amax / np.float32(448)).astype(np.float32)
    assert (s == want).all()
    # the block maximum always encodes to +-448
    assert (np.abs(oracle.e4m3_lut()[q]).reshape(3, 3, 128).max(axis=2)[amax > 0] == 448).all()
    assert (q[1, 128:256] == 0).all()


def test_gemm_fp8_matches_dequant_matmul_both_modes():
    rng = np.random.default_rng(3)
    for mode in (oracle.MODE_MX, oracle.MODE_DS):
        w = oracle.f32_to_bf16((rng.standard_normal((256, 512)) * 0.02).astype(np.float32))
        x = oracle.f32_to_bf16(rng.standard_normal((4, 512)).astype(np.float32))
        wq, ws = oracle.quant_fp8_weight(mode, w)
        xq, xs = oracle.act_quant(mode, x)
        _, out = oracle.gemm_fp8(mode, wq, ws, xq, xs)
        ref = oracle.matmul_f32(oracle.dequant_fp8(mode, wq, ws), oracle.dequant_fp8(mode, xq, xs))
        assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < 1e-5
        full = oracle.bf16_to_f32(x) @ oracle.bf16_to_f32(w).T
        assert np.linalg.norm(out - full) / np.linalg.norm(full) < 0.08  # quantization error itself


def test_gemm_fp4_matches_dequant_matmul_both_act_modes():
    rng = np.random.default_rng(4)
    w = oracle.f32_to_bf16((rng.standard_normal((128, 256)) * 0.02).astype(np.float32))
    x = oracle.f32_to_bf16(rng.standard_normal((3, 256)).astype(np.float32))
    codes, sc = oracle.quant_fp4_weight(w)
    for mode in (oracle.MODE_MX, oracle.MODE_DS):
        xq, xs = oracle.act_quant(mode, x)
        out = oracle.gemm_fp4(mode, codes, sc, xq, xs)
        ref = oracle.matmul_f32(oracle.dequant_fp4(codes, sc), oracle.dequant_fp8(mode, xq, xs))
        assert np.linalg.norm(out - ref) / np.linalg.norm(ref) < 1e-5


def test_route_ties_and_normalisation():
    scores = np.array([[0.1, 0.5, 0.5, 0.2], [0.3, 0.3, 0.3, 0.3]], np.float32)
    ids, w = oracle.route(0, scores, None, 2, route_scale=2.0)
    assert ids.tolist() == [[1, 2], [0, 1]]           # ties -> lowest id first
    assert np.allclose(w.sum(axis=1), 2.0)
    bias = np.array([10, 0, 0, 0], np.float32)        # bias affects selection only
    ids, w = oracle.route(0, scores, bias, 2)
    assert ids[0].tolist() == [0, 1]
    assert np.allclose(w[0], [0.1 / 0.6, 0.5 / 0.6])


def test_permute_plan_is_a_stable_counting_sort():
    rng = np.random.default_rng(5)
    ids = rng.integers(0, 7, size=(40, 3)).astype(np.int32)
    off, row_pair, pair_row, tiles = oracle.permute_plan(ids, 7, tile_rows=8)
    flat = ids.reshape(-1)
    assert (np.diff(off) == np.bincount(flat, minlength=7)).all()
    assert (flat[row_pair] == np.sort(flat, kind="stable")).all()
    assert (row_pair == np.argsort(flat, kind="stable")).all()
    assert (pair_row[row_pair] == np.arange(flat.size)).all()
    assert tiles[:, 2].sum() == flat.size and tiles[:, 2].max() <= 8
    for e, r0, c, _ in tiles:
        assert off[e] <= r0 and r0 + c <= off[e + 1]
    # empty input
    off, rp, pr, tiles = oracle.permute_plan(np.zeros((0, 3), np.int32), 4, 8)
    assert off.tolist() == [0] * 5 and len(tiles) == 0


def _bf16(a):
    """float32 array -> (bf16 bits as uint16, the bf16 values as float32), round to nearest even."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = ((u + 0x7fff + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return r, (r.astype(np.uint32) << 16).view(np.float32)


def test_row_sumsq_and_prenorm_quant():
    """tc_row_sumsq / tc_quant_rows with pre-normalisation (crates/kernels/cu/tcgemm.cu:300-355)."""
    rng = np.random.default_rng(5)
    xb, xf = _bf16(rng.standard_normal((5, 1024)).astype(np.float32) * 3.0)
    ss = oracle.row_sumsq(xb)
    want = (xf.astype(np.float64) ** 2).sum(axis=1)
    assert np.allclose(ss, want, rtol=2e-6)
    # weights of one and rs == 1 exactly (sumsq = K, eps = 0): the pre-normalised quantizer is the plain one
    ones = np.full(1024, 0x3f80, np.uint16)
    for mode in (oracle.MODE_MX, oracle.MODE_DS):
        q0, s0 = oracle.act_quant(mode, xb)
        q1, s1 = oracle.act_quant_prenorm(mode, xb, ones, np.full(5, 1024.0, np.float32), 0.0)
        assert (q0 == q1).all() and (s0 == s1).all()
    # general case against a numpy restatement of v = bf16(w * (x * rs)) followed by the plain quantizer
    wb, wf = _bf16(1.0 + 0.1 * rng.standard_normal(1024).astype(np.float32))
    eps = np.float32(1e-6)
    rs = np.float32(1.0) / np.sqrt(ss / np.float32(1024) + eps, dtype=np.float32)
    vb, _ = _bf16(wf[None, :] * (xf * rs[:, None]))
    for mode in (oracle.MODE_MX, oracle.MODE_DS):
        q0, s0 = oracle.act_quant(mode, vb)
        q1, s1 = oracle.act_quant_prenorm(mode, xb, wb, ss, float(eps))
        assert (q0 == q1).all() and (s0 == s1).all()


def test_sampling_records_known_answers():
    """The per-quad record of the output head (crates/kernels/cu/gemv.cu:651-688) on inputs whose answer is known:
    an ascending ramp, a tie (lower id first), rows masked by valid_rows, and the id offset of a vocabulary shard."""
    z = np.arange(128, dtype=np.float32)[None, :].copy()
    z[0, 70] = z[0, 127]                      # a tie inside the second quad: id 70 comes before id 127
    rec = oracle.sampling_records(z, temperature=2.0, valid_rows=120, id_offset=1000)
    ids = rec.view(np.int32)
    assert rec.shape == (1, 2, 20)
    assert rec[0, 0, 0] == 31.5 and np.array_equal(rec[0, 0, 3:11], np.arange(63, 55, -1) / 2.0) and rec[0, 0, 2] == 27.5
    assert np.array_equal(ids[0, 0, 11:19], 1000 + np.arange(63, 55, -1))
    assert abs(rec[0, 0, 1] - np.exp((np.arange(64) - 63) / 2.0).sum()) < 1e-4
    # second quad: rows 120..127 are masked (-inf), so the maximum is the tie's value at id 70 only
    assert rec[0, 1, 0] == 63.5 and ids[0, 1, 11] == 1070 and rec[0, 1, 4] == 119 / 2.0 and ids[0, 1, 12] == 1119
    lg = oracle.lm_head(oracle.f32_to_bf16(np.eye(64, 32, dtype=np.float32)), oracle.f32_to_bf16(np.ones((2, 32), np.float32)), alpha=0.5)
    assert lg.shape == (2, 64) and np.array_equal(lg[0, :32], np.full(32, 0.5, np.float32)) and not lg[:, 32:].any()
