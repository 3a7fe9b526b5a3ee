"""Host side of libdsuf_qmm without a GPU: the library loads, exports every symbol the header declares, its host
quantizers agree bit-for-bit with the oracle, and the tile-record packers put every byte where the kernels read it."""
import ctypes
import os
import re

import numpy as np

import oracle
from conftest import ROOT


def test_library_exports_every_declared_symbol(pkg):
    hdr = open(os.path.join(ROOT, "include", "dsuf_qmm.h")).read()
    declared = set(re.findall(r"\b(dsuf_[a-z0-9_]+)\s*\(", hdr))
    declared -= {"dsuf_weight_desc", "dsuf_moe_plan", "dsuf_dev_status"}
    assert len(declared) >= 20
    L = ctypes.CDLL(pkg.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} declared in include/dsuf_qmm.h but not exported"
    assert declared == set(pkg.ABI), declared ^ set(pkg.ABI)


def test_bad_arguments_are_rejected_without_a_gpu(pkg):
    L = pkg.lib()
    assert L.dsuf_packed_bytes(pkg.FMT_FP8, pkg.MODE_DS, 128, 100) == 0          # k not a multiple of 128
    assert L.dsuf_pack_fp8_weight(pkg.MODE_MX, None, None, 128, 128, None) == -1
    assert L.dsuf_quant_fp8_weight_host(pkg.MODE_MX, None, 32, 32, None, None) == -1
    assert L.dsuf_ctx_destroy(None) == 0
    assert L.dsuf_moe_plan_scratch_ints(0, 4) >= 4


def test_host_quantizers_match_oracle_bit_for_bit(pkg):
    rng = np.random.default_rng(0)
    w = oracle.f32_to_bf16((rng.standard_normal((256, 384)) * 0.02).astype(np.float32))
    w[0:32, 0:32] = 0                      # an all-zero block
    w[40, 40] = oracle.f32_to_bf16(np.array([3.0], np.float32))[0]   # an outlier
    for mode in (pkg.MODE_MX, pkg.MODE_DS):
        q, s = pkg.quant_fp8_weight_host(mode, w)
        qo, so = oracle.quant_fp8_weight(mode, w)
        assert (q == qo).all() and (s == so).all()
    c, s = pkg.quant_fp4_weight_host(w)
    co, so = oracle.quant_fp4_weight(w)
    assert (c == co).all() and (s == so).all()


def test_reference_roundtrip_fixture_through_the_library(pkg):
    """The reference's seeded 64x96 matrix (formats.rs:250-272) quantized by the library equals the oracle's."""
    w = np.empty(64 * 96, np.uint16)
    q = np.empty(64 * 96, np.uint8)
    s = np.empty(6, np.uint8)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    assert oracle.lib().dsufo_kat_fp8_b32_roundtrip(p(w), p(q), p(s)) == 0
    ql, sl = pkg.quant_fp8_weight_host(pkg.MODE_MX, w.reshape(64, 96))
    assert (ql.reshape(-1) == q).all() and (sl.reshape(-1) == s).all()


def test_fp8_tile_records(pkg):
    rng = np.random.default_rng(1)
    n, k = 200, 256                         # n is padded to 256
    codes = rng.integers(0, 256, (n, k), dtype=np.uint8)
    # MX needs n % 32 == 0
    n_mx = 224
    codes_mx = rng.integers(0, 256, (n_mx, k), dtype=np.uint8)
    sc = rng.integers(100, 140, (n_mx // 32, k // 32), dtype=np.uint8)
    img = pkg.pack_fp8_weight(pkg.MODE_MX, codes_mx, sc)
    rec = 16384 + 512
    assert img.size == 2 * 2 * rec
    for rt in range(2):
        for kt in range(2):
            r = img[(rt * 2 + kt) * rec:(rt * 2 + kt + 1) * rec]
            tile = r[:16384].reshape(128, 128)
            rows = min(128, n_mx - rt * 128)
            assert (tile[:rows] == codes_mx[rt * 128:rt * 128 + rows, kt * 128:(kt + 1) * 128]).all()
            assert (tile[rows:] == 0).all()
            sf = r[16384:]
            for row in range(128):
                for b in range(4):
                    want = sc[(rt * 128 + row) // 32, kt * 4 + b] if rt * 128 + row < n_mx else 127
                    assert sf[(row % 32) * 16 + (row // 32) * 4 + b] == want
    img = pkg.pack_fp8_weight(pkg.MODE_DS, codes, None)
    assert img.size == 2 * 2 * 16384
    assert (img[16384 * 3:].reshape(128, 128)[:72] == codes[128:, 128:]).all()


def test_fp4_tile_records_and_gate_up_interleave(pkg):
    rng = np.random.default_rng(2)
    inter, k = 128, 256
    n = 2 * inter
    codes = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    sc = rng.integers(110, 130, (n, k // 32), dtype=np.uint8)
    rec = 8192 + 512
    for gate_up in (0, 1):
        img = pkg.pack_fp4_weight(codes, sc, gate_up)
        assert img.size == (n // 128) * (k // 128) * rec
        for pr in range(n):
            src = pr
            if gate_up:
                src = (inter if (pr % 16) // 8 else 0) + (pr // 16) * 8 + pr % 8
            rt, r = divmod(pr, 128)
            for kt in range(k // 128):
                record = img[(rt * (k // 128) + kt) * rec:][:rec]
                assert (record[r * 64:(r + 1) * 64] == codes[src, kt * 64:(kt + 1) * 64]).all()
                for b in range(4):
                    assert record[8192 + (r % 32) * 16 + (r // 32) * 4 + b] == sc[src, kt * 4 + b]
