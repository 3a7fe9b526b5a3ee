"""Host-side restatement of the reference's launch arithmetic and weight layouts (oracle/refkernels.py), checked on the
CPU before any reference kernel is launched: the reference's device waits are unbounded, so its kernels only ever get
geometry that has been verified here."""
import ctypes as C

import numpy as np

import oracle.refkernels as rk


def test_parameter_structs_have_the_sizes_the_reference_asserts():
    # crates/engine/src/ops.rs:1165-1166 (TvParams 256, GemvParams 432); the others follow from the field lists
    assert C.sizeof(rk.GemvParams) == 432 and C.sizeof(rk.TvParams) == 256
    assert C.sizeof(rk.TqParams) == 64 and C.sizeof(rk.TgParams) == 96 and C.sizeof(rk.MpParams) == 80 and C.sizeof(rk.MqParams) == 80
    assert rk.GemvParams.plan.offset == 72 and rk.GemvParams.route.offset == 224 and rk.GemvParams.kvr.offset == 272
    assert rk.TvParams.kvr.offset == 144 and rk.TgParams.out2.offset == 72


def test_gemv_geometry_at_the_benchmark_shapes():
    """ops::gemv's cluster size, CTA count and shared memory at the four decode shapes, M = 1 and M = 16, replayed by hand
    from crates/engine/src/ops.rs:298-328 for a GPU with 148 SMs and 227 KB of opt-in shared memory."""
    want = [(4096, 7168, 1, 4, 256, 139648), (7168, 2048, 1, 2, 224, 89696), (18432, 7168, 1, 1, 288, 228928),
            (7168, 16384, 1, 4, 448, 178816), (4096, 7168, 16, 4, 256, 180864), (7168, 2048, 16, 2, 224, 113760),
            (18432, 7168, 16, 4, 1152, 180864), (7168, 16384, 16, 8, 896, 189632)]
    for n, k, m, cs, ctas, smem in want:
        g = rk.gemv_geometry(n, k, m)
        assert (g["cs"], g["grid"][0] * g["grid"][1], g["smem"]) == (cs, ctas, smem), (n, k, m, g)
        assert g["smem"] <= rk.SMEM_OPTIN and g["block"] == (4 * g["ph"] + 1) * 32
    # the tcgen05 decode GEMV qualifies for one of the four shapes only (ops.rs:1105-1107)
    assert rk.tc_gemv_cluster(7168, 2048) == 2
    assert [rk.tc_gemv_cluster(n, k) for n, k in [(4096, 7168), (18432, 7168), (7168, 16384)]] == [None, None, None]
    assert rk.tg_smem(256) == 205824 and rk.TGP_SMEM == 209920


def test_tile_fp8_follows_the_reference_formula():
    """tile_fp8 (crates/model/src/formats.rs:96-118) restated with array operations against its loop form."""
    n, k = 128, 96
    w = np.random.default_rng(3).integers(0, 256, (n, k), dtype=np.uint8)
    got = rk.tile_fp8(w)
    out = np.zeros(n * k, np.uint8)
    steps = k // 32
    for q in range(n // 64):
        for rg in range(4):
            for ks in range(steps):
                base = q * 64 * k + ks * 2048 + rg * 512
                for lane in range(32):
                    g, t = lane // 4, lane % 4
                    kk = [2 * t, 2 * t + 1, 8 + 2 * t, 9 + 2 * t, 16 + 2 * t, 17 + 2 * t, 24 + 2 * t, 25 + 2 * t]
                    for h, r in enumerate((g, g + 8)):
                        for j, c in enumerate(kk):
                            out[base + lane * 16 + h * 8 + j] = w[q * 64 + rg * 16 + r, ks * 32 + c]
    assert (got == out).all()


def test_scale_atoms_follow_the_reference_formula():
    """tile_sf_blocks (crates/model/src/formats.rs:216-228)."""
    n, k = 256, 384
    s = np.random.default_rng(4).integers(0, 256, (n, k // 32), dtype=np.uint8)
    a = rk.sf_atoms(s)
    kt = k // 128
    for r in (0, 37, 130, 255):
        for kb in range(k // 32):
            assert a[((r // 128) * kt + kb // 4) * 512 + (r % 128 % 32) * 16 + (r % 128 // 32) * 4 + kb % 4] == s[r, kb]
    assert (rk.sf_atoms_to_rows(a, n, k) == s).all()
    assert sorted(rk.kpos32(j) for j in range(32)) == list(range(32))


def test_tile_fp4_and_gate_up_interleave_follow_the_reference_formulas():
    """tile_fp4 (crates/model/src/formats.rs:147-180) restated with array operations against the formula evaluated byte by
    byte, the w13 row interleave of packing.rs:237-241, the inverse kpos32 order and the size of TmParams (ops.rs:1511-1534)."""
    n, k = 128, 192
    rng = np.random.default_rng(5)
    w = rng.integers(0, 256, (n, k // 2), dtype=np.uint8)
    s = rng.integers(0, 256, (n, k // 32), dtype=np.uint8)
    got = rk.tile_fp4(w, s)
    steps, step_b = k // 64, rk.FP4_STEP
    assert got.size == (n // 64) * steps * step_b
    for rg, ks, lane, j in [(0, 0, 0, 0), (3, 2, 17, 1), (5, 1, 31, 3), (7, 2, 9, 2), (4, 0, 22, 0)]:
        g, t = lane // 4, lane % 4
        r0, r1 = rg * 16 + g, rg * 16 + g + 8
        o = ((rg // 4) * steps + ks) * step_b + (rg % 4) * 512 + lane * 16 + j * 4
        kb = ks * 64 + j * 16                       # in elements; two per byte
        want = [w[r0, (kb + 2 * t) // 2], w[r0, (kb + 8 + 2 * t) // 2], w[r1, (kb + 2 * t) // 2], w[r1, (kb + 8 + 2 * t) // 2]]
        assert got[o:o + 4].tolist() == want
        so = ((rg // 4) * steps + ks) * step_b + 2048 + (rg % 4) * 32 + g * 4
        assert got[so:so + 4].tolist() == [s[r0, ks * 2], s[r0, ks * 2 + 1], s[r1, ks * 2], s[r1, ks * 2 + 1]]
    gate = np.arange(64 * 3, dtype=np.uint8).reshape(64, 3)
    up = gate + 100
    il = rk.interleave_gate_up(gate, up)
    assert il.shape == (128, 3) and (il[:32] == gate[:32]).all() and (il[32:64] == up[:32]).all() and (il[64:96] == gate[32:]).all()
    rows = rng.integers(0, 256, (3, 64), dtype=np.uint8)
    perm = np.empty_like(rows)
    for kk in range(64):
        perm[:, (kk // 32) * 32 + rk.kpos32(kk % 32)] = rows[:, kk]
    assert (rk.unpermute_k32(perm) == rows).all()
    import ctypes
    assert ctypes.sizeof(rk.TmParams) == 128 and rk.TM_SMEM == 222464
