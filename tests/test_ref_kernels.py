"""The reference's own sm_100a kernels, run on the GPU beside the CPU oracle and beside this library's kernels.

oracle/_ref/*.cubin are the reference's kernels compiled from its own sources (oracle/Makefile); oracle/refkernels.py
launches them with the geometry of the reference's Rust host code.  These tests are what pins the oracle to the
reference beyond its known-answer tests: in the reference's (MX) geometry the quantized codes and scales, the router's
picks and the permute plan must agree bit for bit, and GEMM outputs within the 1e-2 relative Frobenius bar.
The tests need the cubins, which are built where the reference's sources are present and travel with the repository
snapshot; without them every test here is skipped.
"""
import numpy as np
import pytest
import torch

import oracle
import oracle.refkernels as rk
from conftest import randn_bf16, seeded

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not rk.available(), reason="reference cubins / launcher not built")]
TOL = 1e-2


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture
def tc_only(ctx):
    if not ctx.tcgen05:
        pytest.skip("run once (the kernels under test do not depend on the decode path)")
    return ctx


@pytest.mark.parametrize("m,k", [(4, 2048), (130, 7168), (64, 512)])
def test_tc_quant_rows_equals_oracle_and_library(pkg, tc_only, m, k):
    """tc_quant_rows (cu/tcgemm.cu:300-340): codes and UE8M0 scales of the reference kernel == the CPU oracle's == this
    library's MX quantizer, bit for bit; all-zero blocks, an outlier and tiny values included."""
    ctx = tc_only
    g = seeded(1000 + m + k)
    xt, xn = randn_bf16(g, m, k)
    xt[0, :128] = 0
    if m > 1:
        xt[1, 5] = 3.0e4
        xt[1, 200 % k] = -1.0e-3
        xt[2, 32:64] = 1.0e-6       # below the 1e-4 amax floor
    xd = xt.cuda()
    aq, sfa = rk.tc_quant_rows(xd)
    q, s = pkg.act_quant(ctx, pkg.MODE_MX, xd)
    rk.synchronize()
    qo, so = oracle.act_quant(oracle.MODE_MX, xn)
    rows = aq.shape[0]
    ref_q = aq.cpu().numpy()[:m]
    ref_s = rk.sf_atoms_to_rows(sfa.cpu().numpy(), rows, k)[:m]
    assert (ref_q == qo).all() and (ref_s == so).all(), "oracle differs from the reference kernel"
    assert (q.cpu().numpy() == ref_q).all() and (s.cpu().numpy() == ref_s).all(), "library differs from the reference kernel"


def test_row_sumsq_equals_reference_kernel(pkg, tc_only):
    ctx = tc_only
    g = seeded(77)
    xt, xn = randn_bf16(g, 37, 7168)
    xd = xt.cuda()
    part = rk.tc_row_sumsq(xd)
    ss = pkg.row_sumsq(ctx, xd)
    rk.synchronize()
    ref = part.cpu().numpy()[:, 25]
    assert (ss.cpu().numpy().view(np.uint32) == ref.view(np.uint32)).all()
    assert (oracle.row_sumsq(xn).view(np.uint32) == ref.view(np.uint32)).all()


def test_prenorm_quantizer_mismatch_rate_against_the_reference_rsqrt(pkg, tc_only):
    """The reference evaluates 1/sqrt with the approximate rsqrtf instruction; the oracle and the library's default use a
    correctly rounded 1/sqrt (so that a CPU can pin the result).  Codes may differ where bf16(w * (x * rs)) sits on a
    rounding boundary: the rate is measured here and must stay rare; with the library's approximate-rsqrt switch on, the
    codes are the reference kernel's, bit for bit."""
    ctx = tc_only
    g = seeded(78)
    m, k = 256, 7168
    xt, xn = randn_bf16(g, m, k)
    wt, _ = randn_bf16(g, 1, k)
    wt = (1.0 + 0.1 * wt.float()).bfloat16().reshape(k)
    eps = 1e-6
    xd, wd = xt.cuda(), wt.cuda()
    aq, sfa = rk.tc_quant_rows(xd, pw=wd, eps=eps)
    ss = pkg.row_sumsq(ctx, xd)
    q, s = pkg.act_quant_prenorm(ctx, pkg.MODE_MX, xd, wd, eps, sumsq=ss)
    ctx.set_prenorm_rsqrt_approx(True)
    try:
        q2, s2 = pkg.act_quant_prenorm(ctx, pkg.MODE_MX, xd, wd, eps, sumsq=ss)
    finally:
        ctx.set_prenorm_rsqrt_approx(False)
    rk.synchronize()
    ref_q = aq.cpu().numpy()[:m]
    ref_s = rk.sf_atoms_to_rows(sfa.cpu().numpy(), aq.shape[0], k)[:m]
    rate = float((q.cpu().numpy() != ref_q).mean())
    print(f"prenorm quantizer: {rate:.2e} of the codes differ from the reference kernel's (rsqrtf vs correctly rounded)")
    assert rate < 1e-3
    assert float((s.cpu().numpy() != ref_s).mean()) < 1e-3
    assert (q2.cpu().numpy() == ref_q).all() and (s2.cpu().numpy() == ref_s).all()


@pytest.mark.parametrize("t,e,k", [(64, 256, 8), (33, 384, 6), (5, 8, 2)])
def test_moe_route_tokens_equals_oracle_and_library(pkg, tc_only, t, e, k):
    """moe_route_tokens (cu/ops.cu:615-623): picks, tie rule and weights of the reference kernel against the oracle and the
    library's router on the same activated scores and selection bias."""
    ctx = tc_only
    g = seeded(5 + t)
    scores = torch.sqrt(torch.nn.functional.softplus(torch.randn(t, e, generator=g))).contiguous()
    scores[0, :4] = scores[0, 0]                     # exact ties: the lowest id wins
    bias = (0.05 * torch.randn(e, generator=g)).contiguous()
    bias[:4] = 0.0
    ids_r, w_r = rk.moe_route_tokens(scores.cuda(), bias.cuda(), k, route_scale=1.5)
    ids_l, w_l = pkg.moe_route_tokens(ctx, pkg.SCORE_IDENTITY, scores.cuda(), bias.cuda(), k, route_scale=1.5)
    rk.synchronize()
    ids_o, w_o = oracle.route(0, scores.numpy(), bias.numpy(), k, route_scale=1.5)
    assert (ids_r.cpu().numpy() == ids_o).all() and (ids_l.cpu().numpy() == ids_o).all()
    assert np.abs(w_r.cpu().numpy() - w_o).max() <= 2e-6 * 1.5
    assert (w_l.cpu().numpy().view(np.uint32) == w_r.cpu().numpy().view(np.uint32)).all()


def test_moe_perm_and_gather_quant_equal_library_up_to_the_order_inside_an_expert(pkg, tc_only):
    """moe_perm (cu/tcmoe.cu:19-69) places the pairs of an expert in atomicAdd order; the library sorts them by pair index.
    Same expert offsets and tile list; per expert the same SET of pairs; each permuted row carries its pair's weight.
    moe_gather_quant (cu/tcmoe.cu:88-133): every permuted row holds its token's quantized row (codes of each 32-K block in
    the kpos32 order the reference's expert kernels want), equal to tc_quant_rows of the same token."""
    ctx = tc_only
    t, e, k, h = 300, 16, 4, 512
    g = seeded(9)
    logits = torch.randn(t, e, generator=g)
    ids_n, w_n = oracle.route(1, logits.numpy(), None, k)
    ids, w = torch.from_numpy(ids_n).cuda(), torch.from_numpy(w_n).cuda()
    plan_r = rk.PrefillPlan(ids, w, e)
    plan = pkg.MoePlan(ctx, t, k, e, 128)
    pkg.moe_perm(ctx, plan, ids, w)
    rk.synchronize()
    nt = int(plan_r.ntiles.cpu()[0])
    assert nt == int(plan.ntiles.cpu()[0])
    tiles_r, tiles_l = plan_r.tiles.cpu().numpy()[:nt], plan.tiles.cpu().numpy()[:nt]
    assert (tiles_r == tiles_l).all()
    off = plan.expert_off.cpu().numpy()
    rp_r, rp_l = plan_r.row_pair.cpu().numpy(), plan.row_pair.cpu().numpy()
    pr_r = plan_r.pair_row.cpu().numpy()
    rw_r = plan_r.row_w.cpu().numpy()
    for x in range(e):
        assert sorted(rp_r[off[x]:off[x + 1]].tolist()) == rp_l[off[x]:off[x + 1]].tolist()
    assert (rp_r[pr_r] == np.arange(t * k)).all()
    assert (rw_r == w_n.reshape(-1)[rp_r]).all()
    # row_tile = tile << 8 | row inside the tile
    rt = plan_r.row_tile.cpu().numpy()
    rows = np.arange(t * k)
    tile_of = rt >> 8
    assert (tiles_r[tile_of, 1] + (rt & 255) == rows).all()
    # gather + quant: compare with tc_quant_rows (same rsqrtf, same sum of squares) through the permutation
    xt, _ = randn_bf16(g, t, h)
    wt, _ = randn_bf16(g, 1, h)
    wt = (1.0 + 0.1 * wt.float()).bfloat16().reshape(h)
    xd, wd = xt.cuda(), wt.cuda()
    part = rk.tc_row_sumsq(xd)
    xq, sf = rk.moe_gather_quant(xd, wd, 1e-6, plan_r, part=part)
    aq, sfa = rk.tc_quant_rows(xd, pw=wd, eps=1e-6, part=part)
    rk.synchronize()
    tok_q = aq.cpu().numpy()[:t]
    tok_s = rk.sf_atoms_to_rows(sfa.cpu().numpy(), aq.shape[0], h)[:t]
    perm = np.array([rk.kpos32(j) for j in range(32)])
    got = xq.cpu().numpy()[:t * k].reshape(t * k, h // 32, 32)
    want = np.empty_like(got)
    want[:, :, perm] = tok_q[rp_r // k].reshape(t * k, h // 32, 32)
    assert (got == want).all()
    sf_n = sf.cpu().numpy().reshape(-1, h // 128, 512)
    for r in (0, 1, 129, t * k - 1):
        tile, idx = int(rt[r]) >> 8, int(rt[r]) & 255
        for kb in range(h // 32):
            assert sf_n[tile, kb // 4, (idx % 32) * 16 + (idx // 32) * 4 + kb % 4] == tok_s[rp_r[r] // k, kb]


@pytest.mark.parametrize("n,k,m,persistent", [(512, 1024, 200, True), (512, 1024, 200, False), (256, 512, 65, True), (1024, 2048, 384, None)])
def test_tc_gemm_fp8_outputs_pin_the_oracle_and_match_the_library(pkg, tc_only, n, k, m, persistent):
    """tc_quant_rows + tc_gemm_fp8 / tc_gemm_fp8p (cu/tcgemm.cu:20-288): the reference's tcgen05 prefill GEMM against the
    oracle's MX dequantize-then-matmul (this pins the oracle's GEMM by the reference itself, not by formula only) and against
    this library's kernel on the same codes."""
    ctx = tc_only
    g = seeded(n + k + m)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(oracle.MODE_MX, wn)
    tw = rk.TcWeight(wq, ws)
    xd = xt.cuda()
    aq, sfa = rk.tc_quant_rows(xd)
    out_r = rk.tc_gemm(tw, aq, sfa, m, persistent=persistent)
    w = pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, wq, ws)
    out_l = pkg.gemv(ctx, w, xd)
    rk.synchronize()
    assert ctx.status().code == 0
    xq, xs = oracle.act_quant(oracle.MODE_MX, xn)
    _, ref = oracle.gemm_fp8(oracle.MODE_MX, wq, ws, xq, xs)
    got_r, got_l = out_r.float().cpu().numpy(), out_l.float().cpu().numpy()
    assert rel(ref, got_r) < TOL, "oracle differs from the reference kernel"
    assert rel(got_l, got_r) < TOL, "library differs from the reference kernel"
    # both sum exact products of the same codes in fp32 and round once to bf16: differences are single bf16 ulps
    assert np.abs(got_l - got_r).max() <= np.abs(got_r).max() * 2 ** -7


@pytest.mark.parametrize("n,k,m", [(512, 1024, 1), (7168, 2048, 5), (4096, 7168, 16), (1024, 2048, 8)])
def test_gemv_fp8_decode_kernel_pins_the_oracle_and_matches_the_library(pkg, tc_only, n, k, m):
    """gemv_fp8_n{1,2}_p{1,2,4} (cu/gemv.cu:133-540): the reference's mma.sync decode GEMV (bf16 activations in, quantized
    1x32 in the kernel, K split over a cluster) against the oracle and this library's gemv in the reference's geometry."""
    ctx = tc_only
    g = seeded(3 * n + k + m)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(oracle.MODE_MX, wn)
    out_r = rk.gemv_fp8(rk.GemvWeight(wq, ws), xt.cuda())
    out_l = pkg.gemv(ctx, pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, wq, ws), xt.cuda())
    rk.synchronize()
    xq, xs = oracle.act_quant(oracle.MODE_MX, xn)
    _, ref = oracle.gemm_fp8(oracle.MODE_MX, wq, ws, xq, xs)
    got_r, got_l = out_r.float().cpu().numpy(), out_l.float().cpu().numpy()
    assert rel(ref, got_r) < TOL and rel(got_l, got_r) < TOL


@pytest.mark.parametrize("n,k,m", [(7168, 2048, 1), (7168, 2048, 8), (12288, 1024, 3)])
def test_tc_gemv_fp8_pins_the_oracle_and_matches_the_library(pkg, tc_only, n, k, m):
    """tc_gemv_fp8 (cu/tcgemv.cu:33-241): the reference's tcgen05 decode GEMV at the shape that qualifies for it
    (7168 x 2048, K split over clusters of two) against the oracle and this library's tcgen05 streaming GEMV."""
    ctx = tc_only
    g = seeded(n + 5 * k + m)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(oracle.MODE_MX, wn)
    out_r = rk.tc_gemv_fp8(rk.TcWeight(wq, ws), xt.cuda())
    out_l = pkg.gemv(ctx, pkg.Weight.dense_fp8(ctx, pkg.MODE_MX, wq, ws), xt.cuda())
    rk.synchronize()
    xq, xs = oracle.act_quant(oracle.MODE_MX, xn)
    _, ref = oracle.gemm_fp8(oracle.MODE_MX, wq, ws, xq, xs)
    got_r, got_l = out_r.float().cpu().numpy(), out_l.float().cpu().numpy()
    assert rel(ref, got_r) < TOL and rel(got_l, got_r) < TOL


@pytest.mark.parametrize("tile_rows", [128, 8])
def test_tc_moe_w13_w2_pin_the_oracle_and_match_the_library(pkg, ctx, tile_rows):
    """tc_moe_w13 / tc_moe_w2 (cu/tcmoe.cu:184-588), the reference's tcgen05 prefill expert GEMMs, launched after its own
    moe_perm and moe_gather_quant.  Each kernel is checked on the reference's OWN inputs:
      * gate/up + SwiGLU + re-quantization: the FP8 codes and UE8M0 scales it writes against the oracle's grouped FP4 GEMM
        + SwiGLU (bf16 rounds, routing weight folded in) + 1x32 quantizer on the same quantized token rows (a handful of
        codes may differ: the device's and the host's expf round a few bf16 values apart);
      * down projection: its fp32 pair rows against the oracle's GEMM on the reference's re-quantized activations;
      * and this library's grouped kernels (dsuf_moe_w13_swiglu, dsuf_act_quant_fp8, dsuf_moe_w2, MX geometry) on the same
        token codes, pair by pair: the prefill kernels on a 128-row plan and the decode kernels on 8-row slots.
    This pins the expert-GEMM half of the oracle by the reference's kernel, as the dense half is pinned above.  The 8-row
    case runs on both decode paths (tcgen05 and mma.sync streaming kernels)."""
    if not ctx.tcgen05 and tile_rows == 128:
        pytest.skip("128-row plans run on the tcgen05 path only")
    t, e, k, dim, inter = 300, 8, 4, 1024, 512
    g = seeded(77)
    logits = torch.randn(t, e, generator=g)
    ids_n, w_n = oracle.route(1, logits.numpy(), None, k)
    ids, w = torch.from_numpy(ids_n).cuda(), torch.from_numpy(w_n).cuda()
    xt, _ = randn_bf16(g, t, dim)
    pw = torch.ones(dim, dtype=torch.bfloat16)
    w13 = (torch.randn(e, 2 * inter, dim, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(e, dim, inter, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[i]) for i in range(e)]
    q2 = [oracle.quant_fp4_weight(w2[i]) for i in range(e)]
    c13, s13 = np.stack([a for a, _ in q13]), np.stack([b for _, b in q13])
    c2, s2 = np.stack([a for a, _ in q2]), np.stack([b for _, b in q2])
    # ---- the reference's chain ----
    plan_r = rk.PrefillPlan(ids, w, e)
    xq, sf = rk.moe_gather_quant(xt.cuda(), pw.cuda(), 1e-6, plan_r)
    wts = rk.MoeFp4Weights(c13, s13, c2, s2)
    aq, asf, ypair = rk.tc_moe(wts, plan_r, xq, sf)
    rk.synchronize()
    p = t * k
    nt = int(plan_r.ntiles.cpu()[0])
    tiles = plan_r.tiles.cpu().numpy()[:nt]
    rp_r, rw_r = plan_r.row_pair.cpu().numpy(), plan_r.row_w.cpu().numpy()
    rt_r = plan_r.row_tile.cpu().numpy()
    tile_of, idx_of = rt_r >> 8, rt_r & 255
    xq_nat = rk.unpermute_k32(xq.cpu().numpy()[:p])
    xs_rows = rk.sf_atoms_to_rows(sf.cpu().numpy()[:nt * (dim // 128) * 512], nt * 128, dim)[tile_of * 128 + idx_of]
    aq_nat = rk.unpermute_k32(aq.cpu().numpy()[:p])
    as_rows = rk.sf_atoms_to_rows(asf.cpu().numpy()[:nt * (inter // 128) * 512], nt * 128, inter)[tile_of * 128 + idx_of]
    yp = ypair.cpu().numpy()
    lut = oracle.e4m3_lut()
    bad_codes = bad_scales = 0
    act_ref = np.zeros((p, inter), np.float32)
    for ex, row0, cnt, _ in tiles:
        rows = np.arange(row0, row0 + cnt)
        gu = oracle.gemm_fp4(oracle.MODE_MX, c13[ex], s13[ex], xq_nat[rows], xs_rows[rows])
        gt = oracle.bf16_to_f32(oracle.f32_to_bf16(gu[:, :inter]))
        up = oracle.bf16_to_f32(oracle.f32_to_bf16(gu[:, inter:]))
        a16 = oracle.f32_to_bf16((gt / (np.float32(1) + np.exp(-gt, dtype=np.float32)) * up * rw_r[rows, None]).astype(np.float32))
        qc, qs = oracle.act_quant(oracle.MODE_MX, a16)
        bad_codes += int((qc != aq_nat[rows]).sum())
        bad_scales += int((qs != as_rows[rows]).sum())
        act_ref[rows] = lut[aq_nat[rows]] * np.repeat((as_rows[rows].astype(np.uint32) << 23).view(np.float32), 32, axis=1)
        assert rel(act_ref[rows], oracle.bf16_to_f32(a16)) < 0.04          # e4m3 re-quantization error of the same values
        y = oracle.gemm_fp4(oracle.MODE_MX, c2[ex], s2[ex], aq_nat[rows], as_rows[rows])
        assert rel(yp[rp_r[rows]], y) < 1e-4                               # same codes, fp32 accumulation order only
    assert bad_scales <= p * (inter // 32) // 1000 and bad_codes <= p * inter // 500, (bad_codes, bad_scales)
    # ---- this library's kernels on the same token codes ----
    plan = pkg.MoePlan(ctx, t, k, e, tile_rows)
    pkg.moe_perm(ctx, plan, ids, w)
    pr_l, pr_r = plan.pair_row.cpu().numpy(), plan_r.pair_row.cpu().numpy()
    xq_l, xs_l = np.zeros((p, dim), np.uint8), np.zeros((p, dim // 32), np.uint8)
    xq_l[pr_l], xs_l[pr_l] = xq_nat[pr_r], xs_rows[pr_r]
    W13 = pkg.Weight.experts_fp4(ctx, c13, s13, True)
    W2 = pkg.Weight.experts_fp4(ctx, c2, s2, False)
    act = torch.zeros(p, inter, dtype=torch.bfloat16, device="cuda")
    pkg.moe_w13_swiglu(ctx, W13, pkg.MODE_MX, plan, torch.from_numpy(xq_l).cuda(), torch.from_numpy(xs_l).cuda(), act, 0.0)
    aq_l, as_l = pkg.act_quant(ctx, pkg.MODE_MX, act)
    yrows = torch.zeros(p, dim, dtype=torch.float32, device="cuda")
    pkg.moe_w2(ctx, W2, pkg.MODE_MX, plan, aq_l, as_l, yrows)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    aq_ln, as_ln = aq_l.cpu().numpy(), as_l.cpu().numpy()
    assert int((aq_ln[pr_l] != aq_nat[pr_r]).sum()) <= p * inter // 500 and int((as_ln[pr_l] != as_rows[pr_r]).sum()) <= p * (inter // 32) // 1000
    assert rel(yrows.cpu().numpy()[pr_l], yp[np.arange(p)]) < TOL
