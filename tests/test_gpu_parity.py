"""GPU parity: every kernel of the path, called through the C ABI, against the CPU oracle on identical seeded inputs.

Bars: quantized codes, scales and all index work bit-exact; bf16/fp32 matrix-product outputs within 1e-2 relative
Frobenius error of the oracle's fp32 dequantize-then-matmul (the tolerance the task states).
"""
import numpy as np
import pytest
import torch

import oracle
from conftest import randn_bf16, seeded

pytestmark = pytest.mark.gpu
TOL = 1e-2


def rel(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b.astype(np.float64)) / max(np.linalg.norm(b.astype(np.float64)), 1e-30))


# ------------------------------------------------------------------ activation quantizer
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("m,k,ld", [(4, 2048, 2048), (16, 7168, 7168), (1, 128, 128), (3, 384, 512), (64, 2048, 2048),
                                    (1500, 7168, 7168), (1024, 384, 512), (2100, 8320, 8320)])   # >= 1024 rows of >= 6144: the kernel for large inputs
def test_act_quant_bit_exact(pkg, ctx, mode, m, k, ld):
    g = seeded(10 + m + k)
    xt, _ = randn_bf16(g, m, ld)
    xt[0, :128] = 0                                   # all-zero block
    if m > 1:
        xt[1, 5] = 3.0e4                              # outlier: neighbours underflow to tiny codes
        xt[1, 200 % k] = -1.0e-3
    xd = xt.cuda()[:, :k]
    q, s = pkg.act_quant(ctx, mode, xd)
    torch.cuda.synchronize()
    qo, so = oracle.act_quant(mode, xt[:, :k].contiguous().view(torch.uint16).numpy())
    assert (q.cpu().numpy() == qo).all()
    assert (s.cpu().numpy() == so).all()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("m,k,ld", [(4, 2048, 2048), (9, 7168, 7168), (3, 384, 512), (130, 1024, 1024)])
def test_row_sumsq_and_prenorm_quant_bit_exact(pkg, ctx, mode, m, k, ld):
    """tc_row_sumsq + tc_quant_rows with RMS pre-normalisation: sums, codes and scales bit-exact against the oracle."""
    g = seeded(40 + m + k)
    xt, _ = randn_bf16(g, m, ld)
    xt[0, :k] = 0                                     # an all-zero row: rs = 1 / sqrt(eps)
    wt, _ = randn_bf16(g, 1, k)
    wt = (1.0 + 0.1 * wt.float()).bfloat16().reshape(k)
    eps = 1e-6
    xd = xt.cuda()[:, :k]
    ss = pkg.row_sumsq(ctx, xd)
    q, s = pkg.act_quant_prenorm(ctx, mode, xd, wt.cuda(), eps, sumsq=ss)
    torch.cuda.synchronize()
    xn = xt[:, :k].contiguous().view(torch.uint16).numpy()
    sso = oracle.row_sumsq(xn)
    assert (ss.cpu().numpy().view(np.uint32) == sso.view(np.uint32)).all()
    qo, so = oracle.act_quant_prenorm(mode, xn, wt.view(torch.uint16).numpy(), sso, eps)
    assert (q.cpu().numpy() == qo).all()
    assert (s.cpu().numpy() == so).all()


def test_act_quant_rejects_bad_shapes(pkg, ctx):
    x = torch.zeros(2, 100, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.DsufError):
        pkg.act_quant(ctx, 0, x)                      # k % 128 != 0
    q, s = pkg.act_quant(ctx, 1, torch.zeros(0, 128, dtype=torch.bfloat16, device="cuda"))  # empty input is fine
    assert q.shape == (0, 128)


# ------------------------------------------------------------------ dense FP8 GEMV
def _dense_case(pkg, ctx, mode, n, k, m, seed, rows=None):
    g = seeded(seed)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(mode, wn)
    xq, xs = oracle.act_quant(mode, xn)
    w = pkg.Weight.dense_fp8(ctx, mode, wq, ws)
    out = pkg.gemv(ctx, w, xt.cuda())
    out2 = pkg.gemv(ctx, w, xt.cuda())
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    got = out.float().cpu().numpy()
    assert (out.view(torch.uint16) == out2.view(torch.uint16)).all(), "stream-K result depends on timing"
    if rows is None:
        _, ref = oracle.gemm_fp8(mode, wq, ws, xq, xs)
        deq = oracle.matmul_f32(oracle.dequant_fp8(mode, wq, ws), oracle.dequant_fp8(mode, xq, xs))
        assert rel(got, ref) < TOL and rel(got, deq) < TOL
        # bf16 rounding is the only difference left in most entries
        assert np.abs(got - ref).max() <= np.abs(ref).max() * 2 ** -7
    else:
        blk = 32 if mode == 0 else 128
        sel = np.sort(np.random.default_rng(seed).choice(n // blk, rows, replace=False))
        ridx = (sel[:, None] * blk + np.arange(blk)[None]).reshape(-1)
        _, ref = oracle.gemm_fp8(mode, wq[ridx], ws[sel], xq, xs)
        assert rel(got[:, ridx], ref) < TOL


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("m", [1, 4, 8, 16])
def test_dense_gemv_config0(pkg, ctx, mode, m):
    """M=4 N=1024 K=2048 is the CPU-runnable configuration; the other M values are the decode sweep."""
    _dense_case(pkg, ctx, mode, 1024, 2048, m, seed=0)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m", [(128, 128, 1), (256, 512, 3), (4096, 7168, 16), (7168, 2048, 5), (384, 16384, 9)])
def test_dense_gemv_shapes(pkg, ctx, mode, n, k, m):
    _dense_case(pkg, ctx, mode, n, k, m, seed=n + k + m)


@pytest.mark.parametrize("n,k", [(18432, 7168), (7168, 16384)])
def test_dense_gemv_full_size_sampled_rows(pkg, ctx, n, k):
    """The two largest decode shapes: oracle evaluated on a random sample of weight row blocks."""
    _dense_case(pkg, ctx, 1, n, k, 16, seed=7, rows=4)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m", [(1024, 2048, 17), (512, 1024, 33), (7168, 7168, 64)])
def test_dense_gemv_up_to_64_rows_on_tcgen05(pkg, ctx, mode, n, k, m):
    """The tcgen05 decode kernel takes up to 64 token rows per call (one pass over the weight)."""
    if not ctx.tcgen05:
        pytest.skip("the mma.sync decode kernel takes at most 16 rows per call")
    _dense_case(pkg, ctx, mode, n, k, m, seed=n + m)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m", [(1024, 2048, 200), (512, 256, 65), (256, 1024, 384)])
def test_dense_gemm_prefill_rows_on_tcgen05(pkg, ctx, mode, n, k, m):
    """More than 64 token rows take the prefill kernel (128-token tiles x pairs of weight row tiles): a ragged last
    tile, one row past a tile, exactly full tiles."""
    if not ctx.tcgen05:
        pytest.skip("the mma.sync decode kernel takes at most 16 rows per call")
    _dense_case(pkg, ctx, mode, n, k, m, seed=n + m)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m", [(7168, 2048, 1), (7168, 2048, 33), (4096, 7168, 64), (7168, 896, 8), (2048, 512, 16)])
def test_dense_gemv_cluster_k_split(pkg, ctx, mode, n, k, m):
    """Weights with few row tiles run as one row tile per thread-block cluster, K cut into 2 or 4 slices summed through
    distributed shared memory (clusters of 2: 7168 x 2048 and the 8-GPU K shard 7168 x 896; of 4: 4096 x 7168; token
    tiles of 8, 16 and, with the column-split epilogue, 64 columns).  Against the oracle on sampled rows, repeatable bit for
    bit, and equal within rounding to the stream-K decomposition of the same product."""
    if not ctx.tcgen05:
        pytest.skip("cluster K-split is a decomposition of the tcgen05 streaming kernel")
    _dense_case(pkg, ctx, mode, n, k, m, seed=n + k + m, rows=3)
    g = seeded(n + k + m)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(mode, wn)
    w = pkg.Weight.dense_fp8(ctx, mode, wq, ws)
    a = pkg.gemv(ctx, w, xt.cuda())
    ctx.set_dense_ksplit(False)
    try:
        b = pkg.gemv(ctx, w, xt.cuda())
    finally:
        ctx.set_dense_ksplit(True)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    assert rel(a.float().cpu().numpy(), b.float().cpu().numpy()) < 2e-3


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m", [(384, 256, 100), (128, 512, 65), (640, 1024, 300)])
def test_dense_gemm_prefill_odd_number_of_row_tiles(pkg, ctx, mode, n, k, m):
    """The prefill kernel walks weight row tiles in pairs; with an odd number of them (3, 1, 5) the last pair's second
    half repeats the last tile and its outputs are dropped."""
    if not ctx.tcgen05:
        pytest.skip("tcgen05 path only")
    _dense_case(pkg, ctx, mode, n, k, m, seed=n + k + m)


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m,split", [(1024, 2048, 4, 384), (7168, 2048, 3, 4096), (512, 1024, 16, 0), (512, 1024, 200, 128), (2048, 512, 40, 1000)])
def test_dense_gemv_options_fp32_output_and_column_split(pkg, ctx, mode, n, k, m, split):
    """GemvOpts' out_f32 and split on every dense kernel (decode stream-K / cluster K-split, prefill tiles): the fp32
    output rounds to the bf16 output bit for bit, and the two halves of a split output are the columns of the unsplit one."""
    if not ctx.tcgen05 and m > 16:
        pytest.skip("the mma.sync decode kernel takes at most 16 rows per call")
    g = seeded(n + k + m + split)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(mode, wn)
    w = pkg.Weight.dense_fp8(ctx, mode, wq, ws)
    xq, xs = pkg.act_quant(ctx, mode, xt.cuda())
    base = pkg.gemm_fp8(ctx, w, xq, xs, m, alpha=0.5)
    f32 = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, out_f32=True)
    torch.cuda.synchronize()
    assert f32.dtype == torch.float32 and torch.equal(f32.bfloat16().view(torch.uint16), base.view(torch.uint16))
    if split:
        a, b = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, n_split=split)
        af, bf = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, n_split=split, out_f32=True)
        torch.cuda.synchronize()
        assert torch.equal(a.view(torch.uint16), base[:, :split].contiguous().view(torch.uint16))
        assert torch.equal(b.view(torch.uint16), base[:, split:].contiguous().view(torch.uint16))
        assert torch.equal(af, f32[:, :split]) and torch.equal(bf, f32[:, split:])
        with pytest.raises(pkg.DsufError):
            pkg.gemm_fp8_ex(ctx, w, xq, xs, m, n_split=n)          # nothing left for the second output
    # the router-gate epilogue: sqrt(softplus(.)) of the fp32 result, in fp32 (what the router takes as ready scores)
    ssp = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, sqrt_softplus=True)
    torch.cuda.synchronize()
    want = torch.sqrt(torch.where(f32 > 20, f32, torch.log1p(torch.exp(f32))))
    assert ssp.dtype == torch.float32 and torch.allclose(ssp, want, rtol=1e-5, atol=1e-6)
    # accumulate: fp32 out += result, every element written once per launch: two launches give exactly base + 2 * f32
    accum = torch.full_like(f32, 0.25)
    pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, out=accum, accumulate=True)
    pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, out=accum, accumulate=True)
    torch.cuda.synchronize()
    assert torch.equal(accum, (torch.full_like(f32, 0.25) + f32) + f32)
    assert ctx.status().code == 0


@pytest.mark.parametrize("m,limit", [(5, 0.0), (64, 0.0), (200, 0.0), (16, 0.04)])
def test_fp8_shared_expert_gate_up_with_swiglu_epilogue(pkg, ctx, m, limit):
    """The FP8 shared expert's gate/up projection: one dense FP8 (MX) GEMM over interleaved gate / up rows with the SwiGLU
    epilogue (gemm_tc with Epilogue::SwiGlu, model.rs:3081-3084), decode (m <= 64: cluster K-split / stream-K) and prefill
    kernels, against the oracle's GEMM followed by bf16(silu(bf16 gate) * bf16 up) with the optional clamp."""
    if not ctx.tcgen05:
        pytest.skip("the SwiGLU epilogue on dense weights is offered on the tcgen05 path")
    inter, k = 256, 1024
    g = seeded(300 + m)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, 2 * inter, k, std=0.05)
    wq, ws = oracle.quant_fp8_weight(oracle.MODE_MX, wn)
    W = pkg.Weight.dense_fp8_gate_up(ctx, wq, ws)
    xq, xs = pkg.act_quant(ctx, pkg.MODE_MX, xt.cuda())
    act = pkg.gemm_fp8_swiglu(ctx, W, xq, xs, m, swiglu_limit=limit)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    xqo, xso = oracle.act_quant(oracle.MODE_MX, xn)
    _, f = oracle.gemm_fp8(oracle.MODE_MX, wq, ws, xqo, xso)
    b = lambda a: oracle.bf16_to_f32(oracle.f32_to_bf16(a))
    gt, up = b(f[:, :inter]), b(f[:, inter:])
    if limit > 0:
        up, gt = np.clip(up, -limit, limit), np.minimum(gt, limit)
    want = b(gt / (1.0 + np.exp(-gt)) * up)
    assert rel(act.float().cpu().numpy(), want) < TOL
    with pytest.raises(pkg.DsufError, match="SwiGLU"):
        pkg.gemm_fp8(ctx, W, xq, xs, m)        # a plain store would hand out interleaved rows


def test_dense_gemv_linearity_and_alpha(pkg, ctx):
    """Size-independent property: out(alpha) = alpha * out(1) up to bf16 rounding."""
    g = seeded(3)
    xt, xn = randn_bf16(g, 4, 2048)
    _, wn = randn_bf16(g, 1024, 2048, std=0.02)
    wq, ws = oracle.quant_fp8_weight(1, wn)
    w = pkg.Weight.dense_fp8(ctx, 1, wq, ws)
    a = pkg.gemv(ctx, w, xt.cuda()).float()
    b = pkg.gemv(ctx, w, xt.cuda(), alpha=0.5).float()
    torch.cuda.synchronize()
    assert torch.allclose(b, a * 0.5, rtol=2 ** -7, atol=1e-6)


def test_dense_gemv_rejects_bad_arguments(pkg, ctx):
    g = seeded(4)
    _, wn = randn_bf16(g, 128, 128, std=0.02)
    wq, ws = oracle.quant_fp8_weight(1, wn)
    w = pkg.Weight.dense_fp8(ctx, 1, wq, ws)
    if not ctx.tcgen05:
        with pytest.raises(pkg.DsufError):
            pkg.gemv(ctx, w, torch.zeros(17, 128, dtype=torch.bfloat16, device="cuda"))   # more rows than one mma.sync call takes
    xq = torch.zeros(1, 128, dtype=torch.uint8, device="cuda")
    xs = torch.ones(1, 1, dtype=torch.float32, device="cuda")
    with pytest.raises(pkg.DsufError):
        pkg.gemm_fp8(ctx, w, xq, xs, 0)                                               # m = 0


# ------------------------------------------------------------------ router, plan, gather
@pytest.mark.parametrize("score_fn", [0, 1, 2])
@pytest.mark.parametrize("t,e,k", [(64, 256, 8), (5, 8, 2), (1, 384, 6), (33, 512, 16)])
def test_route_matches_oracle(pkg, ctx, score_fn, t, e, k):
    g = seeded(t + e)
    logits = torch.randn(t, e, generator=g)
    if score_fn == 0:
        logits = logits.abs() + 0.01
    bias = torch.randn(e, generator=g) * 0.1
    ids, w = pkg.moe_route_tokens(ctx, score_fn, logits.cuda(), bias.cuda(), k, route_scale=2.5)
    torch.cuda.synchronize()
    io, wo = oracle.route(score_fn, logits.numpy(), bias.numpy(), k, 2.5)
    assert (ids.cpu().numpy() == io).all()
    assert np.allclose(w.cpu().numpy(), wo, rtol=2e-5, atol=1e-7)


def test_route_ties_go_to_the_lowest_id(pkg, ctx):
    s = torch.full((3, 64), 0.25)
    ids, w = pkg.moe_route_tokens(ctx, 0, s.cuda(), None, 4)
    torch.cuda.synchronize()
    assert ids.cpu().tolist() == [[0, 1, 2, 3]] * 3
    assert torch.allclose(w.cpu(), torch.full((3, 4), 0.25))


@pytest.mark.parametrize("t,k,e,tile,e_lo,n_loc", [(64, 8, 256, 8, 0, 256), (64, 8, 256, 16, 64, 64), (1, 1, 4, 8, 0, 4),
                                                   (300, 6, 40, 128, 0, 40), (2000, 8, 256, 128, 128, 128)])
def test_permute_plan_bit_exact(pkg, ctx, t, k, e, tile, e_lo, n_loc):
    rng = np.random.default_rng(t)
    ids = np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)
    w = rng.random((t, k)).astype(np.float32)
    plan = pkg.MoePlan(ctx, t, k, n_loc, tile)
    pkg.moe_perm(ctx, plan, torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), e_lo)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    # oracle on the local experts only: remap foreign experts to a sentinel bucket at the end
    local = ids.reshape(-1) - e_lo
    keep = (local >= 0) & (local < n_loc)
    remap = np.where(keep, local, n_loc).astype(np.int32)
    off, row_pair, pair_row, tiles = oracle.permute_plan(remap, n_loc + 1, tile)
    nrows = int(keep.sum())
    nt = int((tiles[:, 0] < n_loc).sum())
    got_nt, got_rows = plan.ntiles.cpu().tolist()
    assert (got_nt, got_rows) == (nt, nrows)
    assert (plan.expert_off.cpu().numpy() == off[:n_loc + 1]).all()
    assert (plan.row_pair.cpu().numpy()[:nrows] == row_pair[:nrows]).all()
    want_pr = np.where(keep, pair_row, -1)
    assert (plan.pair_row.cpu().numpy() == want_pr).all()
    assert (plan.tiles.cpu().numpy()[:nt] == tiles[:nt]).all()
    assert (plan.row_w.cpu().numpy()[:nrows] == w.reshape(-1)[row_pair[:nrows]]).all()


@pytest.mark.parametrize("mode", [0, 1])
def test_gather_quant_rows_equal_plain_quant(pkg, ctx, mode):
    t, k, e, h = 24, 4, 16, 512
    g = seeded(9)
    xt, xn = randn_bf16(g, t, h)
    rng = np.random.default_rng(1)
    ids = np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)
    plan = pkg.MoePlan(ctx, t, k, e, 8)
    pkg.moe_perm(ctx, plan, torch.from_numpy(ids).cuda(), torch.ones(t, k).cuda())
    blk = 32 if mode == 0 else 128
    xq = torch.zeros(t * k, h, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(t * k, h // blk, dtype=torch.uint8 if mode == 0 else torch.float32, device="cuda")
    pkg.moe_gather_quant(ctx, mode, plan, xt.cuda(), xq, xs)
    torch.cuda.synchronize()
    qo, so = oracle.act_quant(mode, xn)
    row_pair = plan.row_pair.cpu().numpy()
    assert (xq.cpu().numpy() == qo[row_pair // k]).all()
    assert (xs.cpu().numpy() == so[row_pair // k]).all()


@pytest.mark.parametrize("mode", [0, 1])
def test_gather_quant_prenorm_rows_equal_plain_prenorm_quant(pkg, ctx, mode):
    t, k, e, h = 24, 4, 16, 512
    g = seeded(19)
    xt, xn = randn_bf16(g, t, h)
    wt, _ = randn_bf16(g, 1, h)
    wt = (1.0 + 0.1 * wt.float()).bfloat16().reshape(h)
    rng = np.random.default_rng(2)
    ids = np.stack([rng.choice(e, k, replace=False) for _ in range(t)]).astype(np.int32)
    plan = pkg.MoePlan(ctx, t, k, e, 8)
    pkg.moe_perm(ctx, plan, torch.from_numpy(ids).cuda(), torch.ones(t, k).cuda())
    blk = 32 if mode == 0 else 128
    xq = torch.zeros(t * k, h, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(t * k, h // blk, dtype=torch.uint8 if mode == 0 else torch.float32, device="cuda")
    pkg.moe_gather_quant_prenorm(ctx, mode, plan, xt.cuda(), wt.cuda(), 1e-6, xq, xs)
    torch.cuda.synchronize()
    qo, so = oracle.act_quant_prenorm(mode, xn, wt.view(torch.uint16).numpy(), oracle.row_sumsq(xn), 1e-6)
    row_pair = plan.row_pair.cpu().numpy()
    assert (xq.cpu().numpy() == qo[row_pair // k]).all()
    assert (xs.cpu().numpy() == so[row_pair // k]).all()


@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("t,e,k,h,e_lo,n_loc,tile", [(64, 256, 8, 7168, 0, 256, 8), (64, 256, 8, 1024, 32, 32, 8), (1, 8, 2, 128, 0, 8, 8),
                                                     (100, 16, 3, 512, 0, 16, 16), (128, 256, 8, 256, 0, 256, 8), (40, 384, 6, 8320, 128, 128, 8),
                                                     (7, 16, 2, 256, 0, 16, 8), (9, 16, 2, 256, 0, 16, 8), (150, 32, 4, 256, 0, 32, 8)])
def test_fused_decode_front_end_equals_the_separate_kernels(pkg, ctx, mode, t, e, k, h, e_lo, n_loc, tile):
    """Router + permute plan + gather/quant in one launch (at most 1024 pairs) against the three separate entries: routing,
    every plan array and the quantized permuted rows bit for bit; expert-parallel shards (pairs of other ranks' experts
    dropped), a hidden size above one 8192-element pass, and token counts around the cluster size of the shared routing
    (7: no cluster; 9: one cluster of 8 CTAs for 9 tokens; 150: more tokens than CTAs) included."""
    g = seeded(t + e + h)
    xt, _ = randn_bf16(g, t, h)
    logits = torch.randn(t, e, generator=g).cuda()
    bias = (0.01 * torch.randn(e, generator=g)).cuda()
    xd = xt.cuda()
    sdt = torch.uint8 if mode == 0 else torch.float32
    blk = 32 if mode == 0 else 128
    res = []
    for fused in (False, True):
        plan = pkg.MoePlan(ctx, t, k, n_loc, tile)
        ids = torch.full((t, k), -7, dtype=torch.int32, device="cuda")
        w = torch.zeros(t, k, dtype=torch.float32, device="cuda")
        xq = torch.zeros(t * k, h, dtype=torch.uint8, device="cuda")
        xs = torch.zeros(t * k, h // blk, dtype=sdt, device="cuda")
        if fused:
            pkg.moe_route_plan_gather(ctx, pkg.SCORE_SOFTMAX, logits, bias, k, 2.5, ids, w, e_lo, plan, mode, xd, xq, xs)
        else:
            pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, logits, bias, k, 2.5, ids=ids, w=w)
            pkg.moe_perm(ctx, plan, ids, w, e_lo)
            pkg.moe_gather_quant(ctx, mode, plan, xd, xq, xs)
        torch.cuda.synchronize()
        assert ctx.status().code == 0
        nt, rows = plan.ntiles.cpu().tolist()
        res.append(dict(ids=ids.cpu(), w=w.cpu().view(torch.int32), off=plan.expert_off.cpu(), row_pair=plan.row_pair.cpu()[:rows],
                        pair_row=plan.pair_row.cpu(), row_w=plan.row_w.cpu()[:rows].view(torch.int32), tiles=plan.tiles.cpu()[:nt],
                        nt=nt, rows=rows, xq=xq.cpu()[:rows], xs=xs.cpu()[:rows]))
    a, b = res
    assert a["nt"] == b["nt"] and a["rows"] == b["rows"]
    for key in ("ids", "w", "off", "row_pair", "pair_row", "row_w", "tiles", "xq", "xs"):
        assert torch.equal(a[key], b[key]), key
    if e_lo == 0 and n_loc == e:
        assert a["rows"] == t * k


# ------------------------------------------------------------------ routed-expert layer
def _moe_case(pkg, ctx, act_mode, T, H, I, E, K, tile_rows, seed, e_lo=0, n_loc=None, limit=0.0, shared=False, ids_rw=None):
    n_loc = E if n_loc is None else n_loc
    g = seeded(seed)
    xt, xn = randn_bf16(g, T, H)
    logits = torch.randn(T, E, generator=g)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[e]) for e in range(E)]
    q2 = [oracle.quant_fp4_weight(w2[e]) for e in range(E)]
    c13, s13 = np.stack([a for a, _ in q13]), np.stack([b for _, b in q13])
    c2, s2 = np.stack([a for a, _ in q2]), np.stack([b for _, b in q2])
    ids, rw = oracle.route(1, logits.numpy(), None, K) if ids_rw is None else ids_rw
    sh_t, sh_n = randn_bf16(g, T, H, std=0.1) if shared else (None, None)
    ref = oracle.moe_layer(act_mode, xn, ids, rw, c13, s13, c2, s2, swiglu_limit=limit, shared=sh_n, e_lo=e_lo,
                           e_hi=e_lo + n_loc, want_act=True)
    W13 = pkg.Weight.experts_fp4(ctx, c13[e_lo:e_lo + n_loc], s13[e_lo:e_lo + n_loc], True)
    W2 = pkg.Weight.experts_fp4(ctx, c2[e_lo:e_lo + n_loc], s2[e_lo:e_lo + n_loc], False)
    layer = pkg.MoeLayer(ctx, W13, W2, T, K, act_mode, e_lo=e_lo, tile_rows=tile_rows, swiglu_limit=limit)
    y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer.forward(xt.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(rw).cuda(), y,
                  sh_t.cuda() if shared else None)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    # intermediate: SwiGLU activations per permuted row against the oracle's per-pair rows
    nrows = int(layer.plan.ntiles.cpu()[1])
    row_pair = layer.plan.row_pair.cpu().numpy()[:nrows]
    act = layer.act.float().cpu().numpy()[:nrows]
    act_ref = oracle.bf16_to_f32(ref["act_bf16"])[row_pair]
    assert rel(act, act_ref) < TOL
    got = y.float().cpu().numpy()
    assert rel(got, ref["y_f32"]) < TOL
    return layer


@pytest.mark.parametrize("act_mode", [0, 1])
@pytest.mark.parametrize("tile_rows", [8, 16])
def test_moe_layer_small(pkg, ctx, act_mode, tile_rows):
    _moe_case(pkg, ctx, act_mode, T=8, H=256, I=128, E=8, K=2, tile_rows=tile_rows, seed=1)


@pytest.mark.parametrize("act_mode", [0, 1])
def test_moe_layer_decode_shape_reduced(pkg, ctx, act_mode):
    """64 tokens (8 seqs x 8-token draft block), top-8 of 32 experts, hidden 1024, inter 512: several experts get
    more than 8 rows, so slots are split, and some get none."""
    _moe_case(pkg, ctx, act_mode, T=64, H=1024, I=512, E=32, K=8, tile_rows=8, seed=2)


@pytest.mark.parametrize("act_mode", [0, 1])
@pytest.mark.parametrize("T,E,K", [(200, 4, 2), (96, 2, 2), (700, 8, 3)])
def test_moe_layer_prefill_tiles_of_128_rows(pkg, ctx, act_mode, T, E, K):
    """128-row plans (prefill): experts with fewer rows than a tile, exactly full tiles and several tiles."""
    if not ctx.tcgen05:
        pytest.skip("128-row plans run on the tcgen05 path only")
    _moe_case(pkg, ctx, act_mode, T=T, H=256, I=128, E=E, K=K, tile_rows=128, seed=T)


@pytest.mark.parametrize("act_mode", [0, 1])
def test_moe_layer_prefill_odd_number_of_row_tiles(pkg, ctx, act_mode):
    """The prefill kernel pairs weight row tiles; the down projection of a 384-wide model has 3 row tiles: its last pair
    repeats the third tile and drops the repeated outputs (the gate/up projection has 2 row tiles x 3 K tiles)."""
    if not ctx.tcgen05:
        pytest.skip("128-row plans run on the tcgen05 path only")
    _moe_case(pkg, ctx, act_mode, T=300, H=384, I=128, E=4, K=2, tile_rows=128, seed=11)


@pytest.mark.parametrize("act_mode", [0, 1])
def test_moe_layer_prefill_experts_spanning_several_slot_groups(pkg, ctx, act_mode):
    """The prefill kernel deals (slot, row-tile pair) items per expert in groups of 32 slots.  Skewed top-1 routing gives
    one expert 66 slots (groups of 32 + 32 + 2, the last slot ragged), one exactly 33 full slots (32 + 1), one 129 rows
    (a full slot and a single row), one a single row and one nothing: the shape of the 16384-token Zipf benchmark (one
    expert with 112 slots) at a size the CPU oracle evaluates in full.  Two row-tile pairs per expert in both GEMMs."""
    if not ctx.tcgen05:
        pytest.skip("128-row plans run on the tcgen05 path only")
    counts = [65 * 128 + 17, 0, 1, 129, 33 * 128]
    T = sum(counts)
    rng = np.random.default_rng(77)
    ids = np.repeat(np.arange(len(counts), dtype=np.int32), counts)
    rng.shuffle(ids)
    rw = rng.uniform(0.5, 1.5, size=T).astype(np.float32)
    layer = _moe_case(pkg, ctx, act_mode, T=T, H=512, I=256, E=len(counts), K=1, tile_rows=128, seed=31,
                      ids_rw=(ids.reshape(T, 1), rw.reshape(T, 1)))
    tiles = layer.plan.tiles.cpu().numpy()[:int(layer.plan.ntiles.cpu()[0])]
    per_expert = np.bincount(tiles[:, 0], minlength=len(counts))
    assert per_expert.tolist() == [66, 0, 1, 2, 33]


@pytest.mark.parametrize("mode", [0, 1])
def test_dense_gemm_prefill_benchmark_size_sampled(pkg, ctx, mode):
    """The dense projection of the layer stack at its prefill size (7168 x 7168 weights, 16384 token rows = 128 token
    tiles x 28 row-tile pairs): sampled token rows x sampled weight row blocks against the oracle, and two runs bitwise
    equal."""
    if not ctx.tcgen05:
        pytest.skip("more than 16 token rows run on the tcgen05 path only")
    n = k = 7168
    m = 16384
    g = seeded(4242)
    xt, xn = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(mode, wn)
    w = pkg.Weight.dense_fp8(ctx, mode, wq, ws)
    xd = xt.cuda()
    out = pkg.gemv(ctx, w, xd)
    out2 = pkg.gemv(ctx, w, xd)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    assert (out.view(torch.uint16) == out2.view(torch.uint16)).all(), "prefill GEMM result depends on timing"
    rng = np.random.default_rng(5)
    tok = np.sort(np.concatenate([np.arange(0, 8), np.arange(m - 8, m), rng.choice(m, 112, replace=False)]))
    blk = 32 if mode == 0 else 128
    sel = np.sort(np.concatenate([[0, n // blk - 1], rng.choice(n // blk, 4, replace=False)]))
    sel = np.unique(sel)
    ridx = (sel[:, None] * blk + np.arange(blk)[None]).reshape(-1)
    xq, xs = oracle.act_quant(mode, np.ascontiguousarray(xn[tok]))
    _, ref = oracle.gemm_fp8(mode, np.ascontiguousarray(wq[ridx]), np.ascontiguousarray(ws[sel]), xq, xs)
    got = out[torch.from_numpy(tok).cuda()].float().cpu().numpy()[:, ridx]
    assert rel(got, ref) < TOL


@pytest.mark.parametrize("act_mode", [0, 1])
@pytest.mark.parametrize("tile_rows", [8, 16])
def test_moe_decode_two_tiles_per_stage_equals_one(pkg, ctx, act_mode, tile_rows):
    """The decode expert GEMMs stream two 128-K tile records per ring stage when the weight has an even number of K tiles
    (hidden 1024: 8 K tiles for gate/up; inter 512: 4 for down).  Both that kernel and the one-tile-per-stage kernel
    against the oracle."""
    if not ctx.tcgen05:
        pytest.skip("a variant of the tcgen05 streaming kernel")
    _moe_case(pkg, ctx, act_mode, T=64, H=1024, I=512, E=32, K=8, tile_rows=tile_rows, seed=2)
    ctx.set_stage_pairs(False)
    try:
        _moe_case(pkg, ctx, act_mode, T=64, H=1024, I=512, E=32, K=8, tile_rows=tile_rows, seed=2)
    finally:
        ctx.set_stage_pairs(True)


def test_moe_layer_clamp_and_shared_expert_term(pkg, ctx):
    _moe_case(pkg, ctx, 1, T=16, H=256, I=128, E=8, K=2, tile_rows=8, seed=3, limit=0.05, shared=True)


def test_moe_layer_expert_parallel_shards_sum_to_whole(pkg, ctx):
    """Two expert shards (experts 0-3 and 4-7) evaluated separately add up to the full layer (fp32, before rounding)."""
    _moe_case(pkg, ctx, 1, T=16, H=256, I=128, E=8, K=2, tile_rows=8, seed=4, e_lo=0, n_loc=4)
    _moe_case(pkg, ctx, 1, T=16, H=256, I=128, E=8, K=2, tile_rows=8, seed=4, e_lo=4, n_loc=4)


def test_moe_layer_empty_batch_launches_nothing_and_succeeds(pkg, ctx):
    """No tokens: every entry of the layer returns OK (the reference's callers never launch with m = 0; here it is a
    defined no-op instead of an error from one of the five entries)."""
    H, I, E, K = 256, 128, 4, 2
    g = seeded(8)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[e]) for e in range(E)]
    q2 = [oracle.quant_fp4_weight(w2[e]) for e in range(E)]
    W13 = pkg.Weight.experts_fp4(ctx, np.stack([a for a, _ in q13]), np.stack([b for _, b in q13]), True)
    W2 = pkg.Weight.experts_fp4(ctx, np.stack([a for a, _ in q2]), np.stack([b for _, b in q2]), False)
    for tile_rows in ([8, 128] if ctx.tcgen05 else [8]):
        layer = pkg.MoeLayer(ctx, W13, W2, 0, K, pkg.MODE_DS, tile_rows=tile_rows)
        x = torch.zeros(0, H, dtype=torch.bfloat16, device="cuda")
        ids = torch.zeros(0, K, dtype=torch.int32, device="cuda")
        w = torch.zeros(0, K, dtype=torch.float32, device="cuda")
        y = torch.zeros(0, H, dtype=torch.bfloat16, device="cuda")
        layer.forward(x, ids, w, y)
        torch.cuda.synchronize()
        assert ctx.status().code == 0
        assert layer.plan.ntiles.cpu().tolist() == [0, 0]


def test_moe_single_token_single_expert(pkg, ctx):
    _moe_case(pkg, ctx, 1, T=1, H=128, I=128, E=2, K=1, tile_rows=8, seed=5)


def test_moe_layer_full_benchmark_size_sampled_tokens(pkg, ctx):
    """The decode configuration at full size (64 tokens, 256 experts top-8, hidden 7168, inter 2048; 6 GB of expert tiles,
    byte offsets beyond 4 GB): the oracle is evaluated for a sample of tokens on exactly the tile bytes the kernels read
    (downloaded and unpacked), the other tokens are covered by the size-independent check that every output row is the
    sum of its top-k expert rows."""
    import importlib
    synth = importlib.import_module(pkg.__name__ + ".synth")
    if not ctx.tcgen05:
        pytest.skip("full size is run once, on the default decode path")
    T, H, I, E, K = 64, 7168, 2048, 256, 8
    dev = ctx.device
    w13 = synth.fp4_experts(torch, E, 2 * I, H, 0.02, 11, True, dev)
    w2 = synth.fp4_experts(torch, E, H, I, 0.02, 12, False, dev)
    W13 = pkg.Weight.experts_fp4_packed(ctx, w13, 2 * I, H, E, True)
    W2 = pkg.Weight.experts_fp4_packed(ctx, w2, H, I, E, False)
    g = seeded(99)
    xt, xn = randn_bf16(g, T, H)
    logits = torch.randn(T, E, generator=g)
    ids, rw = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, logits.cuda(), None, K)
    layer = pkg.MoeLayer(ctx, W13, W2, T, K, pkg.MODE_DS)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    layer.forward(xt.cuda(), ids, rw, y)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    ids_n, rw_n = ids.cpu().numpy(), rw.cpu().numpy()
    io, wo = oracle.route(1, logits.numpy(), None, K)
    assert (ids_n == io).all()
    # size-independent: out[t] == bf16(sum of the token's k permuted rows)
    pr = layer.plan.pair_row.cpu().numpy().reshape(T, K)
    yr = layer.yrows.cpu().numpy()
    want = torch.from_numpy(yr[pr].sum(axis=1)).bfloat16().float().numpy()
    got = y.float().cpu().numpy()
    assert rel(got, want) < 1e-3
    # sampled tokens against the oracle, on the experts they use (highest expert ids included: largest byte offsets)
    sample = [0, 31, int(np.argmax(ids_n.max(axis=1)))]
    per13 = (2 * I // 128) * (H // 128) * synth.REC_FP4
    per2 = (H // 128) * (I // 128) * synth.REC_FP4
    used = sorted(set(ids_n[sample].reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    c13, s13, c2, s2 = [], [], [], []
    for e in used:
        a, b = synth.unpack_fp4(w13[e * per13:(e + 1) * per13].cpu().numpy(), 2 * I, H, True)
        c13.append(a); s13.append(b)
        a, b = synth.unpack_fp4(w2[e * per2:(e + 1) * per2].cpu().numpy(), H, I, False)
        c2.append(a); s2.append(b)
    ids_l = np.vectorize(remap.get)(ids_n[sample]).astype(np.int32)
    ref = oracle.moe_layer(oracle.MODE_DS, xn[sample], ids_l, rw_n[sample], np.stack(c13), np.stack(s13), np.stack(c2), np.stack(s2))
    assert rel(got[sample], ref["y_f32"]) < TOL


@pytest.mark.parametrize("act_mode", [0, 1])
def test_moe_layer_prefill_benchmark_shapes_sampled_tokens(pkg, ctx, act_mode):
    """The prefill kernels at the benchmark's matrix shapes (hidden 7168, inter 2048: 56 K tiles x 16 row-tile pairs for
    gate/up, 16 x 28 for down) on 1024 tokens, 8 experts, top-2 (two or three 128-row slots per expert, the last one
    ragged): sampled tokens against the oracle on exactly the tile bytes the kernels read, every token against the
    size-independent check that an output row is the sum of its top-k expert rows."""
    import importlib
    synth = importlib.import_module(pkg.__name__ + ".synth")
    if not ctx.tcgen05:
        pytest.skip("128-row plans run on the tcgen05 path only")
    T, H, I, E, K = 1024, 7168, 2048, 8, 2
    dev = ctx.device
    w13 = synth.fp4_experts(torch, E, 2 * I, H, 0.02, 21, True, dev)
    w2 = synth.fp4_experts(torch, E, H, I, 0.02, 22, False, dev)
    W13 = pkg.Weight.experts_fp4_packed(ctx, w13, 2 * I, H, E, True)
    W2 = pkg.Weight.experts_fp4_packed(ctx, w2, H, I, E, False)
    g = seeded(123)
    xt, xn = randn_bf16(g, T, H)
    logits = torch.randn(T, E, generator=g)
    ids, rw = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, logits.cuda(), None, K)
    layer = pkg.MoeLayer(ctx, W13, W2, T, K, act_mode, tile_rows=128)
    y = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    layer.forward(xt.cuda(), ids, rw, y)
    y2 = torch.empty_like(y)
    layer.forward(xt.cuda(), ids, rw, y2)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    assert (y.view(torch.uint16) == y2.view(torch.uint16)).all(), "prefill result depends on timing"
    ids_n, rw_n = ids.cpu().numpy(), rw.cpu().numpy()
    pr = layer.plan.pair_row.cpu().numpy().reshape(T, K)
    yr = layer.yrows.cpu().numpy()
    want = torch.from_numpy(yr[pr].sum(axis=1)).bfloat16().float().numpy()
    got = y.float().cpu().numpy()
    assert rel(got, want) < 1e-3
    sample = [0, 517, T - 1]
    per13 = (2 * I // 128) * (H // 128) * synth.REC_FP4
    per2 = (H // 128) * (I // 128) * synth.REC_FP4
    used = sorted(set(ids_n[sample].reshape(-1).tolist()))
    remap = {e: i for i, e in enumerate(used)}
    c13, s13, c2, s2 = [], [], [], []
    for e in used:
        a, b = synth.unpack_fp4(w13[e * per13:(e + 1) * per13].cpu().numpy(), 2 * I, H, True)
        c13.append(a); s13.append(b)
        a, b = synth.unpack_fp4(w2[e * per2:(e + 1) * per2].cpu().numpy(), H, I, False)
        c2.append(a); s2.append(b)
    ids_l = np.vectorize(remap.get)(ids_n[sample]).astype(np.int32)
    ref = oracle.moe_layer(act_mode, xn[sample], ids_l, rw_n[sample], np.stack(c13), np.stack(s13), np.stack(c2), np.stack(s2))
    assert rel(got[sample], ref["y_f32"]) < TOL


@pytest.mark.gpu
@pytest.mark.parametrize("n,k,m", [(1280, 512, 1), (320, 7168, 5), (2048 + 64, 1024 + 64, 16), (129280 // 10, 7168, 8)])
def test_lm_head_logits_and_sampling_records(pkg, ctx, n, k, m):
    """The output head: fp32 logits against the oracle (bf16 products are exact in fp32; the kernel's accumulation order is
    its own: 2e-3 of the row norm), and the per-quad sampling records against the oracle's selection applied to the
    kernel's own logits: maxima, top-8 values, ids and the 9th value bit for bit, the exponential sums to 1e-5.  Shapes:
    a ragged last row tile (n % 128 = 64), K that is not a multiple of a ring stage, a duplicated weight row (a tie)."""
    g = seeded(n + k + m)
    xt, xn = randn_bf16(g, m, k)
    wt, wn = randn_bf16(g, n, k, std=0.05)
    wt[n // 2 + 3] = wt[n // 2 + 1]            # equal logits inside one quad: the lower id must come first
    wn = wt.view(torch.uint16).numpy()
    want = oracle.lm_head(wn, xn, alpha=0.75)
    valid = n - 40
    logits, rec = pkg.lm_head(ctx, wt.cuda(), xt.cuda(), alpha=0.75, temperature=0.7, valid_rows=valid, id_offset=5000)
    plain = pkg.lm_head(ctx, wt.cuda(), xt.cuda(), alpha=0.75)
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    got = logits.cpu().numpy()
    assert np.array_equal(got, plain.cpu().numpy())
    scale = np.linalg.norm(want, axis=1, keepdims=True) / np.sqrt(n)
    assert np.abs(got - want).max() <= 2e-3 * scale.max() + 1e-6, np.abs(got - want).max()
    ref = oracle.sampling_records(got, 0.7, valid_rows=valid, id_offset=5000)
    r = rec.cpu().numpy()
    assert np.array_equal(r[..., 0], ref[..., 0]) and np.array_equal(r[..., 2:11], ref[..., 2:11])
    assert np.array_equal(r.view(np.int32)[..., 11:19], ref.view(np.int32)[..., 11:19])
    assert np.allclose(r[..., 1], ref[..., 1], rtol=1e-5, atol=1e-6)
    t_ids = r.view(np.int32)[0, (n // 2 + 1) // 64, 11:19]
    if (n // 2 + 1) in (t_ids - 5000):        # the tie made the top 8: its twin follows it directly
        i = list(t_ids - 5000).index(n // 2 + 1)
        assert i == 7 or t_ids[i + 1] - 5000 == n // 2 + 3


@pytest.mark.gpu
def test_lm_head_rejects_bad_arguments_and_takes_an_empty_batch(pkg, ctx):
    """More than 16 token rows, records over a vocabulary that is not a multiple of 64, a zero temperature: refused on the
    host with a message, nothing is launched; zero token rows: a no-op."""
    w = torch.zeros(192, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.DsufError):
        pkg.lm_head(ctx, w, torch.zeros(17, 256, dtype=torch.bfloat16, device="cuda"))
    x = torch.zeros(2, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.DsufError):
        pkg.lm_head(ctx, w[:160], x, temperature=1.0, records=torch.zeros(2, 3, 20, device="cuda"))
    with pytest.raises(pkg.DsufError):
        pkg.lm_head(ctx, w, x, temperature=0.0)
    out = pkg.lm_head(ctx, w, x[:0])
    torch.cuda.synchronize()
    assert out.shape == (0, 192) and ctx.status().code == 0


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("t,topk,h,with_shared", [(64, 8, 7168, False), (5, 2, 256, True), (130, 4, 1024, True)])
def test_unpermute_that_also_quantizes_equals_unpermute_then_act_quant(pkg, ctx, mode, t, topk, h, with_shared):
    """dsuf_moe_unpermute_quant: the bf16 rows of dsuf_moe_unpermute and the codes / scales of dsuf_act_quant_fp8 on those
    rows, all bit for bit, with pairs that live on another rank (row < 0) and the optional shared-expert rows."""
    g = seeded(t * topk + h + mode)
    p = t * topk
    plan = pkg.MoePlan(ctx, t, topk, 8, 8)
    rows = torch.randperm(p, generator=g).to(torch.int32)
    rows[::7] = -1
    plan.pair_row.copy_(rows.cuda())
    yrows = torch.randn(p, h, generator=g).cuda()
    shared = torch.randn(t, h, generator=g).bfloat16().cuda() if with_shared else None
    ref = torch.empty(t, h, dtype=torch.bfloat16, device="cuda")
    pkg.moe_unpermute(ctx, plan, yrows, ref, shared)
    rq, rs = pkg.act_quant(ctx, mode, ref)
    out = torch.zeros_like(ref)
    blk = 32 if mode == pkg.MODE_MX else 128
    xq = torch.zeros(t, h, dtype=torch.uint8, device="cuda")
    xs = torch.zeros(t, h // blk, dtype=torch.uint8 if mode == pkg.MODE_MX else torch.float32, device="cuda")
    pkg.moe_unpermute(ctx, plan, yrows, out, shared, quant=(mode, xq, xs))
    torch.cuda.synchronize()
    assert ctx.status().code == 0
    assert torch.equal(out.view(torch.uint16), ref.view(torch.uint16))
    assert torch.equal(xq, rq) and torch.equal(xs.view(torch.uint8), rs.view(torch.uint8))


@pytest.mark.gpu
def test_programmatic_dependent_launch_changes_no_result(pkg):
    """The same chain of launches (quantizer -> dense GEMV -> decode expert layer with the fused front end) with and
    without programmatic dependent launch: bitwise equal (each kernel's griddepcontrol.wait precedes its first read of a
    predecessor's output)."""
    g = seeded(321)
    H, I, E, K, T = 512, 256, 8, 2, 12
    xt, _ = randn_bf16(g, T, H)
    _, wn = randn_bf16(g, H, H, std=0.05)
    wq, ws = oracle.quant_fp8_weight(1, wn)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[e]) for e in range(E)]
    q2 = [oracle.quant_fp4_weight(w2[e]) for e in range(E)]
    logits = torch.randn(T, E, generator=g).cuda()
    outs = []
    for pdl in (False, True):
        c = pkg.Ctx(0, pdl=pdl)
        wd = pkg.Weight.dense_fp8(c, 1, wq, ws)
        W13 = pkg.Weight.experts_fp4(c, np.stack([a for a, _ in q13]), np.stack([b for _, b in q13]), True)
        W2 = pkg.Weight.experts_fp4(c, np.stack([a for a, _ in q2]), np.stack([b for _, b in q2]), False)
        layer = pkg.MoeLayer(c, W13, W2, T, K, 1, tile_rows=8)
        ids = torch.empty(T, K, dtype=torch.int32, device="cuda")
        wts = torch.empty(T, K, dtype=torch.float32, device="cuda")
        y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
        for _ in range(3):
            xq, xs = pkg.act_quant(c, 1, xt.cuda())
            h = pkg.gemm_fp8(c, wd, xq, xs, T)
            layer.forward(h, ids, wts, y, route=(pkg.SCORE_SOFTMAX, logits, None, 1.0))
        torch.cuda.synchronize()
        assert c.status().code == 0
        outs.append((h.clone(), y.clone(), ids.clone()))
        c.close()
    assert torch.equal(outs[0][0].view(torch.uint16), outs[1][0].view(torch.uint16))
    assert torch.equal(outs[0][1].view(torch.uint16), outs[1][1].view(torch.uint16)) and torch.equal(outs[0][2], outs[1][2])


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [0, 1])
@pytest.mark.parametrize("n,k,m,head,off,split", [(512, 1024, 5, 128, 64, 0), (1024, 512, 64, 192, 128, 768), (768, 2048, 200, 64, 0, 0), (7168, 2048, 2, 128, 64, 0)])
def test_dense_gemv_fused_rotary_embedding(pkg, ctx, mode, n, k, m, head, off, split):
    """GemvOpts.rope on the dense kernels (decode stream-K / cluster split / prefill tiles): the rotated bf16 output against
    the oracle's rotation (crates/kernels/cu/gemv.cu:508-516) of the kernel's own fp32 result -- at most one bf16 step apart
    (the host evaluates the fma in double) -- with heads whose first rows are not rotated, a column split whose second
    output is stored unrotated, and a position offset read from device memory."""
    if not ctx.tcgen05:
        pytest.skip("tcgen05 path only")
    g = seeded(n + k + m + head)
    xt, _ = randn_bf16(g, m, k)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(mode, wn)
    w = pkg.Weight.dense_fp8(ctx, mode, wq, ws)
    xq, xs = pkg.act_quant(ctx, mode, xt.cuda())
    pos0 = 37
    ang = torch.rand(pos0 + m, 32, generator=g) * 6.28
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    pos = torch.tensor([pos0], dtype=torch.int32, device="cuda")
    f32 = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, out_f32=True)
    rope = (cos.cuda(), sin.cuda(), pos, head, off)
    if split:
        a, b = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, n_split=split, rope=rope)
        got = torch.cat([a, b], dim=1)
    else:
        got = pkg.gemm_fp8_ex(ctx, w, xq, xs, m, alpha=0.5, rope=rope)
    torch.cuda.synchronize()
    assert ctx.status().code == 0 and got.dtype == torch.bfloat16
    want = oracle.rope_rows(f32.cpu().numpy(), cos.numpy(), sin.numpy(), pos0, head, off, n_first=split or None)
    gf = got.float().cpu().numpy()
    assert np.abs(gf - want).max() <= np.abs(want).max() * 2.0 ** -7
    assert (gf == want).mean() > 0.99
    cols = np.arange(n)
    plain = ((cols % head) < off) | ((cols >= split) if split else False)
    assert np.array_equal(gf[:, plain], oracle.bf16_to_f32(oracle.f32_to_bf16(f32.cpu().numpy()))[:, plain])   # unrotated columns: the plain store
