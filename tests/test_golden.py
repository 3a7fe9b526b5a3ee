"""Committed golden vectors (tests/golden/*.npz, written by tests/golden/make_golden.py from the CPU oracle).

CPU: the oracle still reproduces them bit for bit (regression pin).  GPU: the CUDA path, through the C ABI, reproduces
the quantized codes / scales / routing exactly and the bf16 outputs within 1e-2 relative Frobenius error."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import oracle

HERE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "make_golden.py"))
make_golden = importlib.util.module_from_spec(spec)
spec.loader.exec_module(make_golden)
MODES = [(oracle.MODE_MX, "mx"), (oracle.MODE_DS, "ds")]


@pytest.mark.parametrize("mode,name", MODES)
def test_oracle_reproduces_golden_vectors(mode, name):
    for case, fn in (("config0", make_golden.config0), ("moe_small", make_golden.moe_small)):
        gold = np.load(os.path.join(HERE, f"{case}_{name}.npz"))
        now = fn(mode)
        assert set(gold.files) == set(now)
        for k in gold.files:
            assert np.array_equal(gold[k], now[k]), (case, name, k)


@pytest.mark.gpu
@pytest.mark.parametrize("mode,name", MODES)
def test_cuda_path_matches_golden_config0(pkg, ctx, mode, name):
    gold = np.load(os.path.join(HERE, f"config0_{name}.npz"))
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 2048, generator=g).bfloat16()
    w = (torch.randn(1024, 2048, generator=g) * 0.02).bfloat16().view(torch.uint16).numpy()
    wq, ws = pkg.quant_fp8_weight_host(mode, w)               # the library's own host quantizer
    assert np.array_equal(ws, gold["ws"]) and wq.astype(np.uint64).sum() == gold["wq_sum"][0]
    xq, xs = pkg.act_quant(ctx, mode, x.cuda())
    out = pkg.gemv(ctx, pkg.Weight.dense_fp8(ctx, mode, wq, ws), x.cuda())
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), gold["xq"]) and np.array_equal(xs.cpu().numpy(), gold["xs"])
    want = oracle.bf16_to_f32(gold["out"])
    got = out.float().cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-2


@pytest.mark.gpu
@pytest.mark.parametrize("mode,name", MODES)
def test_cuda_path_matches_golden_moe(pkg, ctx, mode, name):
    gold = np.load(os.path.join(HERE, f"moe_small_{name}.npz"))
    g = torch.Generator().manual_seed(1)
    T, H, I, E, K = 8, 256, 128, 8, 2
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [pkg.quant_fp4_weight_host(w13[e]) for e in range(E)]
    q2 = [pkg.quant_fp4_weight_host(w2[e]) for e in range(E)]
    c13, s13 = np.stack([a for a, _ in q13]), np.stack([b for _, b in q13])
    c2, s2 = np.stack([a for a, _ in q2]), np.stack([b for _, b in q2])
    assert c13.astype(np.uint64).sum() == gold["c13_sum"][0] and np.array_equal(s13[0, :4], gold["s13"])
    ids, rw = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, logits.cuda(), None, K)
    layer = pkg.MoeLayer(ctx, pkg.Weight.experts_fp4(ctx, c13, s13, True), pkg.Weight.experts_fp4(ctx, c2, s2, False), T, K, mode)
    y = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    layer.forward(x.cuda(), ids, rw, y)
    torch.cuda.synchronize()
    assert np.array_equal(ids.cpu().numpy(), gold["ids"])
    assert np.allclose(rw.cpu().numpy(), gold["w"], rtol=2e-5, atol=1e-7)
    want = oracle.bf16_to_f32(gold["y"])
    got = y.float().cpu().numpy()
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 1e-2


def test_oracle_reproduces_golden_lm_head():
    gold = np.load(os.path.join(HERE, "lm_head_small.npz"))
    now = make_golden.lm_head_small()
    assert set(gold.files) == set(now)
    for k in gold.files:
        assert np.array_equal(gold[k], now[k]), k


@pytest.mark.gpu
def test_cuda_path_matches_golden_lm_head(pkg, ctx):
    """dsuf_lm_head_bf16 against the committed vectors: the ids of the 8 largest logits of every quad exactly (the seeded
    case has no near-ties), row sums and maxima within the rounding the fixture stores."""
    gold = np.load(os.path.join(HERE, "lm_head_small.npz"))
    g = torch.Generator().manual_seed(2)
    x = torch.randn(4, 512, generator=g).bfloat16()
    w = (torch.randn(256, 512, generator=g) * 0.05).bfloat16()
    logits, rec = pkg.lm_head(ctx, w.cuda(), x.cuda(), alpha=0.5, temperature=0.8, valid_rows=236, id_offset=1000)
    torch.cuda.synchronize()
    r = rec.cpu().numpy()
    assert np.array_equal(r.view(np.int32)[..., 11:19], gold["top_ids"])
    assert np.abs(logits.cpu().numpy().astype(np.float64).sum(axis=1) - gold["row_sums"]).max() < 5e-3
    assert np.abs(r[..., 0].astype(np.float64) - gold["zmax"]).max() < 2e-3
