"""Small profiling case for `ncu` (one GPU, a few GB on the device, kernels of well under a millisecond):
one dense FP8 GEMV 18432x7168 and one decode expert layer with 64 experts of the benchmark shape, each run twice.

    python deepseek-ultrafast_b200/prof_case.py [m=1] [experts=64] [tokens=16] [ds|mx]
    ncu --set full --clock-control none -k regex:tc_stream -s 3 -c 3 -o prof python deepseek-ultrafast_b200/prof_case.py

Prefill variant: one expert layer with 128-row token tiles (8 experts, 2048 tokens, top-8 -> 2048 rows per expert) and
one dense 7168x7168 FP8 GEMM over the same tokens, each run twice.

    python deepseek-ultrafast_b200/prof_case.py prefill [experts=8] [tokens=2048] [ds|mx]
    ncu --set full --clock-control none -k regex:tc_prefill -s 3 -c 3 -o prof python deepseek-ultrafast_b200/prof_case.py prefill
"""
import importlib
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402
from __graft_entry__ import load_package  # noqa: E402


def prefill(pkg, synth, argv):
    n_exp = int(argv[0]) if len(argv) > 0 else 8
    tokens = int(argv[1]) if len(argv) > 1 else 2048
    mode = pkg.MODE_MX if (len(argv) > 2 and argv[2] == "mx") else pkg.MODE_DS
    ctx = pkg.Ctx(0)
    dev = ctx.device
    hidden, inter, topk = 7168, 2048, 8
    tiles, sds = synth.fp8_dense(torch, mode == pkg.MODE_MX, hidden, hidden, 0.02, 1, dev)
    wd = pkg.Weight(ctx, 0, mode, hidden, hidden, 1, False, tiles, sds)
    w13 = synth.fp4_experts(torch, n_exp, 2 * inter, hidden, 0.02, 2, True, dev)
    w2 = synth.fp4_experts(torch, n_exp, hidden, inter, 0.02, 3, False, dev)
    layer = pkg.MoeLayer(ctx, pkg.Weight.experts_fp4_packed(ctx, w13, 2 * inter, hidden, n_exp, True),
                         pkg.Weight.experts_fp4_packed(ctx, w2, hidden, inter, n_exp, False), tokens, topk, mode, tile_rows=128)
    xm = torch.randn(tokens, hidden, device=dev).bfloat16()
    xq, xs = pkg.act_quant(ctx, mode, xm)
    h = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    ids, w = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, torch.randn(tokens, n_exp, device=dev), None, topk)
    y = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    for _ in range(2):
        pkg.gemm_fp8(ctx, wd, xq, xs, tokens, h)
        layer.forward(xm, ids, w, y)
    torch.cuda.synchronize()
    print("device status", ctx.status().code, "pairs", tokens * topk)


def main():
    pkg = load_package()
    synth = importlib.import_module(pkg.__name__ + ".synth")
    torch.manual_seed(0)       # same routing (and the same number of active experts) on every run
    torch.cuda.manual_seed(0)
    if len(sys.argv) > 1 and sys.argv[1] == "prefill":
        return prefill(pkg, synth, sys.argv[2:])
    m = int(sys.argv[1]) if len(sys.argv) > 1 else 1
    n_exp = int(sys.argv[2]) if len(sys.argv) > 2 else 64
    tokens = int(sys.argv[3]) if len(sys.argv) > 3 else 16
    mode = pkg.MODE_MX if (len(sys.argv) > 4 and sys.argv[4] == "mx") else pkg.MODE_DS
    ctx = pkg.Ctx(0)
    dev = ctx.device
    n, k = 18432, 7168
    tiles, sds = synth.fp8_dense(torch, mode == pkg.MODE_MX, n, k, 0.02, 1, dev)
    wd = pkg.Weight(ctx, 0, mode, n, k, 1, False, tiles, sds)
    x = torch.randn(m, k, device=dev).bfloat16()
    xq, xs = pkg.act_quant(ctx, mode, x)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    hidden, inter, topk = 7168, 2048, 8
    w13 = synth.fp4_experts(torch, n_exp, 2 * inter, hidden, 0.02, 2, True, dev)
    w2 = synth.fp4_experts(torch, n_exp, hidden, inter, 0.02, 3, False, dev)
    layer = pkg.MoeLayer(ctx, pkg.Weight.experts_fp4_packed(ctx, w13, 2 * inter, hidden, n_exp, True),
                         pkg.Weight.experts_fp4_packed(ctx, w2, hidden, inter, n_exp, False), tokens, topk, mode)
    xm = torch.randn(tokens, hidden, device=dev).bfloat16()
    ids, w = pkg.moe_route_tokens(ctx, pkg.SCORE_SOFTMAX, torch.randn(tokens, n_exp, device=dev), None, topk)
    y = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    for _ in range(2):
        pkg.gemm_fp8(ctx, wd, xq, xs, m, out)
        layer.forward(xm, ids, w, y)
    torch.cuda.synchronize()
    print("device status", ctx.status().code, "active experts", int(torch.unique(ids).numel()))


if __name__ == "__main__":
    main()
