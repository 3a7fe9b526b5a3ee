"""Generates tests/golden/*.npz from the CPU oracle on seeded inputs.

The reference's own implementation cannot run in this environment (Rust host code, no toolchain) and the reference holds
no golden GEMM / MoE outputs, so these vectors are ORACLE-generated: they pin the oracle against regressions and give the
GPU tests a fixed target, they do not add independent evidence of parity with the reference.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import oracle  # noqa: E402


def config0(mode):
    """M=4, N=1024, K=2048; x ~ N(0,1) bf16, W ~ N(0,0.02) bf16, seed 0."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4, 2048, generator=g).bfloat16().view(torch.uint16).numpy()
    w = (torch.randn(1024, 2048, generator=g) * 0.02).bfloat16().view(torch.uint16).numpy()
    wq, ws = oracle.quant_fp8_weight(mode, w)
    xq, xs = oracle.act_quant(mode, x)
    out_bf16, _ = oracle.gemm_fp8(mode, wq, ws, xq, xs)
    return dict(xq=xq, xs=xs, ws=ws, wq_sum=np.array([wq.astype(np.uint64).sum()]), out=out_bf16)


def moe_small(mode):
    """8 tokens, 8 experts top-2, hidden 256, inter 128, seed 1 (the same case as the GPU parity test)."""
    g = torch.Generator().manual_seed(1)
    T, H, I, E, K = 8, 256, 128, 8, 2
    x = torch.randn(T, H, generator=g).bfloat16().view(torch.uint16).numpy()
    logits = torch.randn(T, E, generator=g).numpy()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[e]) for e in range(E)]
    q2 = [oracle.quant_fp4_weight(w2[e]) for e in range(E)]
    c13, s13 = np.stack([a for a, _ in q13]), np.stack([b for _, b in q13])
    c2, s2 = np.stack([a for a, _ in q2]), np.stack([b for _, b in q2])
    ids, rw = oracle.route(1, logits, None, K)
    r = oracle.moe_layer(mode, x, ids, rw, c13, s13, c2, s2)
    return dict(ids=ids, w=rw, y=r["y_bf16"], c13_sum=np.array([c13.astype(np.uint64).sum()]), s13=s13[0, :4])


def lm_head_small():
    """Output head: 4 token rows against a bf16 [256][512] weight, seed 2, alpha 0.5, temperature 0.8, the last 20 rows
    masked, ids offset 1000: the logits' row sums (fp64 of the fp32 values, rounded to 1e-3), and of the per-quad sampling
    records the parts that do not depend on the accumulation order of a dot product: the ids of the 8 largest."""
    g = torch.Generator().manual_seed(2)
    x = torch.randn(4, 512, generator=g).bfloat16().view(torch.uint16).numpy()
    w = (torch.randn(256, 512, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    logits = oracle.lm_head(w, x, alpha=0.5)
    rec = oracle.sampling_records(logits, 0.8, valid_rows=236, id_offset=1000)
    return dict(row_sums=np.round(logits.astype(np.float64).sum(axis=1), 3), top_ids=rec.view(np.int32)[..., 11:19].copy(),
                zmax=np.round(rec[..., 0].astype(np.float64), 3))


if __name__ == "__main__":
    for mode, name in ((oracle.MODE_MX, "mx"), (oracle.MODE_DS, "ds")):
        np.savez_compressed(os.path.join(HERE, f"config0_{name}.npz"), **config0(mode))
        np.savez_compressed(os.path.join(HERE, f"moe_small_{name}.npz"), **moe_small(mode))
    np.savez_compressed(os.path.join(HERE, "lm_head_small.npz"), **lm_head_small())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
