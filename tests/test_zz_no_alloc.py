"""dsuf_gemm_fp8_static: the GEMV entry point for callers that cannot allocate device memory (an engine that gave its
whole device budget to one start-up arena, a plugin without an allocator of its own).  Its stream-K scratch is a fixed
array inside the library, shared by all calls and never cleared between them except for the arrival counters, so the
check is: two calls in a row -- on different weights, the second one after the first has left its partial sums and
counters behind -- each give exactly what the workspace-taking entry point gives."""
import numpy as np
import pytest
import torch

import oracle
from conftest import randn_bf16, seeded

pytestmark = pytest.mark.gpu


def _weight(pkg, ctx, n, k, seed):
    g = seeded(seed)
    _, wn = randn_bf16(g, n, k, std=0.02)
    wq, ws = oracle.quant_fp8_weight(1, wn)
    return pkg.Weight.dense_fp8(ctx, 1, wq, ws), g


def test_static_scratch_matches_workspace_entry_twice_in_a_row(pkg, ctx):
    # shapes whose row tiles are split across CTAs (partials + counters in use) and a second, different shape
    # (the third: more than 64 token rows, which take the tile-pair kernel and leave the scratch alone)
    cases = [(1024, 2048, 4, 21), (384, 4096, 9, 22)] + ([(512, 1024, 100, 23)] if ctx.tcgen05 else [])
    for rep in range(2):
        for n, k, m, seed in cases:
            w, g = _weight(pkg, ctx, n, k, seed)
            xt, _ = randn_bf16(g, m, k)
            xq, xs = pkg.act_quant(ctx, 1, xt.cuda())
            want = pkg.gemm_fp8(ctx, w, xq, xs, m)
            got = pkg.gemm_fp8_static(ctx, w, xq, xs, m)
            torch.cuda.synchronize()
            assert ctx.status().code == 0
            a, b = got.float().cpu().numpy(), want.float().cpu().numpy()
            rel = np.linalg.norm(a - b) / np.linalg.norm(b)
            assert rel < 1e-2, (rep, n, k, rel)          # the tolerance of the parity tests
            assert (got.view(torch.uint16) == want.view(torch.uint16)).all()  # and in fact the same bits


def test_static_scratch_rejects_what_does_not_fit(pkg, ctx):
    # 1025 row tiles: one more than the built-in scratch holds.  Only the descriptor is needed, nothing is launched.
    n, k = 1025 * 128, 128
    tiles = torch.zeros(pkg.lib().dsuf_packed_bytes(pkg.FMT_FP8, pkg.MODE_DS, n, k), dtype=torch.uint8, device="cuda")
    sds = torch.ones(n // 128, 1, dtype=torch.float32, device="cuda")
    w = pkg.Weight(ctx, pkg.FMT_FP8, pkg.MODE_DS, n, k, 1, False, tiles, sds)
    xq = torch.zeros(1, k, dtype=torch.uint8, device="cuda")
    xs = torch.ones(1, 1, dtype=torch.float32, device="cuda")
    with pytest.raises(pkg.DsufError, match="row tiles"):
        pkg.gemm_fp8_static(ctx, w, xq, xs, 1)
