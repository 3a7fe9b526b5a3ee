"""The peer-memory all-reduce kernel of the expert-parallel exchange (csrc/ep_comm.cu, dsuf_ep_allreduce_bf16)."""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _call(pkg, ctx, data, flags, state, out, n):
    lib = pkg.lib()
    ptrs = (C.c_uint64 * 1)(data.data_ptr())
    fl = (C.c_uint64 * 1)(flags.data_ptr())
    return lib.dsuf_ep_allreduce_bf16(ctx.h, ctx.stream(), ptrs, fl, 0, 1, n, state.data_ptr(), out.data_ptr())


def test_single_rank_sum_is_a_copy_and_the_epoch_advances(pkg, ctx):
    """world = 1: the hand-shake is with itself; three calls in a row and a replayed graph keep the flags consistent."""
    n = 64 * 7168
    x = torch.randn(n, device="cuda").bfloat16()
    out = torch.zeros_like(x)
    flags = torch.zeros(pkg.lib().dsuf_ep_flag_bytes(1) // 4, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    for _ in range(3):
        assert _call(pkg, ctx, x, flags, state, out, n) == 0
    torch.cuda.synchronize()
    assert (out.view(torch.uint16) == x.view(torch.uint16)).all()
    assert state.cpu().tolist() == [3, 0] and int(flags.max()) == 3
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        assert _call(pkg, ctx, x, flags, state, out, n) == 0
    for _ in range(4):
        g.replay()
    torch.cuda.synchronize()
    assert state.cpu().tolist()[0] == 7 and ctx.status().code == 0


def test_single_rank_combine_equals_unpermute(pkg, ctx):
    """world = 1: the fused combine is the plain unpermute (sum of the top-k rows, one bf16 round), rows missing on
    this rank (< 0) skipped, optional shared rows added."""
    tokens, topk, h = 24, 4, 512
    plan = pkg.MoePlan(ctx, tokens, topk, 8, 8)
    g = torch.Generator(device="cuda").manual_seed(3)
    pr = torch.randperm(tokens * topk, generator=g, device="cuda").to(torch.int32)
    pr[::5] = -1
    plan.pair_row.copy_(pr)
    yrows = torch.randn(tokens * topk, h, generator=g, device="cuda")
    shared = torch.randn(tokens, h, generator=g, device="cuda").bfloat16()
    want = torch.empty(tokens, h, dtype=torch.bfloat16, device="cuda")
    pkg.moe_unpermute(ctx, plan, yrows, want, shared)
    partial = torch.zeros(tokens, h, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros_like(partial)
    flags = torch.zeros(pkg.lib().dsuf_ep_flag_bytes(1) // 4, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    ptrs, fl = (C.c_uint64 * 1)(partial.data_ptr()), (C.c_uint64 * 1)(flags.data_ptr())
    rc = pkg.lib().dsuf_ep_combine_bf16(ctx.h, ctx.stream(), plan.pair_row.data_ptr(), yrows.data_ptr(), shared.data_ptr(), tokens, topk, h,
                                        ptrs, fl, 0, 1, state.data_ptr(), out.data_ptr())
    torch.cuda.synchronize()
    assert rc == 0 and ctx.status().code == 0
    assert (out.view(torch.uint16) == want.view(torch.uint16)).all()
    assert (partial.view(torch.uint16) == want.view(torch.uint16)).all()


def test_wait_for_a_missing_peer_runs_out_and_reports(pkg, ctx):
    """A peer that never announces: the kernel's wait is given 1 ms, runs out, records a time-out (kernel id 5) in the
    status word and returns; the context stays usable and the next call, whose peer flag is present, sums both
    partials.  Both "ranks" live on this GPU (world = 2 with local buffers), nothing faults and nothing waits for long."""
    lib = pkg.lib()
    n = 16 * 1024
    g = torch.Generator(device="cuda").manual_seed(9)
    mine = torch.randn(n, generator=g, device="cuda").bfloat16()
    peer = torch.randn(n, generator=g, device="cuda").bfloat16()
    out = torch.zeros_like(mine)
    nflag = lib.dsuf_ep_flag_bytes(2) // 4
    my_flags = torch.zeros(nflag, dtype=torch.int32, device="cuda")
    peer_flags = torch.zeros(nflag, dtype=torch.int32, device="cuda")   # where this rank announces itself; nobody reads it
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    data = (C.c_uint64 * 2)(mine.data_ptr(), peer.data_ptr())
    flags = (C.c_uint64 * 2)(my_flags.data_ptr(), peer_flags.data_ptr())
    ctx.set_wait_budget_us(1000)
    try:
        rc = lib.dsuf_ep_allreduce_bf16(ctx.h, ctx.stream(), data, flags, 0, 2, n, state.data_ptr(), out.data_ptr())
        assert rc == 0
        st = pkg.DevStatus()
        rc = lib.dsuf_status_poll(ctx.h, ctx.stream(), C.byref(st))
        assert rc == -3 and st.code == 1 and st.kernel == 5      # DSUF_E_TIMEOUT, a bounded wait expired, the exchange kernel
        assert state.cpu().tolist() == [1, 0]                    # the call is over and counted
        # the peer "arrives" for the second call: its announcements of epoch 2 appear in this rank's flag block
        my_flags.view(-1, 2)[:, 1] = 2
        torch.cuda.synchronize()
        rc = lib.dsuf_ep_allreduce_bf16(ctx.h, ctx.stream(), data, flags, 0, 2, n, state.data_ptr(), out.data_ptr())
        assert rc == 0 and ctx.status().code == 0
        want = (mine.float() + peer.float()).bfloat16()
        assert (out.view(torch.uint16) == want.view(torch.uint16)).all()
        # a peer that is more than one call ahead is reported, not summed in silence
        my_flags.view(-1, 2)[:, 1] = 7
        torch.cuda.synchronize()
        rc = lib.dsuf_ep_allreduce_bf16(ctx.h, ctx.stream(), data, flags, 0, 2, n, state.data_ptr(), out.data_ptr())
        assert rc == 0
        rc = lib.dsuf_status_poll(ctx.h, ctx.stream(), C.byref(st))
        assert rc == -3 and st.code == 3 and st.kernel == 5
    finally:
        ctx.set_wait_budget_us(2000000)


def test_rejects_aliasing_and_bad_sizes(pkg, ctx):
    x = torch.zeros(64, device="cuda").bfloat16()
    flags = torch.zeros(pkg.lib().dsuf_ep_flag_bytes(1) // 4, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    assert _call(pkg, ctx, x, flags, state, x, 64) != 0          # out must not be the partial the peers read
    assert _call(pkg, ctx, x, flags, state, torch.empty_like(x), 60) != 0   # n_elems % 8


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_against_nccl():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29577", os.path.join(HERE, "ep_peer_check.py")], env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
