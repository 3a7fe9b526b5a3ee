"""Child program of test_ep_peer.py: every rank sums seeded partials with the peer-memory all-reduce kernel and checks
them against an fp32 NCCL all-reduce; also through a replayed CUDA graph.  Launched with torch.distributed.run."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402
from __graft_entry__ import load_package  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    pkg = load_package()
    ctx = pkg.Ctx(local)
    ar = pkg.PeerAllReduce(ctx, dist, rank, world)
    rows, width = 64, 7168
    bufs = [ar.buffer((rows, width)) for _ in range(2)]
    out = torch.empty(rows, width, dtype=torch.bfloat16, device="cuda")
    ok = True
    for it in range(6):
        b = bufs[it & 1]                      # a partial buffer is rewritten only after a later call completed
        g = torch.Generator(device="cuda").manual_seed(100 * it + rank)
        b.copy_(torch.randn(rows, width, generator=g, device="cuda").bfloat16())
        ref = b.float().clone()
        dist.all_reduce(ref)
        ar(b, out)
        torch.cuda.synchronize()
        # the kernel adds the bf16 partials in fp32 and rounds once: within one bf16 ulp of the fp32 sum
        ok = ok and bool(((out.float() - ref).abs() <= ref.abs() * 2.0 ** -8 + 1e-6).all()) and ctx.status().code == 0
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ar(bufs[0], out)
        ar(bufs[1], out)
    for _ in range(4):
        graph.replay()                        # the epoch advances on the device
    torch.cuda.synchronize()
    ref = bufs[1].float().clone()
    dist.all_reduce(ref)
    ok = ok and bool(((out.float() - ref).abs() <= ref.abs() * 2.0 ** -8 + 1e-6).all()) and ctx.status().code == 0
    # combine fused with the exchange: every (token, choice) pair lives on exactly one rank
    tokens, topk = rows, 8
    plan = pkg.MoePlan(ctx, tokens, topk, 8, 8)
    g = torch.Generator(device="cuda").manual_seed(7)          # same on every rank
    owner = torch.randint(0, world, (tokens, topk), generator=g, device="cuda")
    rows_of = torch.arange(tokens * topk, device="cuda", dtype=torch.int32).view(tokens, topk)
    plan.pair_row.copy_(torch.where(owner == rank, rows_of, torch.full_like(rows_of, -1)).view(-1))
    gy = torch.Generator(device="cuda").manual_seed(1000 + rank)
    yrows = torch.randn(tokens * topk, width, generator=gy, device="cuda")
    local = torch.where((owner == rank).view(tokens, topk, 1), yrows.view(tokens, topk, width), torch.zeros((), device="cuda")).sum(1)
    ref = local.bfloat16().float()
    dist.all_reduce(ref)
    mag = local.abs()
    dist.all_reduce(mag)     # the partials are rounded to bf16 before they are exchanged: the error scales with their sizes
    for it in range(3):
        ar.combine(plan, yrows, None, bufs[it & 1], out)
        torch.cuda.synchronize()
        ok = ok and bool(((out.float() - ref).abs() <= mag * 2.0 ** -7 + 1e-5).all()) and ctx.status().code == 0
    # the same with the result left quantized for the next projection: codes and scales of act_quant(out), bit for bit
    for mode in (pkg.MODE_DS, pkg.MODE_MX):
        blk = 128 if mode == pkg.MODE_DS else 32
        xq = torch.zeros(tokens, width, dtype=torch.uint8, device="cuda")
        xs = torch.zeros(tokens, width // blk, dtype=torch.float32 if mode == pkg.MODE_DS else torch.uint8, device="cuda")
        ar.combine(plan, yrows, None, bufs[0], out, quant=(mode, xq, xs))
        torch.cuda.synchronize()
        rq, rs = pkg.act_quant(ctx, mode, out)
        torch.cuda.synchronize()
        ok = ok and bool(((out.float() - ref).abs() <= mag * 2.0 ** -7 + 1e-5).all()) and ctx.status().code == 0
        ok = ok and bool((xq == rq).all()) and bool((xs.view(torch.uint8) == rs.view(torch.uint8)).all())
        dist.barrier()      # (bufs[0] is rewritten by the next round only after every rank has read it)
    # all-gather of column slices: rank r fills its own columns, everybody ends up with the same full rows, bit for bit
    gg = torch.Generator(device="cuda").manual_seed(4242)      # same on every rank
    full = torch.randn(rows, width, generator=gg, device="cuda").bfloat16()
    wsl = width // world
    for it in range(3):
        b = bufs[it & 1]
        b.zero_()
        b[:, rank * wsl:(rank + 1) * wsl] = full[:, rank * wsl:(rank + 1) * wsl]
        out.zero_()
        ar.gather_cols(b, out)
        torch.cuda.synchronize()
        ok = ok and bool((out.view(torch.uint16) == full.view(torch.uint16)).all()) and ctx.status().code == 0
    dist.barrier()
    torch.cuda.synchronize()
    print(f"rank {rank}: {'ok' if ok else 'MISMATCH'}", flush=True)
    os._exit(0 if ok else 1)


if __name__ == "__main__":
    main()
