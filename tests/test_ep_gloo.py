"""Expert-parallel exchange on CPU: two gloo ranks run ep.ep_layer_forward with the oracle as the compute steps and must
reproduce the single-rank layer (output-sharded dense + all-gather = dispatch, or the replicated dense projection of the
decode sizes; expert shards; all-reduce = combine)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
T, H, I, E, K = 8, 256, 128, 8, 2


def _inputs():
    import oracle
    g = torch.Generator().manual_seed(11)
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    wd = (torch.randn(H, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w13 = (torch.randn(E, 2 * I, H, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    w2 = (torch.randn(E, H, I, generator=g) * 0.05).bfloat16().view(torch.uint16).numpy()
    q13 = [oracle.quant_fp4_weight(w13[e]) for e in range(E)]
    q2 = [oracle.quant_fp4_weight(w2[e]) for e in range(E)]
    return dict(x=x, logits=logits, wd=wd, c13=np.stack([a for a, _ in q13]), s13=np.stack([b for _, b in q13]),
                c2=np.stack([a for a, _ in q2]), s2=np.stack([b for _, b in q2]))


class OracleCompute:
    def __init__(self, inp, rank, world, dense_replicated=False):
        import oracle
        from __graft_entry__ import load_package
        import importlib
        self.o, self.inp, self.rank, self.world = oracle, inp, rank, world
        ep = importlib.import_module(load_package().__name__ + ".ep")
        self.dense_replicated = dense_replicated    # every rank computes the whole h; the layer skips the gather
        self.n0, self.n1 = (0, H) if dense_replicated else ep.shard_bounds(H, world, rank)
        self.e0, self.e1 = ep.shard_bounds(E, world, rank)
        self.t0, self.t1 = ep.shard_bounds(T, world, rank)
        self.wq, self.ws = oracle.quant_fp8_weight(oracle.MODE_DS, np.ascontiguousarray(inp["wd"][self.n0:self.n1]))

    def dense_slice(self, x_all):
        o = self.o
        xq, xsc = o.act_quant(o.MODE_DS, np.ascontiguousarray(x_all.view(torch.uint16).numpy()))
        ob, _ = o.gemm_fp8(o.MODE_DS, self.wq, self.ws, xq, xsc)
        self.h = torch.zeros(T, H, dtype=torch.bfloat16)
        self.h[:, self.n0:self.n1] = torch.from_numpy(ob.view(np.int16)).view(torch.bfloat16)
        return self.h

    def route(self, h_all):
        ids, w = self.o.route(1, self.inp["logits"].numpy(), None, K)
        return torch.from_numpy(ids), torch.from_numpy(w)

    def experts_partial(self, h_all, ids_all, w_all):
        o, inp = self.o, self.inp
        r = o.moe_layer(o.MODE_DS, h_all.view(torch.uint16).numpy(), ids_all.numpy(), w_all.numpy(), inp["c13"], inp["s13"],
                        inp["c2"], inp["s2"], e_lo=self.e0, e_hi=self.e1)
        return torch.from_numpy(r["y_bf16"].view(np.int16)).view(torch.bfloat16)


def _worker(rank, world, port, out_dir, dense_replicated=False):
    sys.path.insert(0, ROOT)
    import importlib
    import torch.distributed as dist
    from __graft_entry__ import load_package
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ep = importlib.import_module(load_package().__name__ + ".ep")
    inp = _inputs()
    xch = ep.Exchange(dist, rank, world)
    t0, t1 = ep.shard_bounds(T, world, rank)
    comp = OracleCompute(inp, rank, world, dense_replicated)
    x_all = xch.all_gather_rows(torch.empty(T, H, dtype=torch.bfloat16), inp["x"][t0:t1].contiguous())
    y = ep.ep_layer_forward(xch, comp, x_all)
    torch.save((comp.h.clone(), y.clone()), os.path.join(out_dir, f"y{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("dense_replicated", [False, True])
def test_two_rank_layer_equals_single_rank(tmp_path, dense_replicated):
    sys.path.insert(0, ROOT)
    import importlib
    from __graft_entry__ import load_package
    ep = importlib.import_module(load_package().__name__ + ".ep")
    inp = _inputs()
    one = OracleCompute(inp, 0, 1)
    ep.ep_layer_forward(ep.Exchange(None, 0, 1), one, inp["x"].clone())
    ref_h = one.h.float()
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, str(tmp_path), dense_replicated), nprocs=2, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"y{r}.pt")) for r in range(2)]
    h2, y2 = parts[0][0], parts[0][1].float()
    assert (parts[1][0] == h2).all() and (parts[1][1].float() == y2).all()   # every rank holds the same full rows
    # 1) output-sharded dense + all-gather: the unsharded projection, bit for bit (nothing is summed across ranks;
    #    the weight's 128 x 128 scale blocks do not straddle the shard boundary)
    assert (h2.view(torch.uint16) == one.h.view(torch.uint16)).all()
    # 2) dispatch / expert shards / combine: equal to the unsharded expert layer evaluated on the SAME h
    #    (FP8 re-quantization makes the layer discontinuous in h, so the comparison must not mix the two h's)
    ids, w = one.route(None)
    y_ref = one.experts_partial(h2, ids, w).float()
    err = (y2 - y_ref).norm() / y_ref.norm()
    assert err < 5e-3, err
    assert y_ref.abs().max() > 0


def test_shard_bounds_reject_uneven_splits():
    sys.path.insert(0, ROOT)
    import importlib
    from __graft_entry__ import load_package
    ep = importlib.import_module(load_package().__name__ + ".ep")
    assert ep.shard_bounds(256, 8, 3) == (96, 128)
    with pytest.raises(ValueError):
        ep.shard_bounds(10, 4, 0)


def test_exchange_routes_registered_buffers_through_the_peer_kernel():
    """Host logic of the GPU exchange, with stand-ins for the process group and the peer-memory kernel: a registered
    partial buffer is summed by the peer callable into its result tensor, a tensor that a fused compute + exchange
    kernel has already summed passes through untouched, anything else goes to the process group."""
    sys.path.insert(0, ROOT)
    import importlib
    from __graft_entry__ import load_package
    ep = importlib.import_module(load_package().__name__ + ".ep")

    class FakeDist:
        def __init__(self):
            self.calls = 0

        def all_reduce(self, t, group=None):
            self.calls += 1
            t.mul_(2)   # "sum over two ranks holding the same values"

    peer_calls = []

    def peer(partial, out):
        peer_calls.append((partial.data_ptr(), out.data_ptr()))
        out.copy_(partial * 2)
        return out

    dist = FakeDist()
    xch = ep.Exchange(dist, 0, 2, peer=peer)
    partial, result, fused, other = (torch.ones(4) * v for v in (1.0, 0.0, 5.0, 3.0))
    xch.peer_out[partial.data_ptr()] = result
    xch.reduced.add(fused.data_ptr())
    r = xch.all_reduce(partial)
    assert r is result and torch.equal(result, torch.full((4,), 2.0)) and torch.equal(partial, torch.ones(4))
    assert xch.all_reduce(fused) is fused and torch.equal(fused, torch.full((4,), 5.0))
    assert xch.all_reduce(other) is other and torch.equal(other, torch.full((4,), 6.0))
    assert dist.calls == 1 and len(peer_calls) == 1
    # without a peer kernel every tensor goes to the process group; a single rank does nothing at all
    xch2 = ep.Exchange(dist, 0, 2)
    assert xch2.all_reduce(partial) is partial and dist.calls == 2
    assert ep.Exchange(dist, 0, 1, peer=peer).all_reduce(other) is other and dist.calls == 2
