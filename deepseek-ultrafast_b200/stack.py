"""The benchmark's layer stack: per layer one FP8 dense projection (hidden x hidden) followed by the routed-expert
FFN (route -> plan -> gather+quant -> gate/up+SwiGLU -> quant -> down -> unpermute/combine).

Single GPU: every expert is local.  Several GPUs (one process each, torch.distributed over NCCL): experts are
sharded world-ways (rank r owns experts [r*E/W, (r+1)*E/W)), tokens are data parallel (rank r owns T/W of them);
per layer the exchanges are an all-gather of the column slices of the output-sharded dense projection, which delivers
every token row to every expert owner (dispatch), and the sum of the per-rank expert outputs (combine), which also is the
next layer's input (ep.py).
The reference is tensor-parallel only and combines with its own push all-reduce (cu/comm.cu:134-279); the
expert-parallel exchange here is this library's design.
"""
import os
import sys

from . import (MODE_DS, MODE_MX, SCORE_SOFTMAX, MoeLayer, Weight, act_quant, gemm_fp8, moe_route_tokens)
from . import synth


class StackConfig:
    def __init__(self, hidden=7168, inter=2048, n_experts=256, topk=8, layers=4, tokens=64, act_mode=MODE_DS,
                 dense_mode=MODE_DS, std=0.02, seed=0):
        self.hidden, self.inter, self.n_experts, self.topk = hidden, inter, n_experts, topk
        self.layers, self.tokens, self.act_mode, self.dense_mode, self.std, self.seed = layers, tokens, act_mode, dense_mode, std, seed


class LayerStack:
    """Single-GPU stack (world size 1).  All buffers are allocated here; ``forward`` only launches kernels."""

    def __init__(self, ctx, cfg, weights_from=None):
        """``weights_from``: another LayerStack of the same shapes whose weights are shared (a prefill-size stack next to
        a decode-size one); the routing logits are drawn for this stack's token count."""
        t = ctx.torch
        dev = ctx.device
        self.ctx, self.cfg = ctx, cfg
        H, I, E = cfg.hidden, cfg.inter, cfg.n_experts
        self.dense, self.moe, self.logits = [], [], []
        # decode: 8-row slots; prefill (tens of rows per expert and more): 128-row tiles (tcgen05 path only)
        tile_rows = 128 if ctx.tcgen05 and cfg.tokens * cfg.topk >= 32 * E else 8
        for l in range(cfg.layers):
            if weights_from is not None:
                self.dense.append(weights_from.dense[l])
                W13, W2 = weights_from.moe[l].w13, weights_from.moe[l].w2
            else:
                tiles, sds = synth.fp8_dense(t, cfg.dense_mode == MODE_MX, H, H, cfg.std, cfg.seed + 1000 * l + 1, dev)
                self.dense.append(Weight(ctx, 0, cfg.dense_mode, H, H, 1, False, tiles, sds))
                w13 = synth.fp4_experts(t, E, 2 * I, H, cfg.std, cfg.seed + 1000 * l + 2, True, dev)
                w2 = synth.fp4_experts(t, E, H, I, cfg.std, cfg.seed + 1000 * l + 3, False, dev)
                W13 = Weight.experts_fp4_packed(ctx, w13, 2 * I, H, E, True)
                W2 = Weight.experts_fp4_packed(ctx, w2, H, I, E, False)
            self.moe.append(MoeLayer(ctx, W13, W2, cfg.tokens, cfg.topk, cfg.act_mode, tile_rows=tile_rows))
            g = t.Generator(device=dev).manual_seed(cfg.seed + 1000 * l + 4)
            self.logits.append(t.randn(cfg.tokens, E, generator=g, device=dev, dtype=t.float32))
        blk = 32 if cfg.dense_mode == MODE_MX else 128
        self.xq = t.empty((cfg.tokens, H), dtype=t.uint8, device=dev)
        self.xs = t.empty((cfg.tokens, H // blk), dtype=t.uint8 if cfg.dense_mode == MODE_MX else t.float32, device=dev)
        self.h = t.empty((cfg.tokens, H), dtype=t.bfloat16, device=dev)
        self.y = [t.empty((cfg.tokens, H), dtype=t.bfloat16, device=dev) for _ in range(2)]
        self.ids = t.empty((cfg.tokens, cfg.topk), dtype=t.int32, device=dev)
        self.w = t.empty((cfg.tokens, cfg.topk), dtype=t.float32, device=dev)
        self.fuse_quant = H % 128 == 0 and os.environ.get("DSUF_FUSE_QUANT", "1") != "0"

    def dense_forward(self, l, x, out, prequantized=False):
        """x bf16 [T][H] -> out bf16 [T][H]; processed in slabs of the decode kernel's row limit (64 tcgen05, 16 mma.sync).
        ``prequantized``: self.xq / self.xs already hold x's codes and scales (the previous layer's unpermute wrote them)."""
        ctx, w = self.ctx, self.dense[l]
        if not prequantized:
            act_quant(ctx, w.mode, x, self.xq, self.xs)
        T = x.shape[0]
        if ctx.tcgen05:
            return gemm_fp8(ctx, w, self.xq, self.xs, T, out)   # one launch: decode kernel up to 64 rows, prefill kernel above
        slab = 64 if ctx.tcgen05 else 16
        for r0 in range(0, T, slab):
            m = min(slab, T - r0)
            gemm_fp8(ctx, w, self.xq[r0:r0 + m], self.xs[r0:r0 + m], m, out[r0:r0 + m])
        return out

    def forward(self, x, events=None, layers=None):
        cfg = self.cfg
        cur = x
        n_layers = cfg.layers if layers is None else layers
        for l in range(n_layers):
            self.dense_forward(l, cur, self.h, prequantized=l > 0 and self.fuse_quant)
            out = self.y[l & 1]
            # router inside the layer: decode-size batches take one launch for router + plan + gather/quant; the unpermute
            # leaves its result quantized for the next layer's projection
            oq = (cfg.dense_mode, self.xq, self.xs) if self.fuse_quant and l + 1 < n_layers else None
            self.moe[l].forward(self.h, self.ids, self.w, out, events=events, route=(SCORE_SOFTMAX, self.logits[l], None, 1.0), out_quant=oq)
            cur = out
        return cur

    def count_launches(self):
        cfg = self.cfg
        slab = 64 if self.ctx.tcgen05 else 16
        slabs = (cfg.tokens + slab - 1) // slab
        if self.ctx.tcgen05:
            slabs = 1
        # act_quant + dense slabs + front end (router + plan + gather/quant: 1 launch up to 1024 pairs, else 1 + 3 + 1)
        # + w13 + quant + w2 + unpermute
        front = 1 if cfg.tokens * cfg.topk <= 1024 else 5
        quants = 1 if self.fuse_quant else cfg.layers     # only the first layer quantizes its input by itself
        return cfg.layers * (slabs + front + 1 + 1 + 1 + 1) + quants


class _KernelCompute:
    """The three compute steps of ep.ep_layer_forward on this library's CUDA kernels."""

    def __init__(self, stack, l):
        self.s, self.l = stack, l
        self.dense_replicated = stack.dense_replicated

    def dense_slice(self, x_all):
        s, w = self.s, self.s.dense[self.l]
        ctx = s.ctx
        n0, n1 = s.nslice
        if s.prequantized is not x_all:   # (the previous layer's combine may have left x_all quantized in s.xq / s.xs)
            act_quant(ctx, w.mode, x_all, s.xq, s.xs)
        s.prequantized = None
        T = x_all.shape[0]
        if ctx.tcgen05:
            gemm_fp8(ctx, w, s.xq, s.xs, T, s.partial[:, n0:n1])   # decode kernel up to 64 rows, prefill kernel above
            return s.partial
        for r0 in range(0, T, 16):
            m = min(16, T - r0)
            gemm_fp8(ctx, w, s.xq[r0:r0 + m], s.xs[r0:r0 + m], m, s.partial[r0:r0 + m, n0:n1])
        return s.partial

    def route(self, h_all):
        """The router runs inside the expert step (one launch with the plan and the gather/quant); this hands out the
        buffers it fills."""
        s = self.s
        return s.ids, s.w

    def experts_partial(self, h_all, ids_all, w_all):
        s = self.s
        part = s.y_part[self.l & 1]
        route = (SCORE_SOFTMAX, s.logits[self.l], None, 1.0)
        if s.peer is not None and s.fuse_combine:
            # one kernel: local sum of the top-k rows into the mapped partial buffer, hand-shake, sum over the ranks
            out = s.xch.peer_out[part.data_ptr()]
            # the result is the next layer's input: the combine leaves it quantized for that layer's dense projection
            quant = (s.cfg.dense_mode, s.xq, s.xs) if s.fuse_quant and self.l + 1 < s.cfg.layers else None

            def combine(plan, yrows, shared):
                y = s.peer.combine(plan, yrows, shared, part, out, quant=quant)
                s.prequantized = y if quant is not None else None
                return y
            return s.moe[self.l].forward(h_all, ids_all, w_all, part, route=route, combine=combine)
        return s.moe[self.l].forward(h_all, ids_all, w_all, part, route=route)


class EpLayerStack:
    """The layer stack on `world` GPUs, one process each (see ep.py for the sharding and the exchanges)."""

    def __init__(self, ctx, cfg, dist, rank, world):
        from . import ep
        t = ctx.torch
        dev = ctx.device
        self.ctx, self.cfg, self.rank, self.world = ctx, cfg, rank, world
        self.xch = ep.Exchange(dist, rank, world)
        H, I, E, T = cfg.hidden, cfg.inter, cfg.n_experts, cfg.tokens
        # decode: 8-row slots; prefill-size batches (tens of rows per expert and more): 128-row tiles (tcgen05 path only)
        tile_rows = 128 if ctx.tcgen05 and T * cfg.topk >= 32 * E else 8
        self.large = tile_rows == 128
        # decode-size batches: every rank holds the whole dense weight and computes the whole h (one exchange per layer
        # less, see ep.py); DSUF_EP_DENSE=shard keeps the output-sharded projection + gather at every size
        self.dense_replicated = world > 1 and not self.large and os.environ.get("DSUF_EP_DENSE", "replicate") != "shard"
        # this rank's output columns of the dense projection
        self.nslice = (0, H) if self.dense_replicated else ep.shard_bounds(H, world, rank)
        if (self.nslice[1] - self.nslice[0]) % 128:
            raise ValueError("hidden / world must be a multiple of 128")
        self.e_lo, e_hi = ep.shard_bounds(E, world, rank)
        self.t0, self.t1 = ep.shard_bounds(T, world, rank)
        n_loc, nloc_d = e_hi - self.e_lo, self.nslice[1] - self.nslice[0]
        self.dense, self.moe, self.logits = [], [], []
        for l in range(cfg.layers):
            # the shards of ONE set of random-init weights (the seeds of LayerStack): the dense weight's rows of this rank's
            # output columns and the experts at their global ids, so the W-rank result is comparable with the single-GPU one
            base = cfg.seed + 1000 * l
            tiles, sds = synth.fp8_dense(t, cfg.dense_mode == MODE_MX, H, H, cfg.std, base + 1, dev, n_slice=self.nslice)
            self.dense.append(Weight(ctx, 0, cfg.dense_mode, nloc_d, H, 1, False, tiles, sds))
            w13 = synth.fp4_experts(t, n_loc, 2 * I, H, cfg.std, base + 2, True, dev, first_expert=self.e_lo)
            w2 = synth.fp4_experts(t, n_loc, H, I, cfg.std, base + 3, False, dev, first_expert=self.e_lo)
            W13 = Weight.experts_fp4_packed(ctx, w13, 2 * I, H, n_loc, True)
            W2 = Weight.experts_fp4_packed(ctx, w2, H, I, n_loc, False)
            self.moe.append(MoeLayer(ctx, W13, W2, T, cfg.topk, cfg.act_mode, e_lo=self.e_lo, tile_rows=tile_rows))
            g = t.Generator(device=dev).manual_seed(cfg.seed + 1000 * l + 4)   # same logits on every rank
            self.logits.append(t.randn(T, E, generator=g, device=dev, dtype=t.float32))
        blk = 32 if cfg.dense_mode == MODE_MX else 128
        self.xq = t.empty((T, H), dtype=t.uint8, device=dev)
        self.xs = t.empty((T, H // blk), dtype=t.uint8 if cfg.dense_mode == MODE_MX else t.float32, device=dev)
        # The two per-layer sums run as the library's peer-memory all-reduce when the partial buffers can be mapped
        # by every rank (torch symmetric memory); DSUF_EP_PEER=0 or a failed mapping falls back to NCCL.
        self.peer, self.fuse_combine, self.peer_error = None, False, None
        if world > 1 and os.environ.get("DSUF_EP_PEER", "1") != "0":
            try:
                from . import PeerAllReduce
                self.peer = PeerAllReduce(ctx, dist, rank, world)
            except Exception as e:  # noqa: BLE001 - any failure to map means: use the process group
                self.peer_error = f"{type(e).__name__}: {e}"
                print(f"rank {rank}: peer-memory all-reduce unavailable ({self.peer_error}); using NCCL", file=sys.stderr)
                self.peer = None
        if world > 1 and hasattr(dist, "ReduceOp"):
            # every rank must take the same path: one rank that could not map its buffers sends all of them to NCCL
            agreed = t.tensor([1 if self.peer is not None else 0], dtype=t.int32, device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if int(agreed.item()) == 0:
                self.peer = None
        if self.peer is not None:
            # the ranks of this stack run in lock step (one captured graph each, replayed together): a peer that is half a
            # second late is a failed peer, and the kernels report it instead of waiting for the library's default 2 s
            ctx.set_wait_budget_us(500000)
            self.partial = self.peer.buffer((T, H))
            self.y_part = [self.peer.buffer((T, H)) for _ in range(2)]
            self.xch.peer = self.peer
            for buf in [self.partial] + self.y_part:
                self.xch.peer_out[buf.data_ptr()] = t.empty((T, H), dtype=t.bfloat16, device=dev)
            # prefill-size batches: unpermute, then the two-shot all-reduce (reduce-scatter + gather) over a second mapped
            # buffer per partial; decode-size batches: the one-shot combine fused with the unpermute
            self.fuse_combine = os.environ.get("DSUF_EP_FUSE_COMBINE", "1") != "0" and not self.large
            if self.large:
                for buf in self.y_part:
                    self.peer.stage_for(buf)
            if self.fuse_combine:
                for buf in self.y_part:
                    self.xch.reduced.add(self.xch.peer_out[buf.data_ptr()].data_ptr())
        else:
            self.partial = t.empty((T, H), dtype=t.bfloat16, device=dev)
            self.y_part = [t.empty((T, H), dtype=t.bfloat16, device=dev) for _ in range(2)]
        self.prequantized = None   # the tensor whose FP8 codes / scales self.xq / self.xs currently hold, if any
        self.fuse_quant = os.environ.get("DSUF_EP_FUSE_QUANT", "1") != "0"
        self.x_all = t.empty((T, H), dtype=t.bfloat16, device=dev)
        self.ids = t.empty((T, cfg.topk), dtype=t.int32, device=dev)
        self.w = t.empty((T, cfg.topk), dtype=t.float32, device=dev)
        self.compute = [_KernelCompute(self, l) for l in range(cfg.layers)]

    def logits_full(self, l):
        return self.logits[l]

    def exchange_path(self):
        """Which code sums the per-rank partials: "peer_fused" (this library's kernels over peer memory, the combine fused
        with the unpermute), "peer" (this library's all-reduce kernel, unpermute separate) or "nccl"."""
        if self.peer is None:
            return "nccl"
        return "peer_fused" if self.fuse_combine else "peer"

    def forward(self, x_local, events=None, layers=None):
        """x_local bf16 [T/W][H] (this rank's tokens) -> this rank's rows of the stack output (after ``layers`` layers,
        default all)."""
        from . import ep
        cur = self.xch.all_gather_rows(self.x_all, x_local)
        self.prequantized = None
        for l in range(self.cfg.layers if layers is None else layers):
            self.moe[l].events = events
            cur = ep.ep_layer_forward(self.xch, self.compute[l], cur)
        return cur[self.t0:self.t1]

    def count_launches(self):
        cfg = self.cfg
        slabs = 1 if self.ctx.tcgen05 else (cfg.tokens + 15) // 16
        front = 1 if cfg.tokens * cfg.topk <= 1024 else 5
        # this library's exchange kernels (NCCL's kernels are not counted): the gather of the dense slices (none when the
        # projection is replicated), and the combine that either replaces the unpermute (one fused kernel) or follows it as
        # an all-reduce (one kernel; two -- reduce-scatter and gather -- for prefill-size batches)
        unperm = 0 if self.peer is not None and self.fuse_combine else 1
        xchg = 0 if self.peer is None else 2 if self.large and not self.fuse_combine else 1
        gather = 1 if self.peer is not None and not self.dense_replicated else 0
        # the fused combine leaves its result quantized: only the first layer quantizes its dense input by itself
        quants = 1 if self.peer is not None and self.fuse_combine and self.fuse_quant else cfg.layers
        return cfg.layers * (slabs + front + 1 + 1 + 1 + unperm + xchg + gather) + quants
