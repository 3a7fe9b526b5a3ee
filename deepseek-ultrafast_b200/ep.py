"""Expert-parallel / tensor-parallel exchange of the layer stack over torch.distributed (NCCL on GPUs, gloo in CPU tests).

Sharding (world size W, rank r):
    tokens   data parallel at the ends of the stack: rank r owns rows [r*T/W, (r+1)*T/W) of the input and of the output
    dense    OUTPUT-sharded FP8 projection: rank r holds rows [r*H/W, (r+1)*H/W) of the weight and computes those
             columns of h for all T tokens from the full input rows (complete dot products: nothing to sum across ranks)
    experts  rank r owns experts [r*E/W, (r+1)*E/W)
Per layer, two fixed-size exchanges, neither of which needs a host-side count (so the step stays graph-capturable):
    all_gather(h column slices)  every rank ends up with all T rows of h, which IS the dispatch: the token rows are now at
                                 every expert owner.  Each rank receives (W-1)/W of T*H*2 bytes.
    all_reduce(y partials)       combine: per-rank partial sums over local experts; the result doubles as the next
                                 layer's (full) input
At decode sizes (64 tokens x 7168 x bf16 = 0.9 MB) this is the dense, padded form of the dispatch/combine all-to-all:
with top-8 of 256 experts over <= 8 ranks a token reaches 5.25 of 8 ranks on average, so sending every row everywhere
costs < 40 % extra on a sub-megabyte message and removes the count exchange and two collective launches per layer.
Sharding the projection by output columns instead of by K (what the reference's tensor parallelism does for its
projections, crates/engine/src/weights.rs:384-395) makes the first exchange a gather instead of a sum -- an eighth of
the bytes on eight ranks -- and the sharded h equal to the unsharded one bit for bit.
Routing is evaluated redundantly on every rank from the gathered rows (64 x 256 scores).
At decode sizes the stack REPLICATES the dense projection instead (``dense_replicated``): 51 MB of FP8 weights stream from
this GPU's HBM in less time than one hand-shake over NVLink takes (~8 us against ~13 us), every rank computes the
identical h, and the layer is left with a single exchange (the combine).  Prefill-size batches keep the output-sharded
projection and its gather, where the GEMM time, not the latency, is what counts.
The reference has no expert parallelism (tensor parallel + its own push all-reduce,
crates/kernels/cu/comm.cu:134-279); this exchange is this library's design.  On GPUs both exchanges run as this
library's own one-shot kernels over NVLink peer memory (csrc/ep_comm.cu) when torch's symmetric memory can map the
buffers, else as NCCL collectives.

The compute steps are injected (``compute``) so the same exchange code runs on the CUDA kernels (stack.EpLayerStack)
and, in the CPU tests, on the oracle.
"""


class Exchange:
    """Thin wrapper over a torch.distributed process group with the two collectives the layer needs."""

    def __init__(self, dist, rank, world, group=None, peer=None):
        """``peer``: optional callable (partial, out) -> out that sums a partial buffer over the ranks without the
        process-group library (the peer-memory all-reduce kernel); ``peer_out`` maps a partial buffer to its result
        tensor."""
        self.dist, self.rank, self.world, self.group = dist, rank, world, group
        self.peer, self.peer_out = peer, {}
        self.reduced = set()   # data pointers of tensors a fused compute + exchange kernel has already summed over the ranks

    def all_gather_rows(self, out, local):
        """out [W*n][...] <- concatenation of every rank's local [n][...]."""
        if self.world == 1:
            out.copy_(local)
            return out
        self.dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out

    def all_gather_cols(self, t):
        """t [T][H]: every rank has written its own column slice [r*H/W, (r+1)*H/W); returns a tensor holding all slices
        (``t`` itself on the process-group path)."""
        if self.world > 1:
            out = self.peer_out.get(t.data_ptr()) if self.peer is not None else None
            if out is not None:
                return self.peer.gather_cols(t, out)
            w = t.shape[1] // self.world
            mine = t[:, self.rank * w:(self.rank + 1) * w].contiguous()
            parts = [t.new_empty(mine.shape) for _ in range(self.world)]
            self.dist.all_gather(parts, mine, group=self.group)
            for r, p in enumerate(parts):
                t[:, r * w:(r + 1) * w].copy_(p)
        return t

    def all_reduce(self, t):
        """Element-wise sum over ranks; returns the tensor that holds it (``t`` itself on the process-group path)."""
        if self.world > 1:
            if t.data_ptr() in self.reduced:
                return t
            out = self.peer_out.get(t.data_ptr()) if self.peer is not None else None
            if out is not None:
                return self.peer(t, out)
            self.dist.all_reduce(t, group=self.group)
        return t


def shard_bounds(total, world, rank):
    """Even split; ``total`` must divide by ``world`` (tokens, experts and the dense K are chosen that way)."""
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    n = total // world
    return rank * n, (rank + 1) * n


def ep_layer_forward(xch, compute, x_all):
    """One layer on one rank; x_all [T][H] holds ALL token rows (identical on every rank).  ``compute`` provides
         dense_slice(x_all) -> h [T][H] with this rank's column slice filled in (all tokens; overwritten in place);
                               with ``compute.dense_replicated`` set, the whole h (every rank holds the whole dense
                               weight and the gather is skipped)
         route(h_all) -> (ids [T][k], w [T][k])
         experts_partial(h_all, ids, w) -> y partial [T][H] over this rank's experts only (overwritten in place)
    Returns y [T][H], again identical on every rank."""
    h = compute.dense_slice(x_all)
    h_all = h if getattr(compute, "dense_replicated", False) else xch.all_gather_cols(h)
    ids, w = compute.route(h_all)
    return xch.all_reduce(compute.experts_partial(h_all, ids, w))
