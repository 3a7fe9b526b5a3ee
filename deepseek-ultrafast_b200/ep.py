"""Expert-parallel / tensor-parallel exchange of the layer stack over torch.distributed (NCCL on GPUs, gloo in CPU tests).

Sharding (world size W, rank r):
    tokens   data parallel: rank r owns rows [r*T/W, (r+1)*T/W) of every activation
    dense    K-sharded FP8 projection: rank r holds W_dense[:, r*H/W:(r+1)*H/W]; partial products are summed across ranks
    experts  rank r owns experts [r*E/W, (r+1)*E/W)
Per layer, four fixed-size collectives, none of which needs a host-side count (so the step stays graph-capturable):
    all_gather(x)            every rank sees all T token rows for its K-slice of the dense projection
    reduce_scatter(partial)  the tensor-parallel all-reduce, split so each rank keeps only its own token rows
    all_gather(h, ids, w)    dispatch: token rows + routing to the expert owners (a token travels once per rank)
    reduce_scatter(y)        combine: per-rank partial sums over local experts back to the token owners
The last two are the dense, padded form of the dispatch/combine all-to-all: at decode sizes (64 tokens, top-8 of 256
over <= 8 ranks) a token reaches 5.25 of 8 ranks on average, so padding costs < 40 % of a sub-megabyte message and
removes the count exchange.  The reference has no expert parallelism (tensor parallel + its own push all-reduce,
crates/kernels/cu/comm.cu:134-279); this exchange is this library's design.

The compute steps are injected (``compute``) so the same exchange code runs on the CUDA kernels (stack.EpLayerStack)
and, in the CPU tests, on the oracle.
"""


class Exchange:
    """Thin wrapper over a torch.distributed process group with the two collectives the layer needs."""

    def __init__(self, dist, rank, world, group=None):
        self.dist, self.rank, self.world, self.group = dist, rank, world, group

    def all_gather_rows(self, out, local):
        """out [W*n][...] <- concatenation of every rank's local [n][...]."""
        if self.world == 1:
            out.copy_(local)
            return out
        self.dist.all_gather_into_tensor(out, local.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, out, full):
        """out [n][...] <- this rank's row block of the element-wise sum over ranks of full [W*n][...]."""
        if self.world == 1:
            out.copy_(full)
            return out
        if self.dist.get_backend(self.group) == "gloo":  # gloo has no reduce_scatter: reduce everywhere, keep own rows
            tmp = full.clone()
            self.dist.all_reduce(tmp, group=self.group)
            n = out.shape[0]
            out.copy_(tmp[self.rank * n:(self.rank + 1) * n])
            return out
        self.dist.reduce_scatter_tensor(out, full.contiguous(), group=self.group)
        return out


def shard_bounds(total, world, rank):
    """Even split; ``total`` must divide by ``world`` (tokens, experts and the dense K are chosen that way)."""
    if total % world:
        raise ValueError(f"{total} does not divide over {world} ranks")
    n = total // world
    return rank * n, (rank + 1) * n


def ep_layer_forward(xch, compute, x_local, bufs):
    """One layer on one rank.  ``compute`` provides
         dense_partial(x_all) -> partial [T][H]   (this rank's K-slice of the projection, all tokens)
         route(h_local) -> (ids [T/W][k], w [T/W][k])
         experts_partial(h_all, ids_all, w_all) -> y partial [T][H] over this rank's experts only
    ``bufs`` holds preallocated tensors: x_all, partial, h_local, h_all, ids_all, w_all, y_local."""
    x_all = xch.all_gather_rows(bufs["x_all"], x_local)
    partial = compute.dense_partial(x_all)
    h_local = xch.reduce_scatter_rows(bufs["h_local"], partial)
    ids, w = compute.route(h_local)
    h_all = xch.all_gather_rows(bufs["h_all"], h_local)
    ids_all = xch.all_gather_rows(bufs["ids_all"], ids)
    w_all = xch.all_gather_rows(bufs["w_all"], w)
    y_part = compute.experts_partial(h_all, ids_all, w_all)
    return xch.reduce_scatter_rows(bufs["y_local"], y_part)
