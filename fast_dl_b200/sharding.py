"""Row sharding of the path over the GPUs of one box (one process per GPU).

Every op of the path is independent per element or per row, so a tensor is cut into
contiguous blocks of its leading dimension and each rank runs the single-GPU entry points
on its block.  Only two results need an exchange: the full sum (one double per rank) and a
reduction along axis 0 (one [cols] vector per rank).  The collective is issued on the
stream the kernel ran on, on the tensor the kernel wrote: no host round trip.

`local` is the object that computes on one shard; by default the CUDA kernels through the
C ABI.  Tests on machines without a GPU pass a CPU stand-in to exercise the shard arithmetic
and the exchange protocol over gloo.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class RowShard:
    """Rows [start, start + count) of `total` rows, owned by `rank` of `world`."""
    rank: int
    world: int
    total: int
    start: int
    count: int


def shard_rows(total: int, world: int, rank: int) -> RowShard:
    """Contiguous split; the first `total % world` ranks own one extra row."""
    if world < 1 or not 0 <= rank < world or total < 0:
        raise ValueError(f"bad shard request: total={total} world={world} rank={rank}")
    base, extra = divmod(total, world)
    count = base + (1 if rank < extra else 0)
    start = rank * base + min(rank, extra)
    return RowShard(rank, world, total, start, count)


class CudaLocal:
    """Shard-local compute on the current CUDA device through the C ABI."""

    def full_sum_f64(self, x):
        from . import capi
        _, s64 = capi.full_sum(x.reshape(-1), want_f64=True)
        return s64

    def col_sums(self, x2d, global_rows):
        from . import capi
        return capi.reduce_cols(x2d, capi.REDUCE_MEAN, mean_divisor=global_rows)


class CudaFusedLocal:
    """Shard-local compute with the exchange INSIDE the kernels (peer stores over NVLink):
    results are already global, RowSharded must not reduce them again."""

    fused = True

    def __init__(self, exchange):
        self.exchange = exchange

    def full_sum_f64(self, x):
        import torch
        out64 = torch.empty(1, dtype=torch.float64, device=x.device)
        self.exchange.sum(x.reshape(-1), None, out64)
        return out64

    def col_sums(self, x2d, global_rows):
        import torch
        from . import capi
        out = torch.empty(x2d.shape[1], dtype=torch.float32, device=x2d.device)
        return self.exchange.reduce_cols(x2d, capi.REDUCE_MEAN, global_rows, out)


class RowSharded:
    """The two ops of the path that need an exchange, over a torch.distributed group."""

    def __init__(self, shard: RowShard, local=None, group=None):
        self.shard, self.local, self.group = shard, local or CudaLocal(), group

    def _all_reduce(self, t):
        import torch.distributed as dist
        if self.shard.world > 1 and not getattr(self.local, "fused", False):
            dist.all_reduce(t, op=dist.ReduceOp.SUM, group=self.group)
        return t

    def full_sum(self, x_shard):
        """Sum over the WHOLE tensor; every rank gets the same float64 [1] tensor."""
        return self._all_reduce(self.local.full_sum_f64(x_shard))

    def mean_axis0(self, x_shard_2d):
        """Mean over all rows of the whole [total, cols] tensor; every rank gets [cols]."""
        if x_shard_2d.shape[0] != self.shard.count:
            raise ValueError("shard has the wrong number of rows")
        # Each rank divides its column sums by the GLOBAL row count, so the sum of the
        # per-rank vectors is the global mean.
        return self._all_reduce(self.local.col_sums(x_shard_2d, self.shard.total))
