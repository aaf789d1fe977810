"""The two ways this path shards over the GPUs of one box (one process per GPU).

Column-parallel: the non-contracting dimension N of B (and the bias and D with it) is split;
A is replicated; the shards are independent, so there is NO collective -- this is what XLA's SPMD
partitioner produces for a dot sharded on a non-contracting dimension
(xla/service/spmd/dot_handler.cc:2516).  The per-shard amax scalars are combined by a host-side
max, outside any timed region.

Row-parallel: the contracting dimension K of A and B is split; every rank produces a full
bf16 [M,N] partial sum and ONE all-reduce (sum) over NCCL combines them -- the
`AllReduceAlongShardingDims` of dot_handler.cc:2815-2951, executed by
xla/backends/gpu/collectives/nccl_communicator.cc:557-592.  The all-reduce is enqueued on the
same stream right behind the GEMM, with no host round trip in between.

The index arithmetic below is plain Python so that it can be exercised with `gloo` ranks on CPU;
the GPU work goes through `ScaledDotCall` (the FFI boundary).
"""

from __future__ import annotations

from typing import Callable, Optional, Sequence, Tuple


def shard_bounds(extent: int, world: int, rank: int, multiple: int = 16) -> Tuple[int, int]:
    """[begin, end) of `rank`'s slice of a dimension, in units of `multiple` (the rewriter keeps
    every dimension a multiple of 16), remainder spread over the first ranks."""
    if extent % multiple:
        raise ValueError(f"extent {extent} is not a multiple of {multiple}")
    units = extent // multiple
    base, rem = divmod(units, world)
    begin = rank * base + min(rank, rem)
    end = begin + base + (1 if rank < rem else 0)
    return begin * multiple, end * multiple


def column_parallel_slices(n: int, world: int, rank: int) -> slice:
    b, e = shard_bounds(n, world, rank)
    return slice(b, e)


def row_parallel_slices(k: int, world: int, rank: int) -> slice:
    b, e = shard_bounds(k, world, rank)
    return slice(b, e)


def combine_amax(local_amax: float, group=None) -> float:
    """Global amax = max over the shards' scalars (NaN wins, as in XLA's maximum).  A host-side
    object gather: tiny, and deliberately not a device collective."""
    import math

    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return local_amax
    vals = [None] * dist.get_world_size(group)
    dist.all_gather_object(vals, float(local_amax), group=group)
    if any(math.isnan(v) for v in vals):
        return float("nan")
    return max(vals)


class ColumnParallelScaledDot:
    """One rank's share of an N-split scaled dot.  `local_dot(a, b_shard, bias_shard) -> (d_shard,
    amax)` is the single-GPU call; no collective is issued."""

    def __init__(self, n: int, world: int, rank: int, local_dot: Callable):
        self.n, self.world, self.rank = n, world, rank
        self.cols = column_parallel_slices(n, world, rank)
        self.local_dot = local_dot

    def shard_b(self, b, rhs_contracting_dim: int = 0):
        """The rank's weight shard as its own dense row-major buffer."""
        part = b[:, self.cols] if rhs_contracting_dim == 0 else b[self.cols, :]
        return part.contiguous() if hasattr(part, "contiguous") else part.copy()

    def shard_bias(self, bias):
        return None if bias is None else bias[self.cols]

    def __call__(self, a, b_shard, bias_shard=None):
        return self.local_dot(a, b_shard, bias_shard)


class RowParallelScaledDot:
    """One rank's share of a K-split scaled dot followed by the all-reduce of the bf16 partials."""

    def __init__(self, k: int, world: int, rank: int, local_dot: Callable, all_reduce: Optional[Callable] = None):
        self.k, self.world, self.rank = k, world, rank
        self.ks = row_parallel_slices(k, world, rank)
        self.local_dot = local_dot
        self.all_reduce = all_reduce or self._dist_all_reduce

    @staticmethod
    def _dist_all_reduce(t):
        import torch.distributed as dist

        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return t

    def shard_a(self, a, lhs_contracting_dim: int = 1):
        part = a[:, self.ks] if lhs_contracting_dim == 1 else a[self.ks, :]
        return part.contiguous() if hasattr(part, "contiguous") else part.copy()

    def shard_b(self, b, rhs_contracting_dim: int = 0):
        part = b[self.ks, :] if rhs_contracting_dim == 0 else b[:, self.ks]
        return part.contiguous() if hasattr(part, "contiguous") else part.copy()

    def __call__(self, a_shard, b_shard):
        partial = self.local_dot(a_shard, b_shard)
        if self.world > 1:
            partial = self.all_reduce(partial)
        return partial


def gather_columns(shards: Sequence, axis: int = 1):
    """Test helper: reassembles the column shards in rank order."""
    import numpy as np

    return np.concatenate(list(shards), axis=axis)
