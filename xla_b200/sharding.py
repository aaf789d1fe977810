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

from .scaled_dot import Epilogue


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


class OverlappedRowParallelScaledDot:
    """K-split scaled dot whose all-reduce starts while the dot is still running.

    The dense kernel counts finished row blocks of its bf16 partial (b200sd_scaled_dot_f8_progress);
    a second stream waits on each counter with a stream memory operation and all-reduces that row
    block, so all but the last block's reduction hides under the remaining tiles.  The kernel is
    held to `gemm_ctas` SMs so the collective's kernels find room beside it.  The result is the
    same sum of bf16 partials as the plain pattern: every element is reduced exactly once, by the
    same collective.

    XLA's counterpart is the async all-reduce start/done pair scheduled around the dot's thunk
    (xla/backends/gpu/runtime/all_reduce_thunk.cc:89-150); it cannot begin before the dot ends.
    """

    def __init__(self, a_shard, b_shard, a_scale, b_scale, out, *, rows_per_block: int = 2048, gemm_ctas: int = 132,
                 group=None, lhs_contracting_dim: int = 1, rhs_contracting_dim: int = 0):
        import ctypes as C

        import torch

        from . import _native
        from .scaled_dot import _dtype_code

        self._torch, self._native, self._C = torch, _native, C
        self.group = group
        m = a_shard.shape[0] if lhs_contracting_dim == 1 else a_shard.shape[1]
        k = a_shard.shape[1] if lhs_contracting_dim == 1 else a_shard.shape[0]
        n = b_shard.shape[1] if rhs_contracting_dim == 0 else b_shard.shape[0]
        if out.shape != (m, n) or out.dtype != torch.bfloat16 or not out.is_contiguous():
            raise ValueError("out must be a contiguous bf16 [m, n] tensor")
        self.keep = (a_shard, b_shard, a_scale, b_scale, out)
        self.out = out
        self.rows = rows_per_block
        self.args = _native.ScaledDotF8Args(
            struct_size=C.sizeof(_native.ScaledDotF8Args), a=a_shard.data_ptr(), b=b_shard.data_ptr(),
            a_scale=a_scale.data_ptr(), b_scale=b_scale.data_ptr(), d=out.data_ptr(), m=m, n=n, k=k,
            a_dtype=_dtype_code(a_shard.dtype), b_dtype=_dtype_code(b_shard.dtype),
            d_dtype=_dtype_code(out.dtype), lhs_contracting_dim=lhs_contracting_dim,
            rhs_contracting_dim=rhs_contracting_dim, epilogue=int(Epilogue.DEFAULT), alpha=1.0, beta=0.0, kernel=0)
        blocks = (m + rows_per_block - 1) // rows_per_block
        self.counters = torch.zeros(blocks, dtype=torch.int32, device=out.device)
        self.totals = [0] * blocks
        self.progress = _native.ProgressArgs(struct_size=C.sizeof(_native.ProgressArgs), counters=self.counters.data_ptr(),
                                             rows_per_block=rows_per_block, max_ctas=gemm_ctas)
        self.side = torch.cuda.Stream(device=out.device)
        self.reduced = None          # event: the previous call's all-reduces are done with `out`
        self._err = C.create_string_buffer(512)

    def _check(self, rc):
        if rc != 0:
            from .scaled_dot import XlaFfiError

            raise XlaFfiError(rc, self._err.value.decode(errors="replace"))

    def __call__(self):
        """Enqueues the dot on the current stream and the row-block all-reduces on the side stream;
        the current stream then waits for the last of them.  Returns `out`."""
        import torch.distributed as dist

        torch, lib = self._torch, self._native.product
        main = torch.cuda.current_stream(self.out.device)
        start = torch.cuda.Event()
        start.record(main)                       # the side stream may not run ahead of earlier users of `out`
        self._check(lib.b200sd_scaled_dot_f8_progress(self.args, self.progress, main.cuda_stream, self._err, len(self._err)))
        p = self.progress
        self.side.wait_event(start)
        with torch.cuda.stream(self.side):
            for i in range(p.num_blocks):
                inc = p.last_increment if i == p.num_blocks - 1 else p.increment
                self.totals[i] = (self.totals[i] + inc) & 0xFFFFFFFF
                addr = self.counters.data_ptr() + 4 * i
                self._check(lib.b200sd_stream_wait_counter(self.side.cuda_stream, addr, self.totals[i], self._err, len(self._err)))
                dist.all_reduce(self.out[i * self.rows:(i + 1) * self.rows], op=dist.ReduceOp.SUM, group=self.group)
            done = torch.cuda.Event()
            done.record(self.side)
        main.wait_event(done)
        return self.out


class PeerReducedRowParallelScaledDot:
    """K-split scaled dot whose sum is formed inside the dot's kernel over peer memory
    (b200sd_scaled_dot_f8_peer_reduce): no collective launch at all.  Replaces the dot -> all-reduce
    pair of xla/service/spmd/dot_handler.cc:2815-2951.

    The output, staging and flag buffers live in symmetric memory (torch.distributed's
    `_symmetric_memory`, used purely as the allocator / address exchange) so that every rank holds
    a mapping of every other rank's buffers.  All ranks must call the object the same number of
    times: the call count is the protocol's epoch.

    `pull` selects the forms in which no partial is pushed: every rank keeps its partials in its own staging
    buffer and the owner of a row block fetches their sum (`multimem.ld_reduce` through the NVSwitch when a
    multicast mapping exists, so each partial crosses NVLink once and is added in the switch).  pull=1: the warp
    that computed an own tile fetches that tile's sum right away; pull=2: the sums of a round's own rows are
    fetched in small pieces by all warps during the next round, which spreads the traffic over the kernel.

    A rank that is late by more than `peer_wait_ms` makes its peers' waits give up: the kernels
    drain, the device status word gets bit 32 and the result is incomplete.  `check()` reads the
    status word; when it reports a failure on any rank, `rearm()` (a collective: every rank must
    call it) puts the protocol back to its initial state.
    """

    def __init__(self, m: int, n: int, group=None, device=None, multicast: bool = True, peer_wait_ms: int = 0,
                 pull: int = 0):
        import ctypes as C

        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from . import _native

        self._torch, self._native, self._C = torch, _native, C
        group = group or dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.m, self.n = m, n
        words = _native.product.b200sd_peer_reduce_flag_words(m, n, self.world)
        if words == 0:
            raise ValueError(f"m = {m} must be a multiple of 256 x world ({self.world}) for the peer-reduced dot")
        device = device or torch.device("cuda", torch.cuda.current_device())
        self.out = symm.empty((m, n), dtype=torch.bfloat16, device=device)
        self.stage = symm.empty((m, n), dtype=torch.bfloat16, device=device)
        self.flags = symm.empty((words,), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._handles = [symm.rendezvous(t, group) for t in (self.out, self.stage, self.flags)]
        self._handles[2].barrier()                 # every rank's flags are zero before anyone counts on them
        self.peers = _native.PeerReduceArgs(struct_size=C.sizeof(_native.PeerReduceArgs), world=self.world, rank=self.rank,
                                            emulate_ranks=0, epoch=0, peer_wait_ms=int(peer_wait_ms))
        self.group = group
        for r in range(self.world):
            self.peers.d[r] = self._handles[0].buffer_ptrs[r]
            self.peers.stage[r] = self._handles[1].buffer_ptrs[r]
            self.peers.flags[r] = self._handles[2].buffer_ptrs[r]
        # With NVSwitch multicast the finished rows leave this GPU once instead of world-1 times.
        mc = getattr(self._handles[0], "multicast_ptr", 0) if (multicast and self.world > 1) else 0
        self.peers.d_multicast = mc or None
        self.multicast = bool(mc)
        # Pull mode: partials stay with their producer and the owner of the rows fetches them -- through the
        # switch's in-network sum when the staging buffers have a multicast mapping, by peer loads otherwise.
        self.peers.pull = int(pull)
        smc = getattr(self._handles[1], "multicast_ptr", 0) if (pull and multicast and self.world > 1) else 0
        self.peers.stage_multicast = smc or None
        self.pull, self.in_switch_sum = int(pull), bool(smc)
        self._err = C.create_string_buffer(512)

    def __call__(self, a_shard, b_shard, a_scale, b_scale, *, lhs_contracting_dim: int = 1, rhs_contracting_dim: int = 0):
        """Enqueues this rank's part on the current stream; returns the [m,n] bf16 sum (complete on
        this rank when the stream reaches the end of the kernel)."""
        from .scaled_dot import XlaFfiError, _dtype_code

        torch, C, native = self._torch, self._C, self._native
        k = a_shard.shape[1] if lhs_contracting_dim == 1 else a_shard.shape[0]
        args = native.ScaledDotF8Args(
            struct_size=C.sizeof(native.ScaledDotF8Args), a=a_shard.data_ptr(), b=b_shard.data_ptr(),
            a_scale=a_scale.data_ptr(), b_scale=b_scale.data_ptr(), d=self.out.data_ptr(), m=self.m, n=self.n, k=k,
            a_dtype=_dtype_code(a_shard.dtype), b_dtype=_dtype_code(b_shard.dtype), d_dtype=_dtype_code(self.out.dtype),
            lhs_contracting_dim=lhs_contracting_dim, rhs_contracting_dim=rhs_contracting_dim, epilogue=int(Epilogue.DEFAULT), alpha=1.0,
            beta=0.0, kernel=0)
        self.peers.epoch += 1
        stream = torch.cuda.current_stream(self.out.device).cuda_stream
        rc = native.product.b200sd_scaled_dot_f8_peer_reduce(args, self.peers, stream, self._err, len(self._err))
        if rc != 0:
            self.peers.epoch -= 1
            raise XlaFfiError(rc, self._err.value.decode(errors="replace"))
        return self.out

    def check(self) -> int:
        """Synchronises this rank's device and returns (and clears) its status word: 0 when every wait
        of the calls so far was satisfied, bit 32 set when a wait for a peer gave up."""
        from .scaled_dot import device_status

        return device_status()

    def rearm(self) -> None:
        """Collective.  Back to the state of a fresh object after a failed call: each rank waits for its
        own kernels, zeroes its flag counters, the ranks meet, and the epoch restarts."""
        torch = self._torch
        torch.cuda.synchronize(self.out.device)
        self._handles[2].barrier()          # nobody still adds to a peer's counters
        self.flags.zero_()
        torch.cuda.synchronize(self.out.device)
        self._handles[2].barrier()          # every rank's counters are zero before anyone counts on them
        self.peers.epoch = 0
