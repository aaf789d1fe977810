"""Host logic of the two sharded launch patterns, run as world-size-2 `gloo` ranks on CPU.

The GPU call of each rank is replaced by the CPU oracle on that rank's shard, so what is tested is
the shard index arithmetic, the absence of a collective in the column-parallel pattern, the single
all-reduce of the row-parallel pattern and the amax combination -- the parts of
xla/service/spmd/dot_handler.cc:2516, 2815-2951 this repository restates.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scaled_dot_oracle as o
from xla_b200 import sharding


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_shard_bounds_cover_the_dimension():
    for extent, world in [(8192, 8), (28672, 8), (28672, 4), (48, 2), (16, 4), (112, 3)]:
        pieces = [sharding.shard_bounds(extent, world, r) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == extent
        for (b0, e0), (b1, e1) in zip(pieces, pieces[1:]):
            assert e0 == b1
        assert all(b % 16 == 0 and e % 16 == 0 for b, e in pieces)
        sizes = [e - b for b, e in pieces]
        assert max(sizes) - min(sizes) <= 16
    with pytest.raises(ValueError):
        sharding.shard_bounds(100, 2, 0)


def _worker(rank, world, port, tmpdir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, k, n = 64, 96, 80
        a, b, sa, sb = o.make_f8_operands(90, m, k, n)
        bias = o.bf16_bits_to_f32(o.make_bias_bf16(90, n))

        # ---- column-parallel: N split, A replicated, no collective, host-side amax combine.
        calls = {"all_reduce": 0}
        orig = dist.all_reduce

        def counting_all_reduce(*args, **kw):
            calls["all_reduce"] += 1
            return orig(*args, **kw)

        dist.all_reduce = counting_all_reduce

        def local_col(a_, b_shard, bias_shard):
            d, amax = o.scaled_dot_f8(a_, b_shard, sa, sb, bias=bias_shard, epilogue=o.EPI_BIAS_GELU,
                                      out_dtype=o.F32, want_amax=True)
            return d, amax

        col = sharding.ColumnParallelScaledDot(n, world, rank, local_col)
        d_shard, amax_local = col(a, col.shard_b(b), col.shard_bias(bias))
        assert calls["all_reduce"] == 0                      # no data-path collective
        amax = sharding.combine_amax(float(amax_local))
        np.save(os.path.join(tmpdir, f"col_{rank}.npy"), d_shard)

        # ---- row-parallel: K split, one all-reduce (sum) of the bf16 partials.
        def local_row(a_shard, b_shard):
            d, _ = o.scaled_dot_f8(a_shard, b_shard, sa, sb, out_dtype=o.BF16)
            return torch.from_numpy(o.bf16_bits_to_f32(d)).to(torch.bfloat16)

        row = sharding.RowParallelScaledDot(k, world, rank, local_row)
        total = row(row.shard_a(a), row.shard_b(b))
        assert calls["all_reduce"] == 1                      # exactly one collective
        dist.all_reduce = orig
        if rank == 0:
            np.save(os.path.join(tmpdir, "row.npy"), total.float().numpy())
            np.save(os.path.join(tmpdir, "amax.npy"), np.array([amax], np.float32))
    finally:
        dist.destroy_process_group()


def test_column_and_row_parallel_with_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    m, k, n = 64, 96, 80
    a, b, sa, sb = o.make_f8_operands(90, m, k, n)
    bias = o.bf16_bits_to_f32(o.make_bias_bf16(90, n))
    exp, exp_amax = o.scaled_dot_f8(a, b, sa, sb, bias=bias, epilogue=o.EPI_BIAS_GELU, out_dtype=o.F32, want_amax=True)
    got = sharding.gather_columns([np.load(tmp_path / f"col_{r}.npy") for r in range(world)])
    np.testing.assert_allclose(got, exp, rtol=1e-5, atol=1e-6)
    assert np.load(tmp_path / "amax.npy")[0] == pytest.approx(float(exp_amax), rel=1e-6)
    # Row-parallel sums bf16-rounded partials (as BASELINE config 4 specifies): each partial and the
    # sum carry one bf16 rounding (2^-9 relative), so the error is bounded by the partials' magnitudes.
    parts = []
    for r in range(world):
        ks = sharding.row_parallel_slices(k, world, r)
        parts.append(o.scaled_dot_f8(a[:, ks], b[ks, :], sa, sb, out_dtype=o.F32)[0])
    exp_row = parts[0] + parts[1]
    bound = 2.0 ** -8 * (np.abs(parts[0]) + np.abs(parts[1]) + np.abs(exp_row)) + 1e-6
    assert (np.abs(np.load(tmp_path / "row.npy") - exp_row) <= bound).all()


def test_amax_combination_propagates_nan_single_process():
    assert sharding.combine_amax(3.5) == 3.5          # no process group: identity
