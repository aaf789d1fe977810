"""Two-process runs over real peer memory (skipped on a single-GPU machine): the peer-reduced
K-split dot against the sum of the ranks' bf16 partials, and the NCCL pattern beside it."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, m, n, k, multicast, pull):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    try:
        from xla_b200 import device_status, sharding
        from xla_b200.scaled_dot import cublas_lt_matmul_f8

        fused = sharding.PeerReducedRowParallelScaledDot(m, n, device=dev, multicast=multicast, pull=pull)
        ks = sharding.row_parallel_slices(k, world, rank)
        for call in range(3):
            gen = torch.Generator(device=dev).manual_seed(50 + call)       # same full operands on every rank
            a = torch.randn((m, k), device=dev, generator=gen).to(torch.float8_e4m3fn)
            b = torch.randn((k, n), device=dev, generator=gen).to(torch.float8_e4m3fn)
            sa, sb = torch.tensor(0.25, device=dev), torch.tensor(0.5, device=dev)
            a_shard, b_shard = a[:, ks].contiguous(), b[ks, :].contiguous()
            out = fused(a_shard, b_shard, sa, sb)
            partial = cublas_lt_matmul_f8(a_shard, b_shard, sa, sb)[0]
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial)
            acc = torch.zeros((m, n), dtype=torch.float32, device=dev)
            for p in parts:
                acc = acc + p.float()
            torch.cuda.synchronize()
            assert device_status() == 0
            if fused.pull and fused.in_switch_sum:
                # The switch adds the bf16 partials in f32 in an order of its own and rounds once, by a rule of its own:
                # with two ranks the order cannot matter, and results still differ from round-to-nearest-even of the
                # f32 sum -- by at most one bf16 step.
                want = acc.bfloat16().float()
                diff = (out.float() - want).abs()
                bad = diff > 2.0 ** -7 * want.abs() + 1e-30
                assert not bool(bad.any()), (f"rank {rank} call {call}: {int(bad.sum())} of {bad.numel()} beyond one bf16 step, "
                                             f"largest difference {float(diff.max())} where the sum is {float(want[diff == diff.max()][0])}")
                if rank == 0 and call == 0:
                    print(f"in-switch sum: {int((diff > 0).sum())} of {diff.numel()} elements differ from the rank-order sum")
            else:
                assert torch.equal(out, acc.bfloat16()), f"rank {rank} call {call}"
            # and close to the unsplit dot: each bf16 partial and the sum carry one rounding of 2^-9
            full = cublas_lt_matmul_f8(a, b, sa, sb, out_dtype=torch.float32)[0]
            # (the switch's final rounding is not round-to-nearest-even: one whole bf16 step there instead of half a step)
            step = 2.0 ** -7 if (fused.pull and fused.in_switch_sum) else 2.0 ** -8
            bound = step * (sum(p.float().abs() for p in parts) + full.abs()) + 1e-6
            assert bool(((out.float() - full).abs() <= bound).all())
            dist.barrier()                   # the next call's operands are regenerated; keep the ranks in step
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("multicast,pull", [(False, 0), (True, 0), (False, 1), (True, 1), (False, 2), (True, 2)])
def test_peer_reduced_dot_on_two_gpus(multicast, pull):
    """push / pull by the own tile's warp / pull spread over the next round, each with and without the NVSwitch
    multicast mappings (pull + multicast = in-switch sum)."""
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), 1024, 768, 512, multicast, pull), nprocs=world, join=True)
