"""The peer-reduced K-split dot with every rank played by one launch on one GPU
(emulate_ranks == world): tile order, staging pushes, per-warp flags, the in-kernel sum in rank
order, the broadcast of finished rows and the end-of-call handshake.  The two-process run over real
peer memory is bench.py --workload c4 on two or more GPUs."""
import ctypes as C

import pytest
import torch

from xla_b200 import _native, device_status
from xla_b200.scaled_dot import cublas_lt_matmul_f8

pytestmark = pytest.mark.gpu


def _f8(shape, gen, dev):
    return torch.randn(shape, device=dev, generator=gen).to(torch.float8_e4m3fn)


@pytest.mark.parametrize("pull", [0, 1, 2])
@pytest.mark.parametrize("world,m,n,k_per_rank", [(2, 1024, 768, 384), (4, 2048, 512, 256), (2, 512, 272, 128), (1, 512, 256, 256),
                                                  (2, 4096, 2048, 128),       # several tiles per cluster and round
                                                  (4, 4096, 8192, 128)])      # wide enough for rounds cut along the columns too
def test_emulated_ranks_match_sum_of_bf16_partials(cuda_device, world, m, n, k_per_rank, pull):
    """pull = 1 / 2: the partials stay in the producing rank's staging buffer and the owner of the rows fetches them,
    tile by tile (1) or in pieces spread over the next round (2) -- here, on one GPU, with plain loads in rank order;
    the in-switch sum needs real peers."""
    dev = cuda_device
    gen = torch.Generator(device=dev).manual_seed(100 * world + m)
    lib = _native.product
    words = lib.b200sd_peer_reduce_flag_words(m, n, world)
    assert words > 0
    sa, sb = torch.tensor(0.5, device=dev), torch.tensor(0.125, device=dev)
    d = [torch.zeros((m, n), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    stage = [torch.zeros((m, n), dtype=torch.bfloat16, device=dev) for _ in range(world)]
    flags = [torch.zeros(words, dtype=torch.int32, device=dev) for _ in range(world)]
    err = C.create_string_buffer(512)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for epoch in (1, 2, 3):                                   # the flags are never reset between calls
        a = [_f8((m, k_per_rank), gen, dev) for _ in range(world)]
        b = [_f8((k_per_rank, n), gen, dev) for _ in range(world)]
        partials = [cublas_lt_matmul_f8(a[r], b[r], sa, sb)[0] for r in range(world)]
        acc = torch.zeros((m, n), dtype=torch.float32, device=dev)
        for p in partials:                                    # rank order, f32, one rounding at the end
            acc = acc + p.float()
        expect = acc.bfloat16()
        for t in d:
            t.zero_()
        args = _native.ScaledDotF8Args(struct_size=C.sizeof(_native.ScaledDotF8Args), a=a[0].data_ptr(), b=b[0].data_ptr(),
                                       a_scale=sa.data_ptr(), b_scale=sb.data_ptr(), d=d[0].data_ptr(), m=m, n=n, k=k_per_rank,
                                       a_dtype=20, b_dtype=20, d_dtype=16, lhs_contracting_dim=1, rhs_contracting_dim=0,
                                       epilogue=0, alpha=1.0, beta=0.0, kernel=0)
        peers = _native.PeerReduceArgs(struct_size=C.sizeof(_native.PeerReduceArgs), world=world, rank=0, emulate_ranks=world,
                                       epoch=epoch, pull=pull)
        for r in range(world):
            peers.d[r], peers.stage[r], peers.flags[r] = d[r].data_ptr(), stage[r].data_ptr(), flags[r].data_ptr()
            peers.emu_a[r], peers.emu_b[r] = a[r].data_ptr(), b[r].data_ptr()
        rc = lib.b200sd_scaled_dot_f8_peer_reduce(args, peers, stream, err, len(err))
        assert rc == 0, err.value
        torch.cuda.synchronize()
        assert device_status() == 0
        for r in range(world):
            assert torch.equal(d[r], expect), f"rank {r} epoch {epoch}: {(d[r].float() - expect.float()).abs().max().item()}"


def test_peer_reduce_rejects_what_it_cannot_do(cuda_device):
    dev = cuda_device
    lib = _native.product
    assert lib.b200sd_peer_reduce_flag_words(768, 512, 2) == 0           # 768 is not a multiple of 256 x 2
    a = torch.zeros((512, 256), device=dev).to(torch.float8_e4m3fn)
    s = torch.ones((), device=dev)
    d = torch.zeros((512, 256), dtype=torch.bfloat16, device=dev)
    f = torch.zeros(4096, dtype=torch.int32, device=dev)
    err = C.create_string_buffer(512)

    def call(m=512, epoch=1, world=2, d_dtype=16, stage_ptr=d.data_ptr()):
        args = _native.ScaledDotF8Args(struct_size=C.sizeof(_native.ScaledDotF8Args), a=a.data_ptr(), b=a.data_ptr(),
                                       a_scale=s.data_ptr(), b_scale=s.data_ptr(), d=d.data_ptr(), m=m, n=256, k=256,
                                       a_dtype=20, b_dtype=20, d_dtype=d_dtype, lhs_contracting_dim=1, rhs_contracting_dim=1,
                                       epilogue=0, alpha=1.0, beta=0.0, kernel=0)
        peers = _native.PeerReduceArgs(struct_size=C.sizeof(_native.PeerReduceArgs), world=world, rank=0, emulate_ranks=world, epoch=epoch)
        for r in range(min(world, 8)):
            peers.d[r], peers.stage[r], peers.flags[r] = d.data_ptr(), stage_ptr, f.data_ptr()
            peers.emu_a[r], peers.emu_b[r] = a.data_ptr(), a.data_ptr()
        return lib.b200sd_scaled_dot_f8_peer_reduce(args, peers, None, err, len(err))

    assert call(m=256) == 3 and b"256 x world" in err.value
    assert call(epoch=0) == 3
    assert call(world=9) == 3
    assert call(d_dtype=11) == 3 and b"bf16" in err.value
    assert call(stage_ptr=None) == 3
    torch.cuda.synchronize()
    assert int(f.abs().sum().item()) == 0 and device_status() == 0
