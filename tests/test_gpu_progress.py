"""Row-block progress counters of the dense kernel and the stream wait that consumes them
(the single-GPU half of the overlapped K-split pattern; the two-rank half runs under gloo on CPU
and in bench.py --workload c4)."""
import ctypes as C

import pytest
import torch

from xla_b200 import _native, device_status
from xla_b200.scaled_dot import cublas_lt_matmul_f8

pytestmark = pytest.mark.gpu


def _args(a, b, sa, sb, d):
    m, k = a.shape
    n = b.shape[1]
    return _native.ScaledDotF8Args(struct_size=C.sizeof(_native.ScaledDotF8Args), a=a.data_ptr(), b=b.data_ptr(),
                                   a_scale=sa.data_ptr(), b_scale=sb.data_ptr(), d=d.data_ptr(), m=m, n=n, k=k,
                                   a_dtype=20, b_dtype=20, d_dtype=16, lhs_contracting_dim=1, rhs_contracting_dim=0,
                                   epilogue=0, alpha=1.0, beta=0.0, kernel=0)


def test_progress_counters_and_stream_wait(cuda_device):
    dev = cuda_device
    m, k, n, rows = 1280, 512, 768, 512                      # 3 blocks: 512, 512 and a last one of 256 rows
    g = torch.Generator(device=dev).manual_seed(7)
    a = torch.randn((m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn((k, n), device=dev, generator=g).to(torch.float8_e4m3fn)
    sa = torch.tensor(0.5, device=dev)
    sb = torch.tensor(0.25, device=dev)
    expect = cublas_lt_matmul_f8(a, b, sa, sb)[0]
    d = torch.zeros((m, n), dtype=torch.bfloat16, device=dev)
    counters = torch.zeros(3, dtype=torch.int32, device=dev)
    prog = _native.ProgressArgs(struct_size=C.sizeof(_native.ProgressArgs), counters=counters.data_ptr(), rows_per_block=rows,
                                max_ctas=64)
    err = C.create_string_buffer(512)
    lib = _native.product
    main = torch.cuda.current_stream(dev)
    args = _args(a, b, sa, sb, d)
    assert lib.b200sd_scaled_dot_f8_progress(args, prog, main.cuda_stream, err, len(err)) == 0, err.value
    torch.cuda.synchronize()
    # pair kernel: 16 epilogue warps count per 256 x 256 tile; 3 column tiles; 2, 2 and 1 row tiles per block.
    assert (prog.num_blocks, prog.increment, prog.last_increment) == (3, 2 * 3 * 16, 1 * 3 * 16)
    assert counters.tolist() == [96, 96, 48]                 # only now is it safe to wait on these totals
    assert torch.equal(d, expect)

    # Second launch: a side stream copies each row block as soon as its counter reaches the new total.
    d.zero_()
    copy = torch.zeros_like(d)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(main)
    assert lib.b200sd_scaled_dot_f8_progress(args, prog, main.cuda_stream, err, len(err)) == 0, err.value
    with torch.cuda.stream(side):
        for i, total in enumerate([192, 192, 96]):
            assert lib.b200sd_stream_wait_counter(side.cuda_stream, counters.data_ptr() + 4 * i, total, err, len(err)) == 0, err.value
            copy[i * rows:(i + 1) * rows].copy_(d[i * rows:(i + 1) * rows], non_blocking=True)
    torch.cuda.synchronize()
    assert counters.tolist() == [192, 192, 96]
    assert torch.equal(copy, expect)
    assert device_status() == 0


def test_progress_rejects_bad_requests(cuda_device):
    dev = cuda_device
    a = torch.zeros((256, 256), device=dev).to(torch.float8_e4m3fn)
    s = torch.ones((), device=dev)
    d = torch.zeros((256, 256), dtype=torch.bfloat16, device=dev)
    counters = torch.zeros(1, dtype=torch.int32, device=dev)
    err = C.create_string_buffer(512)
    args = _args(a, a, s, s, d)
    for rows, ptr in [(100, counters.data_ptr()), (0, counters.data_ptr()), (256, None)]:
        prog = _native.ProgressArgs(struct_size=C.sizeof(_native.ProgressArgs), counters=ptr, rows_per_block=rows, max_ctas=0)
        assert _native.product.b200sd_scaled_dot_f8_progress(args, prog, None, err, len(err)) == 3
    args.kernel = 2
    prog = _native.ProgressArgs(struct_size=C.sizeof(_native.ProgressArgs), counters=counters.data_ptr(), rows_per_block=256, max_ctas=0)
    assert _native.product.b200sd_scaled_dot_f8_progress(args, prog, None, err, len(err)) == 3
    torch.cuda.synchronize()
    assert counters.item() == 0


def test_amax_with_and_without_a_workspace(cuda_device):
    """With the call site's workspace the kernel clears amax itself (two words at the workspace's end);
    without one the host puts a memset node in front.  Same amax either way, also when the result
    buffer starts out holding something larger, and on the second call with the same buffers."""
    from xla_b200.scaled_dot import Epilogue, GemmBackendConfig

    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(3)
    a = torch.randn((512, 256), device=dev, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn((256, 768), device=dev, generator=g).to(torch.float8_e4m3fn)
    one = torch.ones((), device=dev)
    d = torch.zeros((512, 768), dtype=torch.float8_e4m3fn, device=dev)
    amax = torch.full((), 1e30, dtype=torch.float32, device=dev)
    ws = torch.empty(1 << 20, dtype=torch.int8, device=dev).random_(-128, 127)
    err = C.create_string_buffer(512)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call(workspace):
        args = _native.ScaledDotF8Args(struct_size=C.sizeof(_native.ScaledDotF8Args), a=a.data_ptr(), b=b.data_ptr(),
                                       a_scale=one.data_ptr(), b_scale=one.data_ptr(), d_scale=one.data_ptr(), d=d.data_ptr(),
                                       amax=amax.data_ptr(), workspace=workspace.data_ptr() if workspace is not None else None,
                                       workspace_bytes=workspace.numel() if workspace is not None else 0, m=512, n=768, k=256,
                                       a_dtype=20, b_dtype=20, d_dtype=20, lhs_contracting_dim=1, rhs_contracting_dim=0,
                                       epilogue=0, alpha=1.0, beta=0.0, kernel=0)
        assert _native.product.b200sd_scaled_dot_f8(args, stream, err, len(err)) == 0, err.value
        torch.cuda.synchronize()
        return float(amax.item())

    expect = float((a.float() @ b.float()).abs().max().item())
    for workspace in (None, ws, ws, None):
        amax.fill_(1e30)
        assert call(workspace) == pytest.approx(expect, rel=1e-5)
    assert device_status() == 0
