"""Stream-K tail of the dense pair kernel (kernel variant 5): when the tiles do not fill the last
wave and the call site provides its workspace, the leftover tiles are cut along K.  The s32 path must stay bit-exact;
the FP8 path must stay inside the reference's tolerances (only the f32 summation order moves)."""
import numpy as np
import pytest
import torch

from oracle import scaled_dot_oracle as o
from xla_b200 import device_status
from xla_b200.scaled_dot import Epilogue, GemmBackendConfig, cublas_lt_matmul_f8, cublas_lt_matmul_s8

pytestmark = pytest.mark.gpu
# 10 x 10 tiles of 256 x 256 on 74 clusters: one full wave, 26 tiles left over; 32 k-blocks each.
M = N = 2560
K = 4096


def test_int8_with_and_without_workspace_bit_exact(cuda_device):
    a8, b8, rs, cs = o.make_s8_operands(31, M, K, N)
    a, b = torch.from_numpy(a8).to(cuda_device), torch.from_numpy(b8).to(cuda_device)
    ws = torch.empty(32 << 20, dtype=torch.int8, device=cuda_device)
    plain = cublas_lt_matmul_s8(a, b)[0]
    for _ in range(2):                                       # twice: the flags of the first call are stale for the second
        ws.random_(-128, 127)                                # whatever the workspace holds must not matter
        tail = cublas_lt_matmul_s8(a, b, workspace=ws, selected_algorithm=5)[0]
        torch.cuda.synchronize()
        assert torch.equal(plain, tail)
    assert np.array_equal(plain.cpu().numpy(), o.dot_s8(a8, b8))
    d, acc = cublas_lt_matmul_s8(a, b, a_row_scale=torch.from_numpy(rs).to(cuda_device),
                                 b_col_scale=torch.from_numpy(cs).to(cuda_device), emit_s32=True, workspace=ws, selected_algorithm=5)
    torch.cuda.synchronize()
    assert torch.equal(acc, plain)
    assert np.array_equal(d.view(torch.int16).cpu().numpy().view(np.uint16), o.dequant_s32_to_bf16(o.dot_s8(a8, b8), rs, cs))
    assert device_status() == 0


def test_fp8_epilogue_after_the_tail(cuda_device):
    a8, b8, sa, sb = o.make_f8_operands(32, M, K, N)
    bias = o.make_bias_bf16(32, N)
    dev = cuda_device
    a = torch.from_numpy(a8).to(dev).view(torch.float8_e4m3fn)
    b = torch.from_numpy(b8).to(dev).view(torch.float8_e4m3fn)
    tsa, tsb = torch.tensor(sa, device=dev), torch.tensor(sb, device=dev)
    tb = torch.from_numpy(bias).to(dev).view(torch.int16).view(torch.bfloat16)
    d_scale = torch.tensor(0.25, device=dev)
    cfg = GemmBackendConfig(epilogue=Epilogue.BIAS_GELU, damax_output=True, selected_algorithm=5)
    ws = torch.empty(32 << 20, dtype=torch.int8, device=dev)
    d, amax = cublas_lt_matmul_f8(a, b, tsa, tsb, bias=tb, d_scale=d_scale, out_dtype=torch.float8_e4m3fn, config=cfg, workspace=ws)
    torch.cuda.synchronize()
    exp, exp_amax = o.scaled_dot_f8(a8, b8, sa, sb, bias=o.bf16_bits_to_f32(bias), epilogue=o.EPI_BIAS_GELU, d_scale=0.25,
                                    out_dtype=o.F8E4M3FN, want_amax=True)
    got = d.view(torch.uint8).cpu().numpy()
    assert o.fp8_within_n_values(exp, got, 1) == 0
    assert float((exp == got).mean()) > 0.99
    assert float(amax.item()) == pytest.approx(float(exp_amax), rel=1e-4)
    # f32 output: only the summation order differs from the oracle
    d32 = cublas_lt_matmul_f8(a, b, tsa, tsb, out_dtype=torch.float32, workspace=ws, config=GemmBackendConfig(selected_algorithm=5))[0]
    torch.cuda.synchronize()
    exp32 = o.scaled_dot_f8(a8, b8, sa, sb, out_dtype=o.F32)[0]
    assert o.near_mismatches(exp32, d32.cpu().numpy(), 1e-3, 1e-4)[0] == 0
    assert device_status() == 0
