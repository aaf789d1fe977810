"""Batched scaled dots: one leading batch dimension on a, b, c and D, lhs/rhs_batch_dims = {0} --
the form of gemm_rewriter_fp8_test.cc:941-991 (BatchedScaledABUnscaledDF8)."""
import numpy as np
import pytest
import torch

from oracle import scaled_dot_oracle as o
from xla_b200 import device_status
from xla_b200.scaled_dot import Epilogue, GemmBackendConfig, XlaFfiError, cublas_lt_matmul_f8

pytestmark = pytest.mark.gpu


def _dev(x, dev, dt):
    return torch.from_numpy(np.ascontiguousarray(x)).to(dev).view(dt)


@pytest.mark.parametrize("batch,m,k,n,rc", [(10, 16, 32, 16, 1), (3, 272, 256, 528, 1), (4, 128, 192, 256, 2), (2, 400, 128, 144, 1)])
def test_batched_scaled_dot_f32_out(cuda_device, batch, m, k, n, rc):
    """rc is the rhs contracting dimension in the rank-3 index space: 1 -> b is [batch, k, n], 2 -> [batch, n, k]."""
    rng = np.random.default_rng(batch * 1000 + m)
    a = o.fp8_encode(rng.standard_normal((batch, m, k), dtype=np.float32) * 4, "e4m3fn")
    bshape = (batch, k, n) if rc == 1 else (batch, n, k)
    b = o.fp8_encode(rng.standard_normal(bshape, dtype=np.float32) * 4, "e4m3fn")
    sa, sb = np.float32(0.5), np.float32(0.25)
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(rc,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,))
    d, _ = cublas_lt_matmul_f8(_dev(a, cuda_device, torch.float8_e4m3fn), _dev(b, cuda_device, torch.float8_e4m3fn),
                               torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device),
                               out_dtype=torch.float32, config=cfg)
    torch.cuda.synchronize()
    assert tuple(d.shape) == (batch, m, n)
    got = d.cpu().numpy()
    for i in range(batch):
        exp = o.scaled_dot_f8(a[i], b[i], sa, sb, rhs_contracting=rc - 1, out_dtype=o.F32)[0]
        assert o.near_mismatches(exp, got[i], 1e-3, 1e-4)[0] == 0, f"batch {i}"
    assert device_status() == 0


def test_batched_with_bias_gelu_fp8_out_and_amax(cuda_device):
    batch, m, k, n = 3, 256, 384, 512
    rng = np.random.default_rng(77)
    a = o.fp8_encode(rng.standard_normal((batch, m, k), dtype=np.float32) * 2, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((batch, k, n), dtype=np.float32) * 2, "e4m3fn")
    bias = o.make_bias_bf16(5, n)
    sa, sb = np.float32(0.05), np.float32(0.04)
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,), epilogue=Epilogue.BIAS_GELU, damax_output=True)
    d, amax = cublas_lt_matmul_f8(_dev(a, cuda_device, torch.float8_e4m3fn), _dev(b, cuda_device, torch.float8_e4m3fn),
                                  torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device),
                                  bias=_dev(bias, cuda_device, torch.int16).view(torch.bfloat16),
                                  d_scale=torch.tensor(2.0, device=cuda_device), out_dtype=torch.float8_e4m3fn, config=cfg)
    torch.cuda.synchronize()
    got = d.view(torch.uint8).cpu().numpy()
    top = 0.0
    for i in range(batch):
        exp, am = o.scaled_dot_f8(a[i], b[i], sa, sb, bias=o.bf16_bits_to_f32(bias), epilogue=o.EPI_BIAS_GELU, d_scale=2.0,
                                  out_dtype=o.F8E4M3FN, want_amax=True)
        assert o.fp8_within_n_values(exp, got[i], 1) == 0, f"batch {i}"
        top = max(top, float(am))
    assert float(amax.item()) == pytest.approx(top, rel=1e-4)      # one amax over all batches
    assert device_status() == 0


def test_batched_matrix_bias(cuda_device):
    batch, m, k, n = 2, 128, 128, 256
    rng = np.random.default_rng(78)
    a = o.fp8_encode(rng.standard_normal((batch, m, k), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((batch, k, n), dtype=np.float32), "e4m3fn")
    c = rng.standard_normal((batch, m, n), dtype=np.float32)
    one = torch.ones((), device=cuda_device)
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,), beta=1.0)
    d, _ = cublas_lt_matmul_f8(_dev(a, cuda_device, torch.float8_e4m3fn), _dev(b, cuda_device, torch.float8_e4m3fn), one, one,
                               c=torch.from_numpy(c).to(cuda_device), out_dtype=torch.float32, config=cfg)
    torch.cuda.synchronize()
    for i in range(batch):
        exp = o.scaled_dot_f8(a[i], b[i], 1.0, 1.0, c=c[i], beta=1.0, out_dtype=o.F32)[0]
        assert o.near_mismatches(exp, d[i].cpu().numpy(), 1e-3, 1e-4)[0] == 0


def test_batched_frames_that_must_be_rejected(cuda_device):
    a = torch.zeros((2, 64, 64), device=cuda_device).to(torch.float8_e4m3fn)
    b3 = torch.zeros((3, 64, 64), device=cuda_device).to(torch.float8_e4m3fn)
    one = torch.ones((), device=cuda_device)
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,))
    with pytest.raises(XlaFfiError) as e:
        cublas_lt_matmul_f8(a, b3, one, one, config=cfg)
    assert e.value.code == 3 and "batch" in e.value.message
    with pytest.raises(XlaFfiError) as e:                         # rank-3 operands without batch attributes
        cublas_lt_matmul_f8(a, a, one, one, config=GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,)),
                            out=torch.zeros((2, 64, 64), dtype=torch.bfloat16, device=cuda_device))
    assert e.value.code == 12
    cfg.selected_algorithm = 2
    with pytest.raises(XlaFfiError):                              # the split-K kernel does not take batches
        cublas_lt_matmul_f8(a, a, one, one, config=cfg)


@pytest.mark.parametrize("kernel", [3, 4, 5])
def test_batched_kernel_variants_agree(cuda_device, kernel):
    batch, m, k, n = 5, 512, 1024, 768                  # 5 x 2 x 3 = 30 pair tiles
    rng = np.random.default_rng(21)
    a = _dev(o.fp8_encode(rng.standard_normal((batch, m, k), dtype=np.float32) * 3, "e4m3fn"), cuda_device, torch.float8_e4m3fn)
    b = _dev(o.fp8_encode(rng.standard_normal((batch, k, n), dtype=np.float32) * 3, "e4m3fn"), cuda_device, torch.float8_e4m3fn)
    one = torch.ones((), device=cuda_device)

    def run(alg):
        cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                                rhs_batch_dimensions=(0,), selected_algorithm=alg)
        return cublas_lt_matmul_f8(a, b, one, one, out_dtype=torch.bfloat16, config=cfg)[0]

    ref = run(1)
    got = run(kernel)
    torch.cuda.synchronize()
    if kernel == 3:       # M=128 instead of M=256 MMAs: the same sums up to the f32 order inside the tensor core
        assert o.near_mismatches(ref.float().cpu().numpy(), got.float().cpu().numpy(), 1e-2, 1e-2)[0] == 0
    else:                 # the CTA-pair kernel, with or without a stream-K tail (30 tiles: there is none)
        assert torch.equal(ref, got)
    assert device_status() == 0


def test_batched_int8_through_the_plain_c_entry_point(cuda_device):
    import ctypes as C

    from xla_b200 import _native

    batch, m, k, n = 3, 144, 256, 272
    rng = np.random.default_rng(22)
    a8 = rng.integers(-127, 128, (batch, m, k), dtype=np.int8)
    b8 = rng.integers(-127, 128, (batch, k, n), dtype=np.int8)
    a, b = torch.from_numpy(a8).to(cuda_device), torch.from_numpy(b8).to(cuda_device)
    d = torch.zeros((batch, m, n), dtype=torch.int32, device=cuda_device)
    args = _native.DotS8Args(struct_size=C.sizeof(_native.DotS8Args), a=a.data_ptr(), b=b.data_ptr(), d=d.data_ptr(), m=m, n=n, k=k,
                             d_dtype=4, lhs_contracting_dim=1, rhs_contracting_dim=0, kernel=0, batch_count=batch)
    err = C.create_string_buffer(512)
    assert _native.product.b200sd_dot_s8(args, torch.cuda.current_stream(cuda_device).cuda_stream, err, len(err)) == 0, err.value
    torch.cuda.synchronize()
    got = d.cpu().numpy()
    for i in range(batch):
        assert np.array_equal(got[i], o.dot_s8(a8[i], b8[i])), f"batch {i}"
    assert device_status() == 0


@pytest.mark.parametrize("rhs_contracting_dim", [1, 2])
def test_batched_int8_through_the_ffi_call(cuda_device, rhs_contracting_dim):
    """Rank-3 s8 operands through `b200$dot$s8` (lhs_batch_dims = rhs_batch_dims = {0}), with the s32 copy and the
    dequantised bf16 result; the scale vectors are shared by the batches."""
    from xla_b200 import cublas_lt_matmul_s8

    batch, m, k, n = 4, 80, 192, 112
    rng = np.random.default_rng(31)
    a8 = rng.integers(-128, 128, (batch, m, k), dtype=np.int8)
    b8 = rng.integers(-128, 128, (batch, k, n), dtype=np.int8)
    rs = rng.uniform(0.001, 0.01, m).astype(np.float32)
    cs = rng.uniform(0.001, 0.01, n).astype(np.float32)
    b_in = b8 if rhs_contracting_dim == 1 else np.ascontiguousarray(np.swapaxes(b8, 1, 2))
    a, b = torch.from_numpy(a8).to(cuda_device), torch.from_numpy(b_in).to(cuda_device)
    d, acc = cublas_lt_matmul_s8(a, b, rhs_contracting_dim=rhs_contracting_dim)
    torch.cuda.synchronize()
    want = np.stack([o.dot_s8(a8[i], b8[i]) for i in range(batch)])
    assert acc is None and d.dtype == torch.int32 and np.array_equal(d.cpu().numpy(), want)
    d, acc = cublas_lt_matmul_s8(a, b, rhs_contracting_dim=rhs_contracting_dim, emit_s32=True,
                                 a_row_scale=torch.from_numpy(rs).to(cuda_device), b_col_scale=torch.from_numpy(cs).to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(acc.cpu().numpy(), want)
    got_bits = d.view(torch.int16).cpu().numpy().view(np.uint16)
    for i in range(batch):
        assert np.array_equal(got_bits[i], o.dequant_s32_to_bf16(want[i], rs, cs)), f"batch {i}"
    assert device_status() == 0
