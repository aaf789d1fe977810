"""Guard bands around every buffer a launch may write (the redzone idea of
xla/stream_executor/gpu/redzone_allocator_kernel_lib.cu.h): the result, amax and the workspace sit in
the middle of pattern-filled allocations, and the pattern must survive every launch -- ragged
shapes, every kernel variant, batched and int8 calls included."""
import numpy as np
import pytest
import torch

from xla_b200 import _native, device_status
from xla_b200.scaled_dot import Epilogue, GemmBackendConfig, cublas_lt_matmul_f8, cublas_lt_matmul_s8

pytestmark = pytest.mark.gpu
GUARD = 4096          # bytes on either side
PATTERN = 0xA5


class Guarded:
    """A tensor of `shape` / `dtype` carved out of the middle of a pattern-filled byte buffer."""

    def __init__(self, shape, dtype, dev):
        self.nbytes = int(np.prod(shape, dtype=np.int64)) * torch.empty((), dtype=dtype).element_size()
        self.raw = torch.full((GUARD + self.nbytes + GUARD,), PATTERN, dtype=torch.uint8, device=dev)
        self.tensor = self.raw[GUARD:GUARD + self.nbytes].view(dtype).view(shape)

    def intact(self) -> bool:
        return bool((self.raw[:GUARD] == PATTERN).all()) and bool((self.raw[GUARD + self.nbytes:] == PATTERN).all())


SHAPES = [(16, 16, 16), (48, 80, 32), (144, 272, 128), (240, 400, 112), (512, 768, 256), (128, 1040, 2064), (64, 2048, 1024)]


@pytest.mark.parametrize("m,n,k", SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32, torch.float8_e4m3fn])
def test_fp8_launches_stay_inside_their_buffers(cuda_device, m, n, k, out_dtype):
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(m * 7 + n)
    a = torch.randn((m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn((k, n), device=dev, generator=g).to(torch.float8_e4m3fn)
    bias = torch.randn(n, device=dev, generator=g).bfloat16()
    one = torch.ones((), device=dev)
    f8_out = out_dtype == torch.float8_e4m3fn
    need = _native.product.b200sd_workspace_bytes(m, n, k)    # > 0: a shape the split-K kernel takes (and is chosen for)
    kernels = [0, 3] + ([4, 5] if m > 128 else []) + ([2] if (0 < need <= (16 << 20) and not f8_out) else [])
    reference = None
    for kernel in kernels:
        plain = kernel == 2                                   # the split-K kernel computes the plain scaled dot only
        d = Guarded((m, n), out_dtype, dev)
        amax = Guarded((), torch.float32, dev)
        ws = Guarded((16 << 20,), torch.int8, dev)
        cfg = GemmBackendConfig(epilogue=Epilogue.DEFAULT if plain else Epilogue.BIAS_GELU, damax_output=f8_out,
                                selected_algorithm=kernel)
        cublas_lt_matmul_f8(a, b, one, one, bias=None if plain else bias, d_scale=one if f8_out else None, out_dtype=out_dtype,
                            config=cfg, workspace=ws.tensor, out=d.tensor, amax_out=amax.tensor if f8_out else None)
        torch.cuda.synchronize()
        assert d.intact(), f"kernel {kernel}: wrote outside D"
        assert amax.intact(), f"kernel {kernel}: wrote outside amax"
        assert ws.intact(), f"kernel {kernel}: wrote outside the workspace"
        if not plain:
            got = d.tensor.float()
            assert bool(torch.isfinite(got).all())
            if reference is None:
                reference = got
            else:                                             # the variants agree to within the output's resolution
                tol = 0.13 if f8_out else 1e-2
                assert bool(((got - reference).abs() <= tol * reference.abs() + tol).all()), f"kernel {kernel}"
    assert device_status() == 0


def test_batched_and_int8_launches_stay_inside_their_buffers(cuda_device):
    dev = cuda_device
    g = torch.Generator(device=dev).manual_seed(5)
    batch, m, k, n = 3, 272, 144, 400
    a = torch.randn((batch, m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
    b = torch.randn((batch, k, n), device=dev, generator=g).to(torch.float8_e4m3fn)
    one = torch.ones((), device=dev)
    d = Guarded((batch, m, n), torch.bfloat16, dev)
    ws = Guarded((1 << 20,), torch.int8, dev)
    cfg = GemmBackendConfig(lhs_contracting_dimensions=(2,), rhs_contracting_dimensions=(1,), lhs_batch_dimensions=(0,),
                            rhs_batch_dimensions=(0,))
    cublas_lt_matmul_f8(a, b, one, one, config=cfg, workspace=ws.tensor, out=d.tensor)
    torch.cuda.synchronize()
    assert d.intact() and ws.intact()
    expect = torch.bmm(a.float(), b.float())
    assert bool(((d.tensor.float() - expect).abs() <= 1e-2 * expect.abs() + 1e-2).all())

    a8 = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=g)
    b8 = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g)
    for kernel in (0, 3, 4, 5):
        ws = Guarded((1 << 20,), torch.int8, dev)
        d32, acc = cublas_lt_matmul_s8(a8, b8, selected_algorithm=kernel, workspace=ws.tensor)
        torch.cuda.synchronize()
        assert ws.intact()
        assert torch.equal(d32, (a8.double() @ b8.double()).to(torch.int32))
    assert device_status() == 0


@pytest.mark.parametrize("out_dtype", [torch.float8_e4m3fn, torch.float8_e5m2])
def test_decode_shape_with_fp8_result_takes_the_dense_kernel(cuda_device, out_dtype):
    """A decode-shaped call (m <= 128, n, k >= 1024, a workspace) whose result is FP8: the split-K kernel stores
    bf16 / f16 / f32 only, so automatic selection must send the call to the dense kernel, and naming the
    split-K kernel explicitly must be refused -- with D, one byte per element, inside guard bands."""
    from oracle import scaled_dot_oracle as o
    from xla_b200.scaled_dot import XlaFfiError

    dev = cuda_device
    m, n, k = 64, 1024, 1024
    assert _native.product.b200sd_select_kernel(m, n, k) == 2          # a shape the split-K kernel is chosen for
    b_kind = "e5m2" if out_dtype == torch.float8_e5m2 else "e4m3fn"     # e4m3 x e4m3 -> e5m2 is not in the type table
    a, b, sa, sb = o.make_f8_operands(77, m, k, n)
    if b_kind == "e5m2":
        b = o.fp8_encode(o.fp8_decode(b, "e4m3fn"), "e5m2")
    ta = torch.from_numpy(a).to(dev).view(torch.float8_e4m3fn)
    tb = torch.from_numpy(b).to(dev).view(out_dtype if b_kind == "e5m2" else torch.float8_e4m3fn)
    scales = [torch.tensor(np.float32(v), device=dev) for v in (sa, sb, 3.0)]
    d = Guarded((m, n), out_dtype, dev)
    ws = Guarded((16 << 20,), torch.int8, dev)
    cublas_lt_matmul_f8(ta, tb, scales[0], scales[1], d_scale=scales[2], out_dtype=out_dtype,
                        config=GemmBackendConfig(), workspace=ws.tensor, out=d.tensor)
    torch.cuda.synchronize()
    assert d.intact() and ws.intact()
    out_code = o.F8E5M2 if out_dtype == torch.float8_e5m2 else o.F8E4M3FN
    exp, _ = o.scaled_dot_f8(a, b, sa, sb, b_kind=b_kind, d_scale=3.0, out_dtype=out_code)
    got = d.tensor.view(torch.uint8).cpu().numpy()
    assert o.fp8_within_n_values(exp, got, 1) == 0            # finite values only: the cast saturates
    with pytest.raises(XlaFfiError) as e:
        cublas_lt_matmul_f8(ta, tb, scales[0], scales[1], d_scale=scales[2], out_dtype=out_dtype,
                            config=GemmBackendConfig(selected_algorithm=2), workspace=ws.tensor, out=d.tensor)
    assert e.value.code == 3
    torch.cuda.synchronize()
    assert d.intact() and device_status() == 0
