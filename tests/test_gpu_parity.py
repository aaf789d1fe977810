"""GPU parity: the CUDA path, called through the XLA FFI boundary of the C-ABI library, against
the CPU oracle on the same seeded inputs.

Tolerances are the reference's own (xla/backends/gpu/transforms/gemm_rewriter_fp8_test.cc:110):
abs 1e-2 AND rel 1e-2 for bf16/f16/f32 outputs; FP8 outputs within one representable value;
s8 x s8 -> s32 bit-exact (gemm_rewriter_test.cc:3182-3368 uses 1e-5 on integers, i.e. exact).
"""
import numpy as np
import pytest
import torch

from oracle import scaled_dot_oracle as o
import helpers as h
import xla_b200
from xla_b200.scaled_dot import XlaFfiError

pytestmark = pytest.mark.gpu


def _stored(a, b, lc, rc):
    return (a if lc == 1 else np.ascontiguousarray(a.T)), (b if rc == 0 else np.ascontiguousarray(b.T))


def test_config0_scaled_dot_bf16(cuda_device):
    """BASELINE config 0: A[256,512] . B[512,256], per-tensor scales, bf16 out, no epilogue."""
    a, b, sa, sb = o.make_f8_operands(0, 256, 512, 256)
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb)
    exp, _ = o.scaled_dot_f8(a, b, sa, sb)
    h.check_close(exp, got, o.BF16)
    # Against the strict sequential-k interpreter order as well.
    exp_strict, _ = o.scaled_dot_f8(a, b, sa, sb, strict=True)
    h.check_close(exp_strict, got, o.BF16)


@pytest.mark.parametrize("kernel", [3, 4])
@pytest.mark.parametrize("lc", [0, 1])
@pytest.mark.parametrize("rc", [0, 1])
def test_all_contracting_dim_combinations(cuda_device, lc, rc, kernel):
    """Every {lhs,rhs}_contracting_dim combination on [64,32].[32,16] padded the rewriter's way
    (gemm_rewriter_fp8_test.cc:2825-2890 sweeps these) and on a multi-tile shape, on both
    instantiations of the dense kernel (3 = one CTA per tile, 4 = CTA pairs)."""
    for (m, k, n) in [(64, 32, 16), (384, 640, 768)]:
        a, b, sa, sb = o.make_f8_operands(10 + lc * 2 + rc, m, k, n)
        sa_, sb_ = _stored(a, b, lc, rc)
        got, _ = h.run_scaled_dot(cuda_device, sa_, sb_, sa, sb, lc=lc, rc=rc, kernel=kernel)
        exp, _ = o.scaled_dot_f8(sa_, sb_, sa, sb, lhs_contracting=lc, rhs_contracting=rc)
        h.check_close(exp, got, o.BF16)


@pytest.mark.parametrize("out_dtype", [o.BF16, o.F16, o.F32])
@pytest.mark.parametrize("epilogue", [o.EPI_DEFAULT, o.EPI_BIAS, o.EPI_RELU, o.EPI_BIAS_RELU, o.EPI_GELU, o.EPI_BIAS_GELU])
def test_epilogues(cuda_device, epilogue, out_dtype):
    m, k, n = 272, 528, 304   # ragged against the 256 x 256 x 128 tile of the pair kernel
    a, b, sa, sb = o.make_f8_operands(20 + epilogue, m, k, n)
    bias = o.make_bias_bf16(20, n) if epilogue in (o.EPI_BIAS, o.EPI_BIAS_RELU, o.EPI_BIAS_GELU) else None
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, epilogue=epilogue, bias_bits=bias, out_dtype=out_dtype)
    exp, _ = o.scaled_dot_f8(a, b, sa, sb, epilogue=epilogue,
                             bias=o.bf16_bits_to_f32(bias) if bias is not None else None, out_dtype=out_dtype)
    h.check_close(exp, got, out_dtype)


def test_matrix_bias_beta(cuda_device):
    m, k, n = 256, 384, 512
    a, b, sa, sb = o.make_f8_operands(30, m, k, n)
    c = np.random.default_rng(31).standard_normal((m, n), dtype=np.float32)
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, c_f32=c, beta=1.0, alpha=0.5, out_dtype=o.F32)
    exp, _ = o.scaled_dot_f8(a, b, sa, sb, c=c, beta=1.0, alpha=0.5, out_dtype=o.F32)
    h.check_close(exp, got, o.F32)


@pytest.mark.parametrize("kinds", [("e4m3fn", "e5m2"), ("e5m2", "e4m3fn")])
def test_mixed_e5m2_operands(cuda_device, kinds):
    m, k, n = 256, 256, 256
    rng = np.random.default_rng(40)
    a, sa = o.quantize_per_tensor(rng.standard_normal((m, k), dtype=np.float32), kinds[0])
    b, sb = o.quantize_per_tensor(rng.standard_normal((k, n), dtype=np.float32), kinds[1])
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, a_kind=kinds[0], b_kind=kinds[1])
    exp, _ = o.scaled_dot_f8(a, b, sa, sb, a_kind=kinds[0], b_kind=kinds[1])
    h.check_close(exp, got, o.BF16)


def test_config1_shape_fp8_linear_gelu_amax_reduced(cuda_device):
    """BASELINE config 1's arrangement (bias + GELU + scaled e4m3 output + amax) at 1024^3."""
    m = k = n = 1024
    a, b, sa, sb = o.make_f8_operands(1, m, k, n)
    bias = o.make_bias_bf16(1, n)
    got, amax = h.run_scaled_dot(cuda_device, a, b, sa, sb, epilogue=o.EPI_BIAS_GELU, bias_bits=bias, d_scale=1.0,
                                 out_dtype=o.F8E4M3FN, want_amax=True)
    exp, exp_amax = o.scaled_dot_f8(a, b, sa, sb, epilogue=o.EPI_BIAS_GELU, bias=o.bf16_bits_to_f32(bias), d_scale=1.0,
                                    out_dtype=o.F8E4M3FN, want_amax=True)
    assert o.fp8_within_n_values(exp, got, 1) == 0          # within one e4m3 ulp
    assert float((exp == got).mean()) > 0.98
    assert abs(amax - float(exp_amax)) <= 1e-3 * float(exp_amax)


def test_saturating_fp8_output_and_d_scale(cuda_device):
    """d_scale pushes values past 448: the cast must saturate, not produce NaN
    (clamp-then-convert, gemm_rewriter.cc:1644-1657)."""
    m, k, n = 128, 256, 256
    a, b, sa, sb = o.make_f8_operands(50, m, k, n)
    for out_dtype in (o.F8E4M3FN,):
        got, amax = h.run_scaled_dot(cuda_device, a, b, sa, sb, d_scale=64.0, out_dtype=out_dtype, want_amax=True)
        exp, exp_amax = o.scaled_dot_f8(a, b, sa, sb, d_scale=64.0, out_dtype=out_dtype, want_amax=True)
        assert (got & 0x7F).max() == 0x7E                     # saturated to +-448, never NaN
        assert o.fp8_within_n_values(exp, got, 1) == 0
        assert abs(amax - float(exp_amax)) <= 1e-3 * float(exp_amax)


def test_e5m2_output_needs_an_e5m2_operand(cuda_device):
    rng = np.random.default_rng(51)
    a, sa = o.quantize_per_tensor(rng.standard_normal((128, 128), dtype=np.float32), "e4m3fn")
    b, sb = o.quantize_per_tensor(rng.standard_normal((128, 128), dtype=np.float32), "e5m2")
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, b_kind="e5m2", d_scale=1.0, out_dtype=o.F8E5M2)
    exp, _ = o.scaled_dot_f8(a, b, sa, sb, b_kind="e5m2", d_scale=1.0, out_dtype=o.F8E5M2)
    assert o.fp8_within_n_values(exp, got, 1) == 0
    with pytest.raises(XlaFfiError) as e:
        h.run_scaled_dot(cuda_device, a, a, sa, sa, d_scale=1.0, out_dtype=o.F8E5M2)
    assert e.value.code == 12


def test_nan_propagates_to_amax_and_output(cuda_device):
    """XLA's maximum and clamp propagate NaN (hlo_evaluator_typed_visitor.h:594-613, 843-865)."""
    a, b, sa, sb = o.make_f8_operands(60, 128, 128, 256)
    a = a.copy()
    a[5, 7] = 0x7F                                            # e4m3fn NaN
    got, amax = h.run_scaled_dot(cuda_device, a, b, sa, sb, d_scale=1.0, out_dtype=o.F8E4M3FN, want_amax=True)
    exp, exp_amax = o.scaled_dot_f8(a, b, sa, sb, d_scale=1.0, out_dtype=o.F8E4M3FN, want_amax=True)
    assert np.isnan(exp_amax) and np.isnan(amax)
    assert ((got[5] & 0x7F) == 0x7F).all()
    assert o.fp8_within_n_values(exp, got, 1) == 0


def test_int8_known_answer(cuda_device):
    """cuda_blas_lt_test.cc:48-156: 32x32x32 all-ones s8 -> every output == 32, s32 and f32."""
    import json, os
    ka = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "s8_known_answer.json")))
    a = torch.full((ka["m"], ka["k"]), ka["a_fill"], dtype=torch.int8, device=cuda_device)
    b = torch.full((ka["k"], ka["n"]), ka["b_fill"], dtype=torch.int8, device=cuda_device)
    d, _ = xla_b200.cublas_lt_matmul_s8(a, b)
    assert (d.cpu().numpy() == ka["expected_every_element"]).all()
    d32, _ = xla_b200.cublas_lt_matmul_s8(a, b, out_dtype=torch.float32)
    assert (d32.cpu().numpy() == float(ka["expected_every_element"])).all()


@pytest.mark.parametrize("shape", [(512, 1024, 768), (144, 272, 304)])
def test_int8_dot_bit_exact_and_dequant(cuda_device, shape):
    m, k, n = shape
    a, b, rs, cs = o.make_s8_operands(3, m, k, n)
    ta, tb = torch.from_numpy(a).to(cuda_device), torch.from_numpy(b).to(cuda_device)
    d, acc = xla_b200.cublas_lt_matmul_s8(ta, tb, a_row_scale=torch.from_numpy(rs).to(cuda_device),
                                          b_col_scale=torch.from_numpy(cs).to(cuda_device), emit_s32=True)
    torch.cuda.synchronize()
    exp_acc = o.dot_s8(a, b)
    assert np.array_equal(acc.cpu().numpy(), exp_acc)                           # s32 intermediate: bit-exact
    exp = o.dequant_s32_to_bf16(exp_acc, rs, cs)
    assert np.array_equal(h.result_to_oracle_repr(d, o.BF16), exp)              # same f32 ops, same rounding
    for kernel in (3, 4):
        d2, _ = xla_b200.cublas_lt_matmul_s8(ta, tb, selected_algorithm=kernel)
        assert np.array_equal(d2.cpu().numpy(), exp_acc)
    for lc, rc in [(0, 0), (1, 1), (0, 1)]:
        sa_, sb_ = _stored(a, b, lc, rc)
        d3, _ = xla_b200.cublas_lt_matmul_s8(torch.from_numpy(sa_).to(cuda_device), torch.from_numpy(sb_).to(cuda_device),
                                             lhs_contracting_dim=lc, rhs_contracting_dim=rc)
        assert np.array_equal(d3.cpu().numpy(), exp_acc)


@pytest.mark.parametrize("m", [16, 48, 64, 128])
def test_decode_shape_split_k_kernel(cuda_device, m):
    """BASELINE config 2's arrangement (M in {16,64,128}, K=8192) on a narrower weight matrix so
    that the oracle stays fast; uneven unit split across CTAs exercises the partial-tile fix-up."""
    k, n = 8192, 3584 + 16
    a, b, sa, sb = o.make_f8_operands(2, m, k, n)
    assert xla_b200._native.product.b200sd_select_kernel(m, n, k) == 2
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb)
    exp, _ = o.scaled_dot_f8(a, b, sa, sb)
    h.check_close(exp, got, o.BF16)
    got_dense, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, kernel=1)
    h.check_close(exp, got_dense, o.BF16)


def test_decode_full_width_linearity(cuda_device):
    """Full config-2 width (N=28672): size-independent checks -- the split-K and the dense kernel
    agree, and scaling a_scale by 2 scales the bf16 output exactly by 2."""
    m, k, n = 64, 8192, 28672
    a, b, sa, sb = o.make_f8_operands(2, m, k, n)
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, kernel=2)
    got_dense, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb, kernel=1)
    h.check_close(got_dense, got, o.BF16, abs_tol=1e-3, rel_tol=1e-2)
    got_auto, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb)       # 112 strips: the automatic choice is the dense kernel
    assert np.array_equal(got_auto, got_dense)
    got2, _ = h.run_scaled_dot(cuda_device, a, b, 2 * sa, sb, kernel=2)
    assert np.array_equal(o.bf16_bits_to_f32(got2), 2 * o.bf16_bits_to_f32(got))
    cols = np.random.default_rng(0).choice(n, 64, replace=False)
    exp, _ = o.scaled_dot_f8(a, np.ascontiguousarray(b[:, cols]), sa, sb)
    h.check_close(exp, got[:, cols], o.BF16)


def test_full_size_dense_properties(cuda_device):
    """8192^3 (config 1 size): spot-check sampled rows/columns against the oracle and check amax
    against the maximum of the device's own output."""
    m = k = n = 8192
    a, b, sa, sb = o.make_f8_operands(1, m, k, n)
    bias = o.make_bias_bf16(1, n)
    got, amax = h.run_scaled_dot(cuda_device, a, b, sa, sb, epilogue=o.EPI_BIAS_GELU, bias_bits=bias, d_scale=1.0,
                                 out_dtype=o.F8E4M3FN, want_amax=True)
    rows = np.random.default_rng(1).choice(m, 48, replace=False)
    exp, exp_amax_rows = o.scaled_dot_f8(np.ascontiguousarray(a[rows]), b, sa, sb, epilogue=o.EPI_BIAS_GELU,
                                         bias=o.bf16_bits_to_f32(bias), d_scale=1.0, out_dtype=o.F8E4M3FN,
                                         want_amax=True)
    assert o.fp8_within_n_values(exp, got[rows], 1) == 0
    # amax is taken before the saturating e4m3 cast: it bounds the sampled rows' own amax from above
    # and the largest stored output from below (to within half an e4m3 step); when nothing
    # saturated it also lies within half a step above it.
    top = float(np.abs(o.fp8_decode(got)).max())
    assert amax >= float(exp_amax_rows) * (1 - 1e-3)
    assert amax >= top * (1 - 1 / 16)
    if top < 448.0:
        assert amax <= top * (1 + 1 / 16)


def test_bounded_wait_reports_through_status_word(cuda_device):
    """Failure detection without a fault: a wait that nothing satisfies expires after its limit
    and the kernel reports a status bit the host can read; the context stays usable."""
    import ctypes as C
    err = C.create_string_buffer(256)
    rc = xla_b200._native.product.b200sd_wait_probe(2_000_000, torch.cuda.current_stream().cuda_stream, err, len(err))
    assert rc == 0, err.value
    assert xla_b200.device_status() == 16
    assert xla_b200.device_status() == 0
    a, b, sa, sb = o.make_f8_operands(0, 256, 512, 256)
    got, _ = h.run_scaled_dot(cuda_device, a, b, sa, sb)
    h.check_close(o.scaled_dot_f8(a, b, sa, sb)[0], got, o.BF16)


def test_execute_errors_are_reported_not_raised_as_faults(cuda_device):
    a, b, sa, sb = o.make_f8_operands(0, 256, 512, 256)
    with pytest.raises(XlaFfiError) as e:
        h.run_scaled_dot(cuda_device, a[:, :500], b[:500], sa, sb)   # k = 500 is not a multiple of 16
    assert e.value.code == 3
