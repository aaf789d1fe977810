"""The same HLO text drives the CPU interpreter and, through the rewriter-lite and the FFI
boundary, the CUDA kernels; the results must agree under the reference's tolerances."""
import os
import re

import numpy as np
import pytest
import torch

from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import hlo_runner

pytestmark = pytest.mark.gpu
HLO_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hlo")
_TORCH = {"f8e4m3fn": torch.float8_e4m3fn, "f8e5m2": torch.float8_e5m2, "bf16": torch.bfloat16}


def load(name, shrink=None):
    text = open(os.path.join(HLO_DIR, name + ".hlo")).read()
    for old, new in (shrink or {}).items():
        text = re.sub(rf"\b{old}\b", str(new), text)
    return text


def to_dev(v, kind, dev):
    t = torch.from_numpy(np.ascontiguousarray(v)).to(dev)
    if kind in ("f8e4m3fn", "f8e5m2"):
        return t.view(_TORCH[kind])
    if kind == "bf16":
        return t.view(torch.int16).view(torch.bfloat16)
    return t


def back(t):
    if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
        return t.view(torch.uint8).cpu().numpy()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).cpu().numpy().view(np.uint16)
    return t.cpu().numpy()


def test_config0_module(cuda_device):
    text = load("c0_scaled_dot_f8")
    a, b, sa, sb = o.make_f8_operands(0, 256, 512, 256)
    exp = hlo_eval.evaluate(text, [a, b, np.float32(sa), np.float32(sb)])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device)])
    torch.cuda.synchronize()
    assert o.near_mismatches(o.bf16_bits_to_f32(exp), o.bf16_bits_to_f32(back(got)), 1e-2, 1e-2)[0] == 0


def test_config1_module_reduced(cuda_device):
    text = load("c1_fp8_linear_gelu_amax", {"8192": 512})
    a, b, sa, sb = o.make_f8_operands(1, 512, 512, 512)
    bias = o.make_bias_bf16(1, 512)
    out_scale = np.float32(0.5)
    exp_d, exp_amax = hlo_eval.evaluate(text, [a, b, np.float32(sa), np.float32(sb), bias, out_scale])
    d, amax = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                               torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device),
                                               to_dev(bias, "bf16", cuda_device), torch.tensor(out_scale, device=cuda_device)])
    torch.cuda.synchronize()
    assert o.fp8_within_n_values(exp_d, back(d), 1) == 0
    assert float(amax.item()) == pytest.approx(float(exp_amax), rel=1e-3)


def test_config3_module_reduced(cuda_device):
    text = load("c3_int8_dequant", {"4096": 256})
    a, b, rs, cs = o.make_s8_operands(3, 256, 256, 256)
    exp = hlo_eval.evaluate(text, [a, b, rs, cs])
    got = hlo_runner.run_hlo_module(text, [torch.from_numpy(x).to(cuda_device) for x in (a, b, rs, cs)])
    torch.cuda.synchronize()
    assert np.array_equal(back(got), exp)                      # integer path: bit-exact, also after the dequantisation


def test_divide_scales_e5m2_bias_relu_and_matrix_bias_modules(cuda_device):
    rng = np.random.default_rng(5)
    text = load("scaled_ab_divide_bias_relu_e5m2")
    a = o.fp8_encode(rng.standard_normal((64, 128), dtype=np.float32) * 8, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((96, 128), dtype=np.float32) * 8, "e5m2")
    sa, sb = np.float32(4.0), np.float32(0.5)
    bias = o.f32_to_bf16_bits(rng.standard_normal(96, dtype=np.float32))
    exp = hlo_eval.evaluate(text, [a, b, sa, sb, bias])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e5m2", cuda_device),
                                           torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device),
                                           to_dev(bias, "bf16", cuda_device)])
    torch.cuda.synchronize()
    assert o.near_mismatches(o.bf16_bits_to_f32(exp), o.bf16_bits_to_f32(back(got)), 1e-2, 1e-2)[0] == 0
    text = load("unscaled_matrix_bias_f32")
    a = o.fp8_encode(rng.standard_normal((48, 64), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 80), dtype=np.float32), "e4m3fn")
    c = rng.standard_normal((48, 80), dtype=np.float32)
    exp = hlo_eval.evaluate(text, [a, b, c])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.from_numpy(c).to(cuda_device)])
    torch.cuda.synchronize()
    assert o.near_mismatches(exp, back(got), 1e-2, 1e-2)[0] == 0


def test_ragged_module_is_padded_and_sliced(cuda_device):
    text = load("c1_fp8_linear_gelu_amax", {"8192": 200})            # 200 is not a multiple of 16
    a, b, sa, sb = o.make_f8_operands(7, 200, 200, 200)
    bias = o.make_bias_bf16(7, 200)
    out_scale = np.float32(2.0)
    exp_d, exp_amax = hlo_eval.evaluate(text, [a, b, np.float32(sa), np.float32(sb), bias, out_scale])
    d, amax = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                               torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device),
                                               to_dev(bias, "bf16", cuda_device), torch.tensor(out_scale, device=cuda_device)])
    torch.cuda.synchronize()
    assert tuple(d.shape) == (200, 200)
    assert o.fp8_within_n_values(exp_d, back(d.contiguous()), 1) == 0
    assert float(amax.item()) == pytest.approx(float(exp_amax), rel=1e-3)


def test_batched_module(cuda_device):
    rng = np.random.default_rng(9)
    for shrink, (bt, m, k, n) in [(None, (10, 16, 32, 16)), ({"10": 3, "16": 272, "32": 192}, (3, 272, 192, 272))]:
        text = load("batched_scaled_ab_f32", shrink)
        a = o.fp8_encode(rng.standard_normal((bt, m, k), dtype=np.float32) * 2, "e4m3fn")
        b = o.fp8_encode(rng.standard_normal((bt, k, n), dtype=np.float32) * 2, "e4m3fn")
        sa, sb = np.float32(0.25), np.float32(0.5)
        exp = hlo_eval.evaluate(text, [a, b, sa, sb])
        got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                               torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device)])
        torch.cuda.synchronize()
        assert tuple(got.shape) == (bt, m, n)
        assert o.near_mismatches(exp, back(got), 1e-3, 1e-4)[0] == 0


def test_alpha_and_output_scale_modules(cuda_device):
    rng = np.random.default_rng(12)
    text = load("scaled_ab_alpha_f32")
    a = o.fp8_encode(rng.standard_normal((48, 64), dtype=np.float32) * 2, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32) * 2, "e4m3fn")
    sa, sb = np.float32(0.5), np.float32(0.125)
    exp = hlo_eval.evaluate(text, [a, b, sa, sb])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device)])
    torch.cuda.synchronize()
    assert o.near_mismatches(exp, back(got), 1e-3, 1e-4)[0] == 0
    text = load("unscaled_ab_scaled_f32_d")
    a = o.fp8_encode(rng.standard_normal((32, 64), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 48), dtype=np.float32), "e4m3fn")
    s = np.float32(0.75)
    exp = hlo_eval.evaluate(text, [a, b, s])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.tensor(s, device=cuda_device)])
    torch.cuda.synchronize()
    assert o.near_mismatches(exp, back(got), 1e-3, 1e-4)[0] == 0


def test_bare_fp8_dot_module(cuda_device):
    text = load("bare_fp8_dot")
    rng = np.random.default_rng(13)
    a = o.fp8_encode(rng.standard_normal((32, 64), dtype=np.float32) * 0.5, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 48), dtype=np.float32) * 0.5, "e4m3fn")
    exp = hlo_eval.evaluate(text, [a, b])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device)])
    torch.cuda.synchronize()
    assert o.fp8_within_n_values(exp, back(got), 1) == 0


def test_combined_epilogue_modules(cuda_device):
    rng = np.random.default_rng(15)
    dev = cuda_device
    text = load("matrix_bias_scaled_d_amax")                 # bf16 throughout, as the reference's f16 test of the pattern
    a = o.fp8_encode(rng.standard_normal((64, 128), dtype=np.float32) * 4, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((128, 96), dtype=np.float32) * 4, "e4m3fn")
    c = o.f32_to_bf16_bits(rng.standard_normal((64, 96), dtype=np.float32))
    sa, sb, ds = (o.f32_to_bf16_bits(np.float32(v)) for v in (0.5, 0.25, 0.5))
    exp_d, exp_amax = hlo_eval.evaluate(text, [a, b, c, sa, sb, ds])
    d, amax = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", dev), to_dev(b, "f8e4m3fn", dev), to_dev(c, "bf16", dev),
                                               to_dev(sa, "bf16", dev), to_dev(sb, "bf16", dev), to_dev(ds, "bf16", dev)])
    torch.cuda.synchronize()
    # the interpreter rounds the dot to bf16 before adding the bias, the call adds in f32: ErrorSpec{0.1, 0.1} of the
    # reference's test of this pattern (gemm_rewriter_fp8_test.cc:1882), or one e4m3 step
    fe, fd = o.fp8_decode(exp_d, "e4m3fn"), o.fp8_decode(back(d), "e4m3fn")
    far = np.abs(o.fp8_ordinal(exp_d).astype(np.int64) - o.fp8_ordinal(back(d)).astype(np.int64)) > 1
    assert int((far & (np.abs(fe - fd) > 0.1) & (np.abs(fe - fd) > 0.1 * np.abs(fe))).sum()) == 0
    assert amax.dtype == torch.bfloat16
    assert float(amax.float().item()) == pytest.approx(float(o.bf16_bits_to_f32(exp_amax)), rel=1e-2)

    text = load("relu_amax_e5m2_out")
    a = o.fp8_encode(rng.standard_normal((48, 64), dtype=np.float32) * 4, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 80), dtype=np.float32) * 4, "e5m2")
    sa, sb, dm = np.float32(0.5), np.float32(0.5), np.float32(1.5)
    exp_d, exp_amax = hlo_eval.evaluate(text, [a, b, sa, sb, dm])
    d, amax = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", dev), to_dev(b, "f8e5m2", dev), torch.tensor(sa, device=dev),
                                               torch.tensor(sb, device=dev), torch.tensor(dm, device=dev)])
    torch.cuda.synchronize()
    assert o.fp8_within_n_values(exp_d, back(d), 1) == 0
    assert float(amax.item()) == pytest.approx(float(exp_amax), rel=1e-4)


def test_all_32_layout_combinations_run(cuda_device):
    """ScaledABUnscaledDF8Parameterized (gemm_rewriter_fp8_test.cc:2825-2890) end to end: column-major operands are
    handed over as the row-major matrices they are, a column-major result comes back as D^T."""
    from test_hlo_rewriter import layout_cases, layout_module

    rng = np.random.default_rng(16)
    dev = cuda_device
    sa, sb = np.float32(0.5), np.float32(0.25)
    for d_col, a_col, b_col, lc, rc in layout_cases():
        text = layout_module(d_col, a_col, b_col, lc, rc)
        a_shape = (64, 32) if lc == 1 else (32, 64)
        b_shape = (32, 16) if rc == 0 else (16, 32)
        a = o.fp8_encode(rng.standard_normal(a_shape, dtype=np.float32) * 2, "e4m3fn")
        b = o.fp8_encode(rng.standard_normal(b_shape, dtype=np.float32) * 2, "e4m3fn")
        exp = hlo_eval.evaluate(text, [a, b, sa, sb])                       # layouts do not change what is computed

        def device_param(x, col):      # logical tensor whose memory is column-major when the module says so
            t = to_dev(np.ascontiguousarray(x.T) if col else x, "f8e4m3fn", dev)
            return t.t() if col else t

        got = hlo_runner.run_hlo_module(text, [device_param(a, a_col), device_param(b, b_col), torch.tensor(sa, device=dev),
                                               torch.tensor(sb, device=dev)])
        torch.cuda.synchronize()
        assert tuple(got.shape) == (64, 16)
        case = f"d_col={d_col} a_col={a_col} b_col={b_col} lc={lc} rc={rc}"
        assert o.near_mismatches(exp, got.contiguous().cpu().numpy(), 1e-3, 1e-4)[0] == 0, case


def test_precision_module_meets_the_highest_precision_bound(cuda_device):
    """UnscaledABUnscaledDPrecisionF8 (gemm_rewriter_fp8_test.cc:2793-2823): 1600 x 3200 x 1600, f32 result within
    ErrorSpec{1e-3, 1e-3} of the interpreter at default precision and {1e-4, 1e-4} at `highest`.  The kernel has one
    accumulation mode (full f32 in TMEM), so it has to meet the tighter bound."""
    text = load("precision_1600x3200x1600")
    rng = np.random.default_rng(17)
    a = o.fp8_encode(rng.standard_normal((1600, 3200), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((3200, 1600), dtype=np.float32), "e4m3fn")
    sa, sb = np.float32(1.0), np.float32(1.0)
    exp = hlo_eval.evaluate(text, [a, b, sa, sb])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device)])
    torch.cuda.synchronize()
    got = back(got)
    assert o.near_mismatches(exp, got, 1e-3, 1e-3)[0] == 0
    assert o.near_mismatches(exp, got, 1e-4, 1e-4)[0] == 0


def test_tiny_int8_module(cuda_device):
    text = load("int8_12x4x8")
    rng = np.random.default_rng(19)
    a = rng.integers(-127, 128, (12, 4), dtype=np.int8)
    b = rng.integers(-127, 128, (4, 8), dtype=np.int8)
    got = hlo_runner.run_hlo_module(text, [torch.from_numpy(a).to(cuda_device), torch.from_numpy(b).to(cuda_device)])
    torch.cuda.synchronize()
    assert tuple(got.shape) == (12, 8)
    assert np.array_equal(got.cpu().numpy(), a.astype(np.int32) @ b.astype(np.int32))     # bit-exact


def test_batched_int8_module(cuda_device):
    text = load("batched_int8")
    rng = np.random.default_rng(24)
    a = rng.integers(-128, 128, (3, 40, 64), dtype=np.int8)
    b = rng.integers(-128, 128, (3, 64, 24), dtype=np.int8)
    got, stats = hlo_runner.run_hlo_module(text, [torch.from_numpy(a).to(cuda_device), torch.from_numpy(b).to(cuda_device)], return_stats=True)
    torch.cuda.synchronize()
    assert stats["custom_calls"] == 1 and tuple(got.shape) == (3, 40, 24)
    assert np.array_equal(got.cpu().numpy(), hlo_eval.evaluate(text, [a, b]))          # bit-exact
    assert np.array_equal(got.cpu().numpy(), np.stack([o.dot_s8(a[i], b[i]) for i in range(3)]))


def test_bitcast_operand_module(cuda_device):
    text = load("bitcast_operand")
    rng = np.random.default_rng(21)
    a = o.fp8_encode(rng.standard_normal((2, 24, 64), dtype=np.float32) * 2, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32) * 2, "e4m3fn")
    sa, sb = np.float32(0.5), np.float32(0.25)
    exp = hlo_eval.evaluate(text, [a, b, sa, sb])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           torch.tensor(sa, device=cuda_device), torch.tensor(sb, device=cuda_device)])
    torch.cuda.synchronize()
    assert tuple(got.shape) == (48, 32)
    assert o.near_mismatches(exp, back(got), 1e-3, 1e-4)[0] == 0


def test_rank3_vector_bias_module(cuda_device):
    text = load("rank3_vector_bias")
    rng = np.random.default_rng(23)
    a = o.fp8_encode(rng.standard_normal((4, 16, 64), dtype=np.float32) * 2, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32) * 2, "e4m3fn")
    bias = o.make_bias_bf16(23, 32)
    sa, sb = np.float32(0.5), np.float32(0.25)
    exp = hlo_eval.evaluate(text, [a, b, bias, sa, sb])
    got = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                           to_dev(bias, "bf16", cuda_device), torch.tensor(sa, device=cuda_device),
                                           torch.tensor(sb, device=cuda_device)])
    torch.cuda.synchronize()
    assert tuple(got.shape) == (4, 16, 32)
    assert o.near_mismatches(exp, back(got), 1e-3, 1e-4)[0] == 0


def test_two_layer_mlp_module(cuda_device):
    """Two dots in one module become two calls; the FP8 activation between them never leaves FP8."""
    text = load("two_layer_mlp")
    rng = np.random.default_rng(24)
    dev = cuda_device
    x = o.fp8_encode(rng.standard_normal((64, 128), dtype=np.float32) * 2, "e4m3fn")
    w1 = o.fp8_encode(rng.standard_normal((128, 256), dtype=np.float32) * 2, "e4m3fn")
    w2 = o.fp8_encode(rng.standard_normal((256, 96), dtype=np.float32) * 2, "e4m3fn")
    b1 = o.make_bias_bf16(24, 256)
    scales = [np.float32(v) for v in (0.25, 0.125, 0.25, 0.03125)]
    exp = hlo_eval.evaluate(text, [x, w1, w2, *scales, b1])
    got, stats = hlo_runner.run_hlo_module(
        text, [to_dev(x, "f8e4m3fn", dev), to_dev(w1, "f8e4m3fn", dev), to_dev(w2, "f8e4m3fn", dev),
               *[torch.tensor(v, device=dev) for v in scales], to_dev(b1, "bf16", dev)], return_stats=True)
    torch.cuda.synchronize()
    assert stats["custom_calls"] == 2
    # the hidden activation is an e4m3 value: where the kernel's GELU lands on the other side of a rounding boundary it is one
    # e4m3 step (up to 12.5 %) away, which the second dot averages over 256 terms
    assert o.near_mismatches(o.bf16_bits_to_f32(exp), o.bf16_bits_to_f32(back(got)), 2e-2, 2e-2)[0] == 0


def test_block_scaled_dot_module(cuda_device):
    """`__op$block_scaled_dot` with MX operands: rewritten onto b200$block_scaled_dot$mx, run through the FFI boundary,
    compared with the interpreter's evaluation of the same text (which equals the reference's expansion,
    tests/test_mx_hlo.py)."""
    text = load("block_scaled_dot_mx")
    a, b, sa, sb = o.make_mx_operands(77, 16, 32, 256, batch=4)
    exp = hlo_eval.evaluate(text, [a, b, sa, sb])
    got, stats = hlo_runner.run_hlo_module(text, [to_dev(a, "f8e4m3fn", cuda_device), to_dev(b, "f8e4m3fn", cuda_device),
                                                  to_dev(sa, "u8", cuda_device).view(torch.float8_e8m0fnu),
                                                  to_dev(sb, "u8", cuda_device).view(torch.float8_e8m0fnu)], return_stats=True)
    torch.cuda.synchronize()
    assert stats["custom_calls"] == 1
    absdot = np.matmul(np.abs(o.mx_dequantize(a, sa)).astype(np.float64), np.swapaxes(np.abs(o.mx_dequantize(b, sb)).astype(np.float64), -1, -2))
    assert (np.abs(back(got).astype(np.float64) - exp) <= absdot * 2.0 ** -16 + np.abs(exp) * 2.0 ** -23).all()
