"""Rewriter-lite and the fixture HLO modules (host only).

The assertions on the emitted custom call play the part of the FileCheck patterns in
xla/backends/gpu/transforms/gemm_rewriter_fp8_test.cc (operands, result tuple, backend_config);
the mini interpreter is checked against the scaled-dot oracle on the same modules.
"""
import os
import re

import numpy as np
import pytest

from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import hlo_runner
from xla_b200.scaled_dot import XlaFfiError

HLO_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hlo")


def load(name, shrink=None):
    text = open(os.path.join(HLO_DIR, name + ".hlo")).read()
    for old, new in (shrink or {}).items():
        text = re.sub(rf"\b{old}\b", str(new), text)
    return text


def roles(plan):
    return [s["role"] for s in plan["operands"]]


def call_line(hlo):
    """The custom-call instruction of a rewritten module (the first one)."""
    return next(line.strip() for line in hlo.splitlines() if " custom-call(" in line)


def test_config0_lowering():
    hlo, plan = hlo_runner.rewrite(load("c0_scaled_dot_f8"))
    assert plan["rewritten"] and plan["target"] == "b200$scaled_dot$f8" and len(plan["calls"]) == 1
    assert roles(plan) == ["a", "b", "a_scale", "b_scale"]
    assert (plan["m"], plan["k"], plan["n"]) == (256, 512, 256)
    assert plan["attrs"]["epilogue"] == o.EPI_DEFAULT and plan["attrs"]["lhs_contracting_dim"] == 1 and plan["attrs"]["rhs_contracting_dim"] == 0
    assert [r["role"] for r in plan["results"]] == ["d", "workspace"]
    assert plan["results"][0]["dtype"] == 16
    # No transposes on Blackwell (gemm_rewriter.cc:1535-1554): operands are the parameters themselves.
    assert [s["param"] for s in plan["operands"]] == [0, 1, 2, 3] and all(s["chain"] == [] for s in plan["operands"])
    assert re.search(r"= \(bf16\[256,256\], s8\[33554432\]\) custom-call\(a, b, a_scale, b_scale\), custom_call_target=\"b200\$scaled_dot\$f8\"", hlo)
    assert "api_version=API_VERSION_TYPED_FFI" in hlo and "transpose" not in hlo


def test_config1_lowering_matches_the_expected_custom_call():
    """bias + GELU + scaled e4m3 output + amax: operands a, b, a_scale, b_scale, bias, 1/out_scale;
    results (f8e4m3fn, f32[], workspace); epilogue BIAS_GELU, damax_output (thunk_emitter.cc:776-862)."""
    hlo, plan = hlo_runner.rewrite(load("c1_fp8_linear_gelu_amax"))
    assert roles(plan) == ["a", "b", "a_scale", "b_scale", "bias", "d_scale"]
    d_scale = plan["operands"][-1]
    assert d_scale["param"] == 5 and d_scale["reciprocal"]          # the HLO divides by out_scale
    assert plan["operands"][4]["dtype"] == 16 and plan["operands"][4]["param"] == 4     # the bf16 value feeding the convert
    assert plan["attrs"]["epilogue"] == o.EPI_BIAS_GELU and plan["attrs"]["damax_output"] is True
    assert [r["role"] for r in plan["results"]] == ["d", "amax", "workspace"]
    assert plan["results"][0]["dtype"] == 20
    assert "(f8e4m3fn[8192,8192], f32[], s8[33554432]) custom-call(a, b, a_scale, b_scale, bias, d_scale_inv)" in hlo
    assert "tanh" not in hlo and "clamp" not in hlo and "reduce" not in hlo     # everything was folded
    assert re.search(r"ROOT \S+ = \(f8e4m3fn\[8192,8192\], f32\[\]\) tuple\(gemm, amax", hlo)


def test_int8_lowering_folds_the_dequantisation():
    hlo, plan = hlo_runner.rewrite(load("c3_int8_dequant"))
    assert plan["target"] == "b200$dot$s8"
    assert roles(plan) == ["a", "b", "a_row_scale", "b_col_scale"]
    assert plan["results"][0]["dtype"] == 16 and plan["attrs"]["emit_s32"] is False
    assert "custom-call(a, b, a_scale, b_scale), custom_call_target=\"b200$dot$s8\"" in hlo
    assert "multiply" not in hlo and "convert" not in hlo
    # when the raw accumulator is an output of the module as well, the call returns both
    both = load("c3_int8_dequant", {"4096": 64})
    both = both.replace("ROOT ", "").rstrip().rstrip("}")
    root = re.findall(r"^\s*(\S+) = bf16\[64,64\] convert", both, flags=re.M)[-1]
    acc = re.findall(r"^\s*(\S+) = s32\[64,64\] dot", both, flags=re.M)[-1]
    both += f"  ROOT both = (bf16[64,64], s32[64,64]) tuple({root}, {acc})\n}}\n"
    hlo, plan = hlo_runner.rewrite(both)
    assert plan["attrs"]["emit_s32"] is True and [r["role"] for r in plan["results"]] == ["d", "acc", "workspace"]
    assert "(bf16[64,64], s32[64,64], s8[33554432]) custom-call(" in hlo


def test_divide_scales_e5m2_bias_relu_and_matrix_bias():
    _, plan = hlo_runner.rewrite(load("scaled_ab_divide_bias_relu_e5m2"))
    assert roles(plan) == ["a", "b", "a_scale", "b_scale", "bias"]
    assert plan["operands"][2]["reciprocal"] and plan["operands"][3]["reciprocal"]
    assert plan["operands"][1]["dtype"] == 19 and plan["attrs"]["rhs_contracting_dim"] == 1
    assert plan["attrs"]["epilogue"] == o.EPI_BIAS_RELU
    assert plan["results"][0]["dtype"] == 16                         # the final convert became the output type
    _, plan = hlo_runner.rewrite(load("unscaled_matrix_bias_f32"))
    assert roles(plan) == ["a", "b", "c", "a_scale", "b_scale"]      # c at operand index 2 (gemm_rewriter.cc:1829-1978)
    assert plan["attrs"]["beta"] == 1.0
    assert plan["operands"][3]["param"] == -1 and plan["operands"][3]["constant"] == 1.0


def test_ragged_shapes_are_padded_to_16_and_sliced():
    """PadOperandToMultipleOf16 / the slice of the result (gemm_rewriter.cc:1556-1580; FileCheck'd in
    gemm_rewriter_fp8_test.cc:521-577)."""
    hlo, plan = hlo_runner.rewrite(load("c0_scaled_dot_f8", {"256": 250, "512": 500}))
    assert plan["rewritten"] and (plan["m"], plan["k"], plan["n"]) == (250, 500, 250)
    assert plan["operands"][0]["source_dims"] == [250, 500] and plan["operands"][0]["dims"] == [256, 512]
    assert plan["operands"][0]["chain"] == ["pad"] and plan["operands"][2]["dims"] == []      # scalars are left alone
    assert plan["results"][0]["dims"] == [256, 256]
    assert "a_pad = f8e4m3fn[256,512] pad(a, zero" in hlo and "padding=0_6x0_12" in hlo
    assert "(bf16[256,256], s8[33554432]) custom-call(a_pad, b_pad, a_scale, b_scale)" in hlo
    assert re.search(r"= bf16\[250,250\] slice\(gemm\), slice=\{\[0:250\], \[0:250\]\}", hlo)
    _, plan = hlo_runner.rewrite(load("c0_scaled_dot_f8"))
    assert plan["operands"][0]["chain"] == []


def test_batched_dot_lowering_and_interpreter():
    """BatchedScaledABUnscaledDF8 (gemm_rewriter_fp8_test.cc:941-991): batch dimension 0 stays on the operands, the
    dimension numbers are kept in the rank-3 index space; no transposes on Blackwell."""
    text = load("batched_scaled_ab_f32")
    hlo, plan = hlo_runner.rewrite(text)
    assert plan["rewritten"] and plan["batch"] == 10 and (plan["m"], plan["k"], plan["n"]) == (16, 32, 16)
    assert plan["attrs"]["lhs_contracting_dim"] == 2 and plan["attrs"]["rhs_contracting_dim"] == 1
    assert plan["attrs"]["lhs_batch_dims"] == [0] and plan["attrs"]["rhs_batch_dims"] == [0]
    assert "(f32[10,16,16], s8[33554432]) custom-call(a, b, a_scale, b_scale)" in hlo
    # ragged matrix dimensions are padded, the batch dimension is not
    _, plan = hlo_runner.rewrite(load("batched_scaled_ab_f32", {"10": 7, "16": 20}))
    assert plan["operands"][0]["dims"] == [7, 32, 32] and plan["results"][0]["dims"] == [7, 32, 32]
    rng = np.random.default_rng(3)
    a = o.fp8_encode(rng.standard_normal((10, 16, 32), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((10, 32, 16), dtype=np.float32), "e4m3fn")
    out = hlo_eval.evaluate(text, [a, b, np.float32(0.5), np.float32(2.0)])
    for i in range(10):
        exp = o.scaled_dot_f8(a[i], b[i], 0.5, 2.0, out_dtype=o.F32)[0]
        np.testing.assert_allclose(out[i], exp, rtol=1e-6, atol=1e-6)
    # a batch dimension that is not the major-most one of its buffer: still one call, behind a transpose
    mixed = text.replace("rhs_batch_dims={0}", "rhs_batch_dims={2}").replace("rhs_contracting_dims={1}", "rhs_contracting_dims={0}")
    mixed = re.sub(r"\[10,32,16\]", "[32,16,10]", mixed)
    hlo, plan = hlo_runner.rewrite(mixed)
    assert plan["rewritten"] and "transpose" in plan["operands"][1]["chain"] and plan["batch"] == 10


def test_alpha_and_output_scale_without_an_fp8_cast():
    """ScaledABAlphaDF8 (gemm_rewriter_fp8_test.cc:993-1047): a constant factor behind the dot becomes alpha_real.
    UnscaledABScaledF32DF8 (:1514-1561, F8ScaleD gemm_rewriter.cc:1593-1633): a scalar factor on a non-FP8 result
    travels as a_scale -- only while a_scale is still the constant 1."""
    text = load("scaled_ab_alpha_f32")
    hlo, plan = hlo_runner.rewrite(text)
    assert plan["attrs"]["alpha_real"] == 3.0 and roles(plan) == ["a", "b", "a_scale", "b_scale"]
    assert "alpha_real = 3.0 : f64" in hlo and "multiply" not in hlo
    rng = np.random.default_rng(11)
    a = o.fp8_encode(rng.standard_normal((48, 64), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32), "e4m3fn")
    out = hlo_eval.evaluate(text, [a, b, np.float32(0.5), np.float32(0.25)])
    np.testing.assert_allclose(out, o.scaled_dot_f8(a, b, 0.5, 0.25, alpha=3.0, out_dtype=o.F32)[0], rtol=1e-6, atol=1e-6)

    text = load("unscaled_ab_scaled_f32_d")
    _, plan = hlo_runner.rewrite(text)
    assert roles(plan) == ["a", "b", "a_scale", "b_scale"]
    assert plan["operands"][2]["param"] == 2 and not plan["operands"][2]["reciprocal"]       # out_scale took a_scale's place
    assert plan["operands"][3]["param"] == -1 and plan["operands"][3]["constant"] == 1.0
    assert plan["results"][0]["dtype"] == 11
    _, plan = hlo_runner.rewrite(text.replace("multiply(dot0, s_b)", "divide(dot0, s_b)"))
    assert plan["operands"][2]["param"] == 2 and plan["operands"][2]["reciprocal"]
    # with scaled operands the factor cannot be forwarded: the dot still becomes a call, the multiply stays behind it
    scaled = load("c0_scaled_dot_f8").replace("ROOT out = bf16[256,256] dot(", "dot0 = f32[256,256] dot(")
    head, _, _ = scaled.rpartition("}")
    scaled = head + "  s = f32[] parameter(4)\n  s_b = f32[256,256] broadcast(s), dimensions={}\n  ROOT out = f32[256,256] multiply(dot0, s_b)\n}\n"
    assert "multiply(dot0, s_b)" in scaled and "dot0 = f32[256,256] dot(" in scaled
    hlo, plan = hlo_runner.rewrite(scaled)
    assert plan["rewritten"] and [s["param"] for s in plan["operands"]] == [0, 1, 2, 3]
    assert re.search(r"ROOT out = f32\[256,256\] multiply\(gemm, s_b\)", hlo)


def test_bare_fp8_dot():
    """UnscaledABUnscaledDF8 (gemm_rewriter_fp8_test.cc:313-350): custom-call(a, b, 1, 1) with an FP8 result and no
    d_scale operand of its own -- the emitter then reads the last operand as d_scale (thunk_emitter.cc:812-818)."""
    hlo, plan = hlo_runner.rewrite(load("bare_fp8_dot"))
    assert roles(plan) == ["a", "b", "a_scale", "b_scale"] and plan["results"][0]["dtype"] == 20
    assert all(s["param"] == -1 and s["constant"] == 1.0 for s in plan["operands"][2:])
    assert "(f8e4m3fn[32,48], s8[33554432]) custom-call(a, b, a_scale_one, b_scale_one)" in hlo


def test_combined_epilogues():
    """ScaledABScaledDMatrixBiasWithDAmaxF8 (gemm_rewriter_fp8_test.cc:1839-1917): a, b, c, a_scale, b_scale, d_scale ->
    (FP8, amax).  ScaledABScaledDReluActivationF8 with amax (:2715-2790): after ReLU the amax reduce needs no abs."""
    text = load("matrix_bias_scaled_d_amax")
    _, plan = hlo_runner.rewrite(text)
    assert roles(plan) == ["a", "b", "c", "a_scale", "b_scale", "d_scale"] and plan["operands"][5]["reciprocal"]
    assert plan["attrs"]["beta"] == 1.0 and plan["attrs"]["damax_output"] is True and plan["attrs"]["epilogue"] == o.EPI_DEFAULT
    rng = np.random.default_rng(14)
    a = o.fp8_encode(rng.standard_normal((64, 128), dtype=np.float32) * 4, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((128, 96), dtype=np.float32) * 4, "e4m3fn")
    c = o.f32_to_bf16_bits(rng.standard_normal((64, 96), dtype=np.float32))
    half, quarter = (o.f32_to_bf16_bits(np.float32(v)) for v in (0.5, 0.25))
    d, amax = hlo_eval.evaluate(text, [a, b, c, half, quarter, half])
    exp, exp_amax = o.scaled_dot_f8(a, b, 0.5, 0.25, c=o.bf16_bits_to_f32(c), beta=1.0, d_scale=2.0, out_dtype=o.F8E4M3FN, want_amax=True)
    # the module computes in bf16, the oracle call in f32: an element may sit one e4m3 step away, or -- where the
    # sum cancels -- within the ErrorSpec{0.1, 0.1} the reference's own test of this pattern uses (gemm_rewriter_fp8_test.cc:1882)
    fe, fd = o.fp8_decode(exp, "e4m3fn"), o.fp8_decode(d, "e4m3fn")
    far = np.abs(o.fp8_ordinal(exp).astype(np.int64) - o.fp8_ordinal(d).astype(np.int64)) > 1
    assert int((far & (np.abs(fe - fd) > 0.1) & (np.abs(fe - fd) > 0.1 * np.abs(fe))).sum()) == 0
    assert float(o.bf16_bits_to_f32(amax)) == pytest.approx(float(exp_amax), rel=1e-2)

    text = load("relu_amax_e5m2_out")
    _, plan = hlo_runner.rewrite(text)
    assert roles(plan) == ["a", "b", "a_scale", "b_scale", "d_scale"] and not plan["operands"][4]["reciprocal"]
    assert plan["attrs"]["epilogue"] == o.EPI_RELU and plan["attrs"]["damax_output"] is True
    assert plan["operands"][1]["dtype"] == 19 and plan["results"][0]["dtype"] == 19
    a = o.fp8_encode(rng.standard_normal((48, 64), dtype=np.float32) * 4, "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 80), dtype=np.float32) * 4, "e5m2")
    d, amax = hlo_eval.evaluate(text, [a, b, np.float32(0.5), np.float32(0.5), np.float32(1.5)])
    exp, exp_amax = o.scaled_dot_f8(a, b, 0.5, 0.5, b_kind="e5m2", epilogue=o.EPI_RELU, d_scale=1.5, out_dtype=o.F8E5M2, want_amax=True)
    assert o.fp8_within_n_values(exp, d, 1) == 0 and float(amax) == pytest.approx(float(exp_amax), rel=1e-6)


LAYOUT_TEMPLATE = """HloModule layouts
ENTRY main {
  x = f8e4m3fn<<A>><<AL>> parameter(0)
  x_f32 = f32<<A>><<AL>> convert(x)
  x_scale = f32[] parameter(2)
  x_sb = f32<<A>> broadcast(x_scale), dimensions={}
  x_dq = f32<<A>> multiply(x_f32, x_sb)
  y = f8e4m3fn<<B>><<BL>> parameter(1)
  y_f32 = f32<<B>><<BL>> convert(y)
  y_scale = f32[] parameter(3)
  y_sb = f32<<B>> broadcast(y_scale), dimensions={}
  y_dq = f32<<B>> multiply(y_f32, y_sb)
  ROOT out = f32[64,16]<<OL>> dot(x_dq, y_dq), lhs_contracting_dims={<<LC>>}, rhs_contracting_dims={<<RC>>}
}
"""


def layout_cases():
    for d_col in (False, True):
        for a_col in (False, True):
            for b_col in (False, True):
                for lc in (0, 1):
                    for rc in (0, 1):
                        yield d_col, a_col, b_col, lc, rc


def layout_module(d_col, a_col, b_col, lc, rc):
    rep = {"<<A>>": "[64,32]" if lc == 1 else "[32,64]", "<<B>>": "[32,16]" if rc == 0 else "[16,32]",
           "<<AL>>": "{0,1}" if a_col else "{1,0}", "<<BL>>": "{0,1}" if b_col else "{1,0}", "<<OL>>": "{0,1}" if d_col else "{1,0}",
           "<<LC>>": str(lc), "<<RC>>": str(rc)}
    text = LAYOUT_TEMPLATE
    for key, val in rep.items():
        text = text.replace(key, val)
    return text


@pytest.mark.parametrize("d_col,a_col,b_col,lc,rc", list(layout_cases()))
def test_all_32_layout_combinations_are_rewritten(d_col, a_col, b_col, lc, rc):
    """ScaledABUnscaledDF8Parameterized (gemm_rewriter_fp8_test.cc:2825-2890): row / column-major A, B and D with either
    contracting dimension.  The call takes row-major buffers only, so the plan must describe the same product."""
    hlo, plan = hlo_runner.rewrite(layout_module(d_col, a_col, b_col, lc, rc))
    assert plan["rewritten"], plan
    a, b = plan["operands"][0], plan["operands"][1]
    L, R = plan["attrs"]["lhs_contracting_dim"], plan["attrs"]["rhs_contracting_dim"]
    assert a["dims"][L] == 32 and b["dims"][R] == 32                           # both contract over k = 32
    want = (16, 64) if d_col else (64, 16)                                      # D^T when the result is column-major
    assert (a["dims"][1 - L], b["dims"][1 - R]) == want and tuple(plan["results"][0]["dims"]) == want
    assert plan["swapped"] == d_col
    first, second = (b_col, a_col) if d_col else (a_col, b_col)                 # the operands swap places for D^T
    assert ("bitcast" in a["chain"]) == first and ("bitcast" in b["chain"]) == second     # a column-major buffer read as the row-major matrix it is
    assert a["param"] == (1 if d_col else 0) and plan["operands"][2]["param"] == (3 if d_col else 2)
    assert "transpose" not in hlo and " copy(" not in hlo


def test_tiny_int8_dot_is_padded_and_sliced():
    """Int8Gemm / Int8GemmNotMultipleOfFour (gemm_rewriter_test.cc:3182-3209, 3324-3368): the reference pads s8 operands
    (CublasPadForGemms, to multiples of 4) and slices the s32 result; this library's unit is 16."""
    text = load("int8_12x4x8")
    hlo, plan = hlo_runner.rewrite(text)
    assert plan["target"] == "b200$dot$s8" and plan["results"][0]["dtype"] == 4
    assert [s["dims"] for s in plan["operands"]] == [[16, 16], [16, 16]] and plan["results"][0]["dims"] == [16, 16]
    assert "slice={[0:12], [0:8]}" in hlo
    rng = np.random.default_rng(18)
    a = rng.integers(-127, 128, (12, 4), dtype=np.int8)
    b = rng.integers(-127, 128, (4, 8), dtype=np.int8)
    assert np.array_equal(hlo_eval.evaluate(text, [a, b]), a.astype(np.int32) @ b.astype(np.int32))


def test_int8_dot_with_an_f32_result():
    """s8 x s8 -> f32 is a row of the run-time type table next to s8 x s8 -> s32 (cuda_blas_lt.cc:444-445): taken by the
    s8 call with an f32 D; epilogue ops behind it (here a ReLU) are not folded into the integer call."""
    text = """HloModule int8_f32
ENTRY main {
  a = s8[48,64] parameter(0)
  b = s8[64,32] parameter(1)
  d = f32[48,32] dot(a, b), lhs_contracting_dims={1}, rhs_contracting_dims={0}
  z = f32[] constant(0)
  zb = f32[48,32] broadcast(z), dimensions={}
  ROOT r = f32[48,32] maximum(d, zb)
}
"""
    hlo, plan = hlo_runner.rewrite(text)
    (c,) = plan["calls"]
    assert c["target"] == "b200$dot$s8" and c["results"][0]["dtype"] == 11 and (c["m"], c["n"], c["k"]) == (48, 32, 64)
    assert len(c["operands"]) == 2 and c["attrs"]["emit_s32"] is False
    assert "maximum(" in hlo and " dot(" not in hlo                  # the ReLU stays an HLO op
    from xla_b200.scaled_dot import Buffer, Int8DotCall
    Int8DotCall([Buffer(2, (48, 64)), Buffer(2, (64, 32))], [Buffer(11, (48, 32)), Buffer(2, (1 << 20,))]).instantiate()
    rng = np.random.default_rng(33)
    a = rng.integers(-128, 128, (48, 64), dtype=np.int8)
    b = rng.integers(-128, 128, (64, 32), dtype=np.int8)
    want = np.maximum(a.astype(np.int64) @ b.astype(np.int64), 0).astype(np.float32)
    assert np.array_equal(hlo_eval.evaluate(text, [a, b]), want)


def test_operands_written_as_nested_instructions():
    """HLO text may spell an operand as a whole instruction (`dot(f32[..] convert(x), ...)`, as the reference's
    block_scaling_rewriter_cudnn_test.cc:147-165 does); the parser gives such operands names of their own."""
    text = """HloModule nested
ENTRY main {
  x = f8e4m3fn[64,128] parameter(0)
  w = f8e4m3fn[128,32] parameter(1)
  ROOT d = f32[64,32] dot(f32[64,128] convert(x), f32[128,32] convert(f8e4m3fn[128,32] copy(w))), lhs_contracting_dims={1}, rhs_contracting_dims={0}
}
"""
    hlo, plan = hlo_runner.rewrite(text)
    (c,) = plan["calls"]
    assert c["target"] == "b200$scaled_dot$f8" and (c["m"], c["n"], c["k"]) == (64, 32, 128)
    assert [op["param"] for op in c["operands"][:2]] == [0, 1] and c["operands"][1]["chain"] == ["copy"]
    assert " dot(" not in hlo
    # the interpreter reads the same spelling, and gives what it gives for the module written out flat
    flat = text.replace("dot(f32[64,128] convert(x), f32[128,32] convert(f8e4m3fn[128,32] copy(w)))", "dot(xf, wf)").replace(
        "  ROOT d", "  xf = f32[64,128] convert(x)\n  wf = f32[128,32] convert(w)\n  ROOT d")
    rng = np.random.default_rng(29)
    x = o.fp8_encode(rng.standard_normal((64, 128), dtype=np.float32), "e4m3fn")
    w = o.fp8_encode(rng.standard_normal((128, 32), dtype=np.float32), "e4m3fn")
    assert np.array_equal(hlo_eval.evaluate(text, [x, w]), hlo_eval.evaluate(flat, [x, w]))


def test_batched_int8_dot_keeps_its_batch_dimension():
    """s8 x s8 -> s32 is in the type table for batched dots as for plain ones (gemm_rewriter.cc:2425-2677 does not look
    at the rank); the call carries the same batch attributes as the FP8 call."""
    text = load("batched_int8")
    hlo, plan = hlo_runner.rewrite(text)
    (c,) = plan["calls"]
    assert c["target"] == "b200$dot$s8" and (c["batch"], c["m"], c["n"], c["k"]) == (3, 40, 24, 64)
    assert c["attrs"]["lhs_batch_dims"] == [0] and c["attrs"]["rhs_batch_dims"] == [0]
    assert (c["attrs"]["lhs_contracting_dim"], c["attrs"]["rhs_contracting_dim"]) == (2, 1)
    assert [s["dims"] for s in c["operands"]] == [[3, 48, 64], [3, 64, 32]] and "slice={[0:3], [0:40], [0:24]}" in hlo
    rng = np.random.default_rng(23)
    a = rng.integers(-127, 128, (3, 40, 64), dtype=np.int8)
    b = rng.integers(-127, 128, (3, 64, 24), dtype=np.int8)
    assert np.array_equal(hlo_eval.evaluate(text, [a, b]), np.matmul(a.astype(np.int32), b.astype(np.int32)))


def test_bitcast_between_dequantisation_and_dot():
    """ScaledABUnscaledDBitcastF8 (gemm_rewriter_fp8_test.cc:579-612)."""
    text = load("bitcast_operand")
    hlo, plan = hlo_runner.rewrite(text)
    assert plan["rewritten"] and (plan["m"], plan["k"], plan["n"]) == (48, 64, 32)
    assert plan["operands"][0]["dims"] == [48, 64] and plan["operands"][0]["source_dims"] == [2, 24, 64]
    assert plan["operands"][0]["chain"] == ["bitcast"] and plan["operands"][1]["chain"] == []
    assert re.search(r"(\S+) = f8e4m3fn\[48,64\] bitcast\(a\)", hlo)
    rng = np.random.default_rng(20)
    a = o.fp8_encode(rng.standard_normal((2, 24, 64), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32), "e4m3fn")
    out = hlo_eval.evaluate(text, [a, b, np.float32(0.5), np.float32(2.0)])
    np.testing.assert_allclose(out, o.scaled_dot_f8(a.reshape(48, 64), b, 0.5, 2.0, out_dtype=o.F32)[0], rtol=1e-6, atol=1e-6)


def test_rank3_activation_with_vector_bias_on_the_view():
    """Rank3ScaledABUnscaledDVectorBiasF8 (gemm_rewriter_fp8_test.cc:2112-2186): bitcast in, matrix product, bitcast out,
    bias added on the rank-3 view -- one custom call producing the [m, n] matrix, viewed as [4, 16, 32]."""
    text = load("rank3_vector_bias")
    hlo, plan = hlo_runner.rewrite(text)
    assert roles(plan) == ["a", "b", "a_scale", "b_scale", "bias"] and plan["attrs"]["epilogue"] == o.EPI_BIAS
    assert plan["operands"][0]["dims"] == [64, 64] and plan["operands"][0]["chain"] == ["bitcast"]
    assert plan["results"][0]["dims"] == [64, 32]
    assert re.search(r"ROOT \S+ = f32\[4,16,32\] bitcast\(gemm\)", hlo) and " add(" not in hlo
    rng = np.random.default_rng(22)
    a = o.fp8_encode(rng.standard_normal((4, 16, 64), dtype=np.float32), "e4m3fn")
    b = o.fp8_encode(rng.standard_normal((64, 32), dtype=np.float32), "e4m3fn")
    bias = o.make_bias_bf16(22, 32)
    out = hlo_eval.evaluate(text, [a, b, bias, np.float32(0.5), np.float32(2.0)])
    exp = o.scaled_dot_f8(a.reshape(64, 64), b, 0.5, 2.0, bias=o.bf16_bits_to_f32(bias), epilogue=o.EPI_BIAS, out_dtype=o.F32)[0]
    np.testing.assert_allclose(out.reshape(64, 32), exp, rtol=1e-6, atol=1e-6)


def test_modules_that_must_be_left_alone():
    hlo, plan = hlo_runner.rewrite(load("not_rewritten_both_e5m2"))
    assert not plan["rewritten"] and "e5m2" in plan["reason"] and plan["not_rewritten"][0]["dot"]
    assert "custom-call" not in hlo
    f32_dot = load("c0_scaled_dot_f8").replace("f8e4m3fn", "f32")
    assert not hlo_runner.rewrite(f32_dot)[1]["rewritten"]
    # The GELU pre-activation has another user: that would need the AUX epilogue, which this library does not
    # produce, so the bias is folded and the GELU arithmetic stays behind the call.
    aux = load("c1_fp8_linear_gelu_amax", {"8192": 64}).replace("tuple(d, amax)", "tuple(d, x)").replace(
        "(f8e4m3fn[64,64], f32[]) tuple", "(f8e4m3fn[64,64], f32[64,64]) tuple")
    hlo, plan = hlo_runner.rewrite(aux)
    assert plan["rewritten"] and plan["attrs"]["epilogue"] == o.EPI_BIAS and "tanh" in hlo and plan["results"][0]["dtype"] == 11
    with pytest.raises(XlaFfiError) as e:
        hlo_runner.rewrite("HloModule broken\nENTRY main {\n  x = oops\n}\n")
    assert e.value.code == 3


def test_two_dots_in_one_module_become_two_calls():
    """GemmRewriterVisitor rewrites every dot it visits (gemm_rewriter.cc:657-779): a two-layer MLP -- FP8 linear +
    GELU + scaled FP8 cast feeding a second FP8 linear -- lowers onto two calls, the second taking the first's
    FP8 result as its A operand."""
    text = load("two_layer_mlp")
    hlo, plan = hlo_runner.rewrite(text)
    assert plan["rewritten"] and len(plan["calls"]) == 2 and plan["not_rewritten"] == []
    first, second = plan["calls"]
    assert first["attrs"]["epilogue"] == o.EPI_BIAS_GELU and first["results"][0]["dtype"] == 20
    assert [s["role"] for s in second["operands"]] == ["a", "b", "a_scale", "b_scale"] and second["results"][0]["dtype"] == 16
    assert second["operands"][0]["source"] == first["name"]           # the FP8 activation never leaves FP8
    assert hlo.count(" custom-call(") == 2 and " dot(" not in hlo and "tanh" not in hlo


def test_interpreter_agrees_with_the_scaled_dot_oracle():
    m = k = n = 64
    text = load("c1_fp8_linear_gelu_amax", {"8192": 64})
    a, b, sa, sb = o.make_f8_operands(1, m, k, n)
    bias = o.make_bias_bf16(1, n)
    d, amax = hlo_eval.evaluate(text, [a, b, np.float32(sa), np.float32(sb), bias, np.float32(2.0)])
    exp, exp_amax = o.scaled_dot_f8(a, b, sa, sb, bias=o.bf16_bits_to_f32(bias), epilogue=o.EPI_BIAS_GELU, d_scale=0.5,
                                    out_dtype=o.F8E4M3FN, want_amax=True)
    assert o.fp8_within_n_values(exp, d, 1) == 0 and float((exp == d).mean()) > 0.99
    assert float(amax) == pytest.approx(float(exp_amax), rel=1e-6)
    a8, b8, rs, cs = o.make_s8_operands(3, 32, 48, 64)
    text = load("c3_int8_dequant")
    text = re.sub(r"s8\[4096,4096\] parameter\(0\)", "s8[32,48] parameter(0)", text)
    text = re.sub(r"s8\[4096,4096\] parameter\(1\)", "s8[48,64] parameter(1)", text)
    text = text.replace("f32[4096] parameter(2)", "f32[32] parameter(2)").replace("f32[4096] parameter(3)", "f32[64] parameter(3)")
    text = text.replace("[4096,4096]", "[32,64]")
    out = hlo_eval.evaluate(text, [a8, b8, rs, cs])
    assert np.array_equal(out, o.dequant_s32_to_bf16(o.dot_s8(a8, b8), rs, cs))


FIXTURES = ["c0_scaled_dot_f8", "c1_fp8_linear_gelu_amax", "c2_decode_m64", "c3_int8_dequant",
            "c4_row_parallel_rank_of_2", "scaled_ab_divide_bias_relu_e5m2", "unscaled_matrix_bias_f32",
            "batched_scaled_ab_f32", "scaled_ab_alpha_f32", "unscaled_ab_scaled_f32_d", "bare_fp8_dot",
            "matrix_bias_scaled_d_amax", "relu_amax_e5m2_out", "precision_1600x3200x1600", "int8_12x4x8", "bitcast_operand",
            "rank3_vector_bias", "two_layer_mlp", "batched_int8", "block_scaled_dot_mx"]


@pytest.mark.parametrize("name", FIXTURES)
def test_every_emitted_call_instantiates_through_the_ffi_boundary(name):
    """Every custom call of the rewritten module -- operands, result tuple, backend_config, as the text spells
    them -- must form a call frame the handler accepts at instantiate time (buffer data is null there, as in
    custom_call_thunk.cc:179-240)."""
    from xla_b200.scaled_dot import Buffer, FfiCall

    hlo, plan = hlo_runner.rewrite(load(name))
    assert plan["rewritten"], plan
    comps, entry = hlo_runner.parse_module(hlo)
    shapes = {i["name"]: i["shape"] for i in comps[entry]}
    code = {"pred": 1, "s8": 2, "s32": 4, "f16": 10, "f32": 11, "bf16": 16, "f8e5m2": 19, "f8e4m3fn": 20, "f8e8m0fnu": 33}
    n = 0
    for ins in comps[entry]:
        if ins["opcode"] != "custom-call":
            continue
        ops = [Buffer(code[shapes[o_][0]], tuple(shapes[o_][1])) for o_ in ins["operands"]]
        res = [Buffer(code[s[0]], tuple(s[1])) for s in ins["shape"][1]]
        target = re.search(r'custom_call_target="([^"]+)"', ins["attrs"]).group(1)
        call = FfiCall(target, ops, res, hlo_runner._backend_config(ins["attrs"]))
        call.instantiate()
        call.close()
        n += 1
    assert n == len(plan["calls"])


def test_small_dot_threshold_against_the_reference_cases():
    """GetMatrixSizeRewriteThresholdTest of xla/service/gpu/matmul_utils_test.cc:250-360 (tests/golden/rewrite_threshold_known.json):
    the same shapes and dimension numbers as FP8 dots -- the rewriter-lite leaves a dot to the elementwise emitters exactly
    where IsMatrixMultiplicationTooSmallForRewriting(dot, 100) holds (per batch entry, (m + n) * k < 100)."""
    import json

    with open(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rewrite_threshold_known.json")) as f:
        cases = json.load(f)["cases"]
    assert len(cases) == 4
    for c in cases:
        x, y, r = (",".join(map(str, c[k])) for k in ("x_dims", "y_dims", "result_dims"))
        text = f"""HloModule threshold
ENTRY main {{
  x = f8e4m3fn[{x}] parameter(0)
  y = f8e4m3fn[{y}] parameter(1)
  xf = f32[{x}] convert(x)
  yf = f32[{y}] convert(y)
  ROOT dot = f32[{r}] dot(xf, yf), {c['dimension_numbers']}
}}
"""
        _, plan = hlo_runner.rewrite(text)
        assert c["threshold"] == 100
        assert plan["rewritten"] == (not c["too_small"]), c["name"]
        if c["too_small"]:
            assert "too small" in plan["not_rewritten"][0]["reason"]
