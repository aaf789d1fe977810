"""The reference's own `__op$block_scaled_dot` test modules (tests/golden/ref_block_scaled.json, extracted as text by
tests/golden/make_ref_rewrites.py from block_scaling_rewriter_test.cc and block_scaling_rewriter_cudnn_test.cc) against
the rewriter-lite and the oracle, on CPU.

The reference, given a library with block-scaled kernels, hands the MX forms to it and expands every other form into
dequantize + dot.  The rewriter-lite must make the same decision for the MX forms with FP8 values (the kernels this
library has); the 4-bit NVFP4 forms are not implemented and must stay with the expansion."""
import json
import os
import re

import numpy as np
import pytest

from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import hlo_runner

import ref_cases

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "ref_block_scaled.json")) as f:
    _FIXTURE = json.load(f)
CASES = _FIXTURE["cases"]
SCALED_DOT = _FIXTURE["scaled_dot"]          # modules built on the `scaled-dot` instruction
BY_NAME = {c["name"]: c for c in CASES}
# What the rewriter-lite makes of each `scaled-dot` module, with the reason where it differs from cuDNN's answer.
SCALED_DOT_TAKEN = {
    "CudnnFusionSupportedE4M3": True,
    "CudnnFusionUnsupportedE5M2": True,          # a cuDNN restriction; tcgen05 kind::mxf8f6f4 multiplies e5m2 x e5m2 (tests/test_gpu_mx.py)
    "CudnnFusionUnsupportedDimensions": True,    # rhs is [k, n]: transposed (with its scales) in front of the call
    "CudnnFusionUnupportedLayout": False,        # column-major lhs
    "CudnnFusionUnsupportedInputs": True,        # a rule about cuDNN fusion inputs (a broadcast); a custom call takes any value
    "MxFp8Correctness": True, "MxFp8BatchedCorrectness": True, "MxFp8MixedTypesBatchedCorrectness": True,
    "MxFp8ReshapedOperandsCorrectness": True,
    "MxFp4Correctness": False, "MxFp4BatchedCorrectness": False, "MxFp4Fp8MixedBatchedCorrectness": False,   # 4-bit values: not implemented
}


def is_mx_fp8(case) -> bool:
    """FP8 values with f8e8m0fnu scales: the MXFP8 form (block_scaling_rewriter.cc:280-293)."""
    call = case["hlo"][case["hlo"].index("ROOT"):]
    names = re.search(r"custom-call\(([^)]*)\)", call).group(1).replace("%", "").split(",")
    types = []
    for n in names:
        m = re.search(r"%" + re.escape(n.strip()) + r"\s*=\s*([a-z0-9]+)\[", case["hlo"])
        types.append(m.group(1))
    return (len(types) == 4 and all(t in ("f8e4m3fn", "f8e5m2") for t in types[:2]) and all(t == "f8e8m0fnu" for t in types[2:]))


def test_the_fixture_holds_the_reference_tests():
    assert len(CASES) == 13
    assert sorted(c["name"] for c in CASES if c["library"]) == sorted([
        "CudnnScaledDotSimple", "CudnnScaledDotTransforms", "CudnnScaledDotPaddedScales", "Mxfp8", "Mxfp8_MixedTypes",
        "Mxfp8_PaddedScales", "Nvfp4", "Nvfp4_GlobalScale"])
    assert all(c["error_spec"] == [1e-4, 1e-5] for c in CASES if c["numeric"])


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_rewriter_decides_as_the_reference_does(case):
    hlo, plan = hlo_runner.rewrite(case["hlo"])
    if "f4e2m1fn" in case["hlo"]:
        # NVFP4 (4-bit values, e4m3 scales per 16, optionally a global scale): not implemented, left to the expansion.
        # (These modules also spell operands as nested instructions, `convert(f16[..] multiply(%p0, %mult))`.)
        assert not plan["rewritten"] and "block-scaled" in plan["not_rewritten"][0]["reason"]
        return
    if case["library"] and is_mx_fp8(case):
        assert plan["rewritten"] and not plan["not_rewritten"], case["name"]
        (c,) = plan["calls"]
        assert c["target"] == "b200$block_scaled_dot$mx"
        assert [x["role"] for x in c["operands"]] == ["a", "b", "a_scale", "b_scale"]
        params = {n: (t, d) for n, t, d in ref_cases.parameters(case["hlo"])}
        a_dims, b_dims = params[0][1], params[1][1]
        assert (c["m"], c["n"], c["k"]) == (a_dims[-2], b_dims[-2], a_dims[-1])
        assert c["batch"] == (a_dims[0] if len(a_dims) == 3 else 0)
        assert "__op$block_scaled_dot" not in hlo
    else:
        assert not case["library"]            # every form the reference expands, this library leaves to the expansion too
        assert not plan["rewritten"] and "block-scaled" in plan["not_rewritten"][0]["reason"]


def test_every_library_mx_case_is_taken():
    taken = [c["name"] for c in CASES if c["library"] and is_mx_fp8(c)]
    assert taken == ["CudnnScaledDotSimple", "CudnnScaledDotTransforms", "CudnnScaledDotPaddedScales", "Mxfp8",
                     "Mxfp8_MixedTypes", "Mxfp8_PaddedScales"]


def test_padded_scales_are_sliced_like_the_reference():
    """CudnnScaledDotPaddedScales: operands [4,120,96], scales [4,128,4] with block_size 32 in the backend config.
    The reference slices the scales to [4,120,3] before dequantizing (block_scaling_rewriter.cc:469-518); the
    interpreter must give what the oracle gives on the sliced arrays, whatever the padding holds."""
    case = BY_NAME["CudnnScaledDotPaddedScales"]
    a, b, sa, sb = ref_cases.make_inputs(case["hlo"], 5)
    assert sa.shape == (4, 128, 4) and a.shape == (4, 120, 96)
    sa[:, 120:, :] = 0xFF            # NaN codes in the padding
    sa[:, :, 3:] = 0xFF
    sb[:, 120:, :] = 0xFF
    sb[:, :, 3:] = 0xFF
    got = hlo_eval.evaluate(case["hlo"], [a, b, sa, sb])
    want = o.block_scaled_dot(a, b, sa[:, :120, :3], sb[:, :120, :3], out_dtype=o.F16)
    assert got.shape == (4, 120, 120) and np.array_equal(got, want)
    assert np.isfinite(np.asarray(got).view(np.float16)).all()
    with pytest.raises(ValueError):           # scales that do not cover the rows
        o.block_scaled_dot(a, b, sa[:, :100], sb)
    with pytest.raises(ValueError):           # explicit block size, too few scale columns
        o.block_scaled_dot(a, b, sa[:, :, :2], sb, block_size=32)


def test_padded_scales_need_the_explicit_block_size():
    """Without block_size in the backend config the block size is implied by the shapes (block_scaling_rewriter.cc:98-113),
    so [.., 4] scale columns over k = 96 is not block size 32 and the call is not taken."""
    case = BY_NAME["CudnnScaledDotPaddedScales"]
    text = re.sub(r",\s*backend_config=\{.*\}\}", "", case["hlo"])
    assert "block_size" not in text
    _, plan = hlo_runner.rewrite(text)
    assert not plan["rewritten"] and "block size" in plan["not_rewritten"][0]["reason"]
    _, plan = hlo_runner.rewrite(case["hlo"].replace("block_size:32", "block_size:16"))
    assert not plan["rewritten"] and "block size" in plan["not_rewritten"][0]["reason"]


@pytest.mark.parametrize("case", SCALED_DOT, ids=[c["name"] for c in SCALED_DOT])
def test_scaled_dot_instruction_becomes_the_mx_call(case):
    """The reference turns a `scaled-dot` into `__cublas$lt$matmul$mx` when a BLAS library wins its autotuning
    (autotuner/hipblaslt.cc:430-505; mx_scaled_dot_execution_test.cc expects that call or a Triton fusion for every
    module listed with `mx_call`).  The rewriter-lite takes the MXFP8 ones in the form that call has."""
    hlo, plan = hlo_runner.rewrite(case["hlo"])
    taken = SCALED_DOT_TAKEN[case["name"]]
    assert plan["rewritten"] == taken
    if case["mx_call"] and "f4e2m1fn" not in case["hlo"]:
        assert taken                       # every FP8 module the reference runs through the MX call is taken
    if case["supported"]:
        assert taken                       # and everything cuDNN's helper accepts
    if taken:
        (c,) = plan["calls"]
        assert c["target"] == "b200$block_scaled_dot$mx" and "scaled-dot(" not in hlo
        assert [x["role"] for x in c["operands"]] == ["a", "b", "a_scale", "b_scale"]
        if case["name"] == "CudnnFusionUnsupportedDimensions":
            assert c["operands"][1]["chain"] == ["transpose"] and c["operands"][3]["chain"] == ["transpose"]
            assert c["operands"][1]["dims"] == [128, 256] and c["operands"][3]["dims"] == [128, 8]
            assert (c["m"], c["n"], c["k"]) == (128, 128, 256)
    else:
        assert "scaled-dot" in plan["not_rewritten"][0]["reason"]


def test_scaled_dot_interpreter_against_the_block_scaled_oracle():
    """`scaled-dot` evaluated term by term as HandleScaledDot does (hlo_evaluator_typed_visitor.h:1783-1990) against the
    oracle's dequantize-then-dot: the same products (exact in f32), summed in a different order."""
    for name, kind_b in (("MxFp8Correctness", "e4m3fn"), ("MxFp8MixedTypesBatchedCorrectness", "e5m2"),
                         ("MxFp8ReshapedOperandsCorrectness", "e4m3fn")):
        case = next(c for c in SCALED_DOT if c["name"] == name)
        a, b, sa, sb = ref_cases.make_inputs(case["hlo"], 9)
        got = hlo_eval.evaluate(case["hlo"], [a, b, sa, sb])
        a2, b2 = a.reshape(sa.shape[:-1] + (-1,)), b.reshape(sb.shape[:-1] + (-1,))
        want = o.block_scaled_dot(a2, b2, sa, sb, b_kind=kind_b)
        absdot = np.matmul(np.abs(o.mx_dequantize(a2, sa)).astype(np.float64),
                           np.swapaxes(np.abs(o.mx_dequantize(b2, sb, kind_b)).astype(np.float64), -1, -2))
        assert got.shape == want.shape
        assert (np.abs(got.astype(np.float64) - want) <= absdot * 2.0 ** -20).all()
    # coarser scales (one per 32 rows x 256 columns, scaled_dot_rewriter_test.cc:57-67) and a scalar scale (= 1)
    text = """HloModule m
ENTRY main {
  lhs = f8e4m3fn[64,512] parameter(0)
  rhs = f8e4m3fn[32,512] parameter(1)
  lhs_scale = f8e8m0fnu[2,2] parameter(2)
  rhs_scale = f8e8m0fnu[] parameter(3)
  ROOT d = f32[64,32] scaled-dot(lhs, rhs, lhs_scale, rhs_scale), lhs_contracting_dims={1}, rhs_contracting_dims={1}
}
"""
    rng = np.random.default_rng(4)
    a = o.fp8_encode(rng.uniform(-1, 1, (64, 512)).astype(np.float32))
    b = o.fp8_encode(rng.uniform(-1, 1, (32, 512)).astype(np.float32))
    sa = np.array([[126, 128], [127, 129]], np.uint8)
    got = hlo_eval.evaluate(text, [a, b, sa, np.uint8(140)])
    scale = np.repeat(np.repeat(o.e8m0_decode(sa), 32, axis=0), 256, axis=1)
    want = (o.fp8_decode(a).astype(np.float64) * scale) @ o.fp8_decode(b).astype(np.float64).T
    np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4)
    _, plan = hlo_runner.rewrite(text)
    assert not plan["rewritten"] and "scalar scale" in plan["not_rewritten"][0]["reason"]
