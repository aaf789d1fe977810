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
from xla_b200.scaled_dot import XlaFfiError

import ref_cases

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "ref_block_scaled.json")) as f:
    CASES = json.load(f)["cases"]
BY_NAME = {c["name"]: c for c in CASES}


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
    if "f4e2m1fn" in case["hlo"]:
        # NVFP4: 4-bit values, not implemented; the module also spells an operand as a nested instruction, which the
        # rewriter-lite's parser refuses.  Either way nothing is rewritten.
        with pytest.raises(XlaFfiError):
            hlo_runner.rewrite(case["hlo"])
        return
    hlo, plan = hlo_runner.rewrite(case["hlo"])
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
