"""The MX block-scaled dot at the HLO level (CPU): the reference's expansion pins the oracle, and the
rewriter-lite turns `__op$block_scaled_dot` into this library's call exactly when the operands are MX."""
import os

import numpy as np

from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import hlo_runner

import ref_cases

HLO_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "hlo")


def _load(name):
    return open(os.path.join(HLO_DIR, name + ".hlo")).read()


def test_oracle_equals_the_reference_expansion():
    """block_scaled_dot_mx_expanded.hlo is, instruction by instruction, what the reference's test expects
    BlockScalingRewriter to produce (block_scaling_rewriter_test.cc:104-122).  Interpreting it op by op must give
    what the oracle's block_scaled_dot gives for the un-expanded custom call."""
    call, expanded = _load("block_scaled_dot_mx"), _load("block_scaled_dot_mx_expanded")
    assert ref_cases.parameters(call) == [(n, t, d) for n, t, d in ref_cases.parameters(expanded)]
    for seed in (1, 2):
        args = ref_cases.make_inputs(call, seed)
        via_call = hlo_eval.evaluate(call, args)
        via_ops = hlo_eval.evaluate(expanded, args)
        assert via_call.shape == (4, 16, 32) and via_call.dtype == np.float32
        np.testing.assert_allclose(via_call, via_ops, rtol=2e-6, atol=0)
        a, b, sa, sb = args
        np.testing.assert_array_equal(via_call, o.block_scaled_dot(a, b, sa, sb))


def test_rewriter_takes_the_mx_call_as_it_is():
    hlo, plan = hlo_runner.rewrite(_load("block_scaled_dot_mx"))
    assert plan["rewritten"] and len(plan["calls"]) == 1 and not plan["not_rewritten"]
    c = plan["calls"][0]
    assert c["target"] == "b200$block_scaled_dot$mx" and (c["batch"], c["m"], c["n"], c["k"]) == (4, 16, 32, 256)
    assert [x["role"] for x in c["operands"]] == ["a", "b", "a_scale", "b_scale"]           # thunk_emitter.cc:939-988
    assert [x["param"] for x in c["operands"]] == [0, 1, 2, 3] and all(x["chain"] == [] for x in c["operands"])
    assert [x["dtype"] for x in c["operands"]] == [20, 20, 33, 33]
    assert [r["role"] for r in c["results"]] == ["d", "workspace"]
    assert 'custom_call_target="b200$block_scaled_dot$mx"' in hlo and "__op$block_scaled_dot" not in hlo


def test_rewriter_leaves_other_block_scaled_forms_to_the_expansion():
    base = _load("block_scaled_dot_mx")
    cases = {
        "f8e5m2 scales (the reference test's own types)": base.replace("f8e8m0fnu", "f8e5m2"),
        "block size 16": base.replace("f8e8m0fnu[4,16,8]", "f8e8m0fnu[4,16,16]").replace("f8e8m0fnu[4,32,8]", "f8e8m0fnu[4,32,16]"),
        "global scale": base.replace("rhs_scale = f8e8m0fnu[4,32,8] parameter(3)",
                                     "rhs_scale = f8e8m0fnu[4,32,8] parameter(3)\n  g = f32[] parameter(4)")
                            .replace("custom-call(lhs, rhs, lhs_scale, rhs_scale)", "custom-call(lhs, rhs, lhs_scale, rhs_scale, g)"),
    }
    for what, text in cases.items():
        hlo, plan = hlo_runner.rewrite(text)
        assert not plan["rewritten"], what
        assert plan["not_rewritten"] and "block-scaled" in plan["not_rewritten"][0]["reason"], what


def test_a_module_with_an_mx_dot_and_a_scaled_dot_gets_both_calls():
    text = """HloModule two
ENTRY main {
  x = f8e4m3fn[64,256] parameter(0)
  w = f8e4m3fn[128,256] parameter(1)
  xs = f8e8m0fnu[64,8] parameter(2)
  ws = f8e8m0fnu[128,8] parameter(3)
  h = bf16[64,128] custom-call(x, w, xs, ws), custom_call_target="__op$block_scaled_dot"
  y = f8e4m3fn[64,128] parameter(4)
  v = f8e4m3fn[128,32] parameter(5)
  s = f32[] parameter(6)
  yf = f32[64,128] convert(y)
  sb = f32[64,128] broadcast(s), dimensions={}
  yd = f32[64,128] multiply(yf, sb)
  vf = f32[128,32] convert(v)
  d = f32[64,32] dot(yd, vf), lhs_contracting_dims={1}, rhs_contracting_dims={0}
  ROOT t = (bf16[64,128], f32[64,32]) tuple(h, d)
}
"""
    hlo, plan = hlo_runner.rewrite(text)
    assert sorted(c["target"] for c in plan["calls"]) == ["b200$block_scaled_dot$mx", "b200$scaled_dot$f8"]
