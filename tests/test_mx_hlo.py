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


def _mx_module(m, n, k, batch, a_rows, a_cols, b_rows, b_cols, out="f32", block_size=None):
    lead = f"{batch}," if batch else ""
    cfg = f', backend_config={{"block_scaled_dot_backend_config":{{block_size:{block_size}}}}}' if block_size else ""
    return f"""HloModule generated
ENTRY main {{
  lhs = f8e4m3fn[{lead}{m},{k}] parameter(0)
  rhs = f8e5m2[{lead}{n},{k}] parameter(1)
  lhs_scale = f8e8m0fnu[{lead}{a_rows},{a_cols}] parameter(2)
  rhs_scale = f8e8m0fnu[{lead}{b_rows},{b_cols}] parameter(3)
  ROOT result = {out}[{lead}{m},{n}] custom-call(lhs, rhs, lhs_scale, rhs_scale), custom_call_target="__op$block_scaled_dot"{cfg}
}}
"""


def test_generated_mx_modules_padding_and_block_size():
    """Shapes drawn at random: the call is taken exactly when the scales cover [rows, k / 32] -- extra rows always,
    extra columns only with the explicit block size (block_scaling_rewriter.cc:469-518) -- and the interpreter's
    result does not depend on what the padding holds."""
    rng = np.random.default_rng(2024)
    for trial in range(40):
        m, n = int(rng.integers(1, 70)), int(rng.integers(1, 70))
        k = 32 * int(rng.integers(1, 6))
        batch = int(rng.integers(0, 3))
        pad_rows_a, pad_rows_b = int(rng.integers(0, 9)) * int(rng.integers(0, 2)), int(rng.integers(0, 9)) * int(rng.integers(0, 2))
        pad_cols = int(rng.integers(0, 4)) * int(rng.integers(0, 2))
        explicit = bool(rng.integers(0, 2))
        text = _mx_module(m, n, k, batch, m + pad_rows_a, k // 32 + pad_cols, n + pad_rows_b, k // 32 + pad_cols,
                          out=("f32", "bf16", "f16")[trial % 3], block_size=32 if explicit else None)
        _, plan = hlo_runner.rewrite(text)
        want_taken = explicit or pad_cols == 0
        assert plan["rewritten"] == want_taken, text
        if want_taken:
            (c,) = plan["calls"]
            assert (c["m"], c["n"], c["k"], c["batch"]) == (m, n, k, batch)
            assert c["operands"][2]["dims"][-2:] == [m + pad_rows_a, k // 32 + pad_cols]
            assert c["attrs"].get("block_size") == (32 if explicit else None)
        if not explicit and pad_cols:
            continue                      # block size implied by the shapes is not 32: only the generic expansion applies
        args = ref_cases.make_inputs(text, trial)
        a, b, sa, sb = args
        base = hlo_eval.evaluate(text, [a, b, sa, sb])
        sa2, sb2 = sa.copy(), sb.copy()
        sa2[..., m:, :] = 0xFF
        sb2[..., n:, :] = 0xFF
        if explicit:
            sa2[..., k // 32:] = 0xFF
            sb2[..., k // 32:] = 0xFF
        assert np.array_equal(hlo_eval.evaluate(text, [a, b, sa2, sb2]), base), text
        code = {"f32": o.F32, "bf16": o.BF16, "f16": o.F16}[("f32", "bf16", "f16")[trial % 3]]
        assert np.array_equal(base, o.block_scaled_dot(a, b, sa[..., :m, : k // 32], sb[..., :n, : k // 32], b_kind="e5m2", out_dtype=code))
