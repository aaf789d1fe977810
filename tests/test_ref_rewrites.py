"""The rewriter-lite against the reference's own expectations (host only).

tests/golden/ref_rewrites.json holds every module of xla/backends/gpu/transforms/gemm_rewriter_fp8_test.cc and
the Int8Gemm* modules of gemm_rewriter_test.cc together with what their FileCheck lines expect of the
rewrite (extracted as text by tests/golden/make_ref_rewrites.py).  For every case this file checks that
  * the module is rewritten exactly when the reference rewrites it,
  * every operand of the custom call comes from the same parameter / constant, through the same ops
    (modulo `transpose` / `bitcast`: the reference's expectations are for a Hopper target, which
    transposes B; on Blackwell no transposes are inserted, gemm_rewriter.cc:1535-1554),
  * the result tuple has the same element types (and dims where stated), and
  * alpha, beta, epilogue and damax_output agree.
The interpreter used for expected values elsewhere (oracle/hlo_eval.py) must also evaluate every one of
these modules.
"""
import numpy as np
import pytest

import ref_cases as rc
from oracle import hlo_eval
from xla_b200 import hlo_runner

FP8, INT8 = rc.load()
LAYOUT_ONLY = {"transpose", "bitcast", "copy", "reshape"}
# ops both sides walk through, by their first operand, when naming where an operand comes from
WALKED = LAYOUT_ONLY | {"pad", "broadcast", "slice", "dynamic-slice", "convert", "divide"}
TYPE_NAME = {1: "pred", 2: "s8", 4: "s32", 10: "f16", 11: "f32", 16: "bf16", 19: "f8e5m2", 20: "f8e4m3fn"}


def _ids(cases):
    return [c["name"] for c in cases]


def _filtered(chain):
    return sorted(op for op in chain if op not in LAYOUT_ONLY)


@pytest.mark.parametrize("case", FP8 + INT8, ids=_ids(FP8 + INT8))
def test_rewrite_matches_the_reference_expectation(case):
    if not rc.applies_to_blackwell(case):
        pytest.skip("the reference skips this test on a Blackwell CUDA GPU: " + "; ".join(case["skip_notes"]) + case["test"])
    hlo, plan = hlo_runner.rewrite(case["hlo"])
    exp = case["expect"]
    if exp is None:
        # numeric-only test (RunAndCompare): every such module contains an FP8 / s8 dot this library must take
        assert plan["rewritten"], plan
        return
    assert plan["rewritten"] == exp["rewritten"], plan.get("reason")
    if not exp["rewritten"]:
        return
    assert len(plan["calls"]) == 1
    is_f8 = exp["target"].endswith("$f8")
    assert plan["target"] == ("b200$scaled_dot$f8" if is_f8 else "b200$dot$s8")
    cfg = exp["backend_config"]
    if is_f8:
        if "epilogue" in cfg:
            assert plan["attrs"]["epilogue"] == rc.EPILOGUE_NUMBER[cfg["epilogue"]]
        if "beta" in cfg:
            assert plan["attrs"]["beta"] == cfg["beta"]
        if "alpha_real" in cfg:
            assert plan["attrs"]["alpha_real"] == cfg["alpha_real"]
        if "damax_output" in cfg:
            assert plan["attrs"]["damax_output"] == cfg["damax_output"]
        if "lhs_batch_dimensions" in cfg:
            assert bool(cfg["lhs_batch_dimensions"]) == (plan["batch"] > 0)
    ops = exp.get("operands")
    if ops and not plan["swapped"]:
        # a CHECK line may stop in the middle of the operand list: the operands it names must be the first ones
        full_list = "unknown" not in ops[0]["root"]
        assert len(plan["operands"]) == len(ops) if full_list else len(plan["operands"]) >= len(ops), (plan["operands"], ops)
        for mine, theirs in zip(plan["operands"], ops):
            root = theirs["root"]
            if not set(theirs["chain"]) <= WALKED:
                # e.g. select (the CHECK line's first operand is the predicate) or arithmetic on a scale
                assert set(theirs["chain"]) - WALKED <= set(mine["chain"]) | {mine["source_opcode"]}, (mine, theirs)
            elif "parameter" in root:
                assert mine["param"] == root["parameter"], (mine, theirs)
                assert _filtered(mine["chain"]) == _filtered(theirs["chain"]), (mine, theirs)
                assert mine["reciprocal"] == ("divide" in theirs["chain"])
            elif "constant" in root and not theirs["chain"]:
                assert mine["param"] == -1 and mine["constant"] == float(root["constant"]), (mine, theirs)
    res = exp.get("result")
    if res:
        mine = [TYPE_NAME[r["dtype"]] for r in plan["results"]]
        assert mine == res["element_types"], (mine, res)
        if res["dims"] and not plan["swapped"]:
            assert plan["results"][0]["dims"] == res["dims"]


def test_summary_of_the_reference_cases():
    """How many of the reference's cases are rewritten, and why the others are not -- printed with `pytest -s`."""
    rewritten, refused, skipped = 0, [], 0
    for case in FP8 + INT8:
        if not rc.applies_to_blackwell(case):
            skipped += 1
            continue
        _, plan = hlo_runner.rewrite(case["hlo"])
        if plan["rewritten"]:
            rewritten += 1
        else:
            refused.append((case["name"], plan["reason"]))
    print(f"\n{rewritten} reference modules rewritten, {len(refused)} left alone, {skipped} not applicable on Blackwell")
    for name, why in refused:
        print(f"  {name}: {why}")
    want_refused = {c["name"] for c in FP8 + INT8 if rc.applies_to_blackwell(c) and c["expect"] and not c["expect"]["rewritten"]}
    assert {n for n, _ in refused} == want_refused
    assert rewritten >= 105


@pytest.mark.parametrize("case", [c for c in FP8 + INT8 if rc.applies_to_blackwell(c)], ids=_ids([c for c in FP8 + INT8 if rc.applies_to_blackwell(c)]))
def test_interpreter_evaluates_every_reference_module(case):
    out = hlo_eval.evaluate(case["hlo"], rc.make_inputs(case["hlo"], seed=7))
    outs = out if isinstance(out, tuple) else (out,)
    types = hlo_eval.root_types(case["hlo"]) or ["f32"] * len(outs)
    for t, v in zip(types, outs):
        assert np.isfinite(rc.to_f32(t, v)).all()
