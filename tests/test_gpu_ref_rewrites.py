"""The reference's own GemmRewriter test modules, end to end on the GPU.

Every module of tests/golden/ref_rewrites.json (extracted from gemm_rewriter_fp8_test.cc and the Int8Gemm*
tests of gemm_rewriter_test.cc) that carries a numeric check in the reference (RunAndCompare /
CheckFp8IfSupported against the HLO interpreter) is rewritten, executed through the custom calls, and
compared with the CPU interpreter (oracle/hlo_eval.py) on seeded inputs under the ErrorSpec the reference's
test itself states (1e-2 / 1e-2 by default; 0.1 / 0.1, 2e-3, 1e-3 / 1e-4, 1e-5 where the test says so).
The comparison rule is the reference's: an element is a mismatch when it is outside the absolute AND the
relative bound (xla/literal_comparison.cc:456-556).  Where the module's result is FP8, an element one
representable value away also passes (an FP8 step is up to 12.5 %, wider than most of the bounds).
"""
import numpy as np
import pytest
import torch

import ref_cases as rc
from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import device_status, hlo_runner

pytestmark = pytest.mark.gpu
FP8, INT8 = rc.load()
CASES = [c for c in FP8 + INT8 if rc.applies_to_blackwell(c) and (c["expect"] is None or c["expect"]["rewritten"])]
_TORCH = {"f8e4m3fn": torch.float8_e4m3fn, "f8e5m2": torch.float8_e5m2, "bf16": torch.bfloat16, "f16": torch.float16}


def to_dev(v, t, dev):
    x = torch.from_numpy(np.ascontiguousarray(v)).to(dev)
    if t in ("f8e4m3fn", "f8e5m2"):
        return x.view(_TORCH[t])
    if t in ("bf16", "f16"):
        return x.view(torch.int16).view(_TORCH[t])
    return x


def to_f32(t):
    return t.float().cpu().numpy() if t.dtype != torch.bool else t.cpu().numpy().astype(np.float32)


@pytest.mark.parametrize("case", CASES, ids=[c["name"] for c in CASES])
def test_reference_module_runs_through_the_custom_calls(cuda_device, case):
    hlo = case["hlo"]
    inputs = rc.make_inputs(hlo, seed=11)
    exp = hlo_eval.evaluate(hlo, inputs)
    params = [to_dev(v, t, cuda_device) for v, (_, t, _) in zip(inputs, rc.parameters(hlo))]
    got, stats = hlo_runner.run_hlo_module(hlo, params, return_stats=True)
    torch.cuda.synchronize()
    assert stats["custom_calls"] >= 1
    exps = exp if isinstance(exp, tuple) else (exp,)
    gots = got if isinstance(got, tuple) else (got,)
    types = hlo_eval.root_types(hlo) or ["f32"] * len(exps)
    abs_tol, rel_tol = case["error_spec"]
    for t, e, g in zip(types, exps, gots):
        e32, g32 = rc.to_f32(t, e), to_f32(g).reshape(np.shape(e))
        if t == "s32":
            assert np.array_equal(np.asarray(e), g.cpu().numpy().reshape(np.shape(e)))      # integer path: bit-exact
            continue
        bad = (np.abs(e32 - g32) > abs_tol) & (np.abs(e32 - g32) > rel_tol * np.abs(e32))
        bad |= np.isnan(e32) != np.isnan(g32)
        if t in ("f8e4m3fn", "f8e5m2"):
            codes = g.view(torch.uint8).cpu().numpy().reshape(np.shape(e))
            bad &= np.abs(o.fp8_ordinal(np.asarray(e)).astype(np.int64) - o.fp8_ordinal(codes).astype(np.int64)) > 1
        assert int(bad.sum()) == 0, f"{int(bad.sum())} of {bad.size} elements outside ErrorSpec{{{abs_tol}, {rel_tol}}}"
    assert device_status() == 0
