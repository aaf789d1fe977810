"""The reference's own MX block-scaled test modules (tests/golden/ref_block_scaled.json), rewritten onto
b200$block_scaled_dot$mx and run through the FFI boundary, against the interpreter's evaluation of the same text
-- which is the reference's expansion (tests/test_mx_hlo.py, tests/test_ref_block_scaled.py).

This is the comparison block_scaling_rewriter_cudnn_test.cc makes (library kernel against the expanded module under
ErrorSpec{1e-4, 1e-5}); every element must also satisfy the summation-order bound of tests/test_gpu_mx.py."""
import numpy as np
import pytest
import torch

from oracle import hlo_eval
from oracle import scaled_dot_oracle as o
from xla_b200 import hlo_runner

import ref_cases
from test_ref_block_scaled import CASES, SCALED_DOT, SCALED_DOT_TAKEN, is_mx_fp8

pytestmark = pytest.mark.gpu
MX_CASES = [c for c in CASES if c["library"] and is_mx_fp8(c)]
_TORCH = {"f8e4m3fn": torch.float8_e4m3fn, "f8e5m2": torch.float8_e5m2, "f8e8m0fnu": torch.float8_e8m0fnu}


SD_CASES = [c for c in SCALED_DOT if SCALED_DOT_TAKEN[c["name"]]]


@pytest.mark.parametrize("case", MX_CASES + SD_CASES, ids=[c["name"] for c in MX_CASES + SD_CASES])
def test_reference_mx_module(cuda_device, case):
    """`__op$block_scaled_dot` modules and `scaled-dot` modules (the latter as mx_scaled_dot_execution_test.cc runs
    them: the MX call against the expansion under ErrorSpec{1e-4, 1e-5})."""
    text = case["hlo"]
    params = ref_cases.parameters(text)
    rng = np.random.default_rng(11)
    args = ref_cases.make_inputs(text, 11)
    for i, (_, t, dims) in enumerate(params):
        if t == "f8e8m0fnu":          # block scales 2^-3 .. 1: results of order one, where the reference's absolute bound means something
            args[i] = rng.integers(124, 128, size=dims, dtype=np.uint8)
    exp = hlo_eval.evaluate(text, args)
    dev_args = [torch.from_numpy(np.ascontiguousarray(v)).to(cuda_device).view(_TORCH[t]) for v, (_, t, _) in zip(args, params)]
    got, stats = hlo_runner.run_hlo_module(text, dev_args, return_stats=True)
    torch.cuda.synchronize()
    assert stats["custom_calls"] == 1
    out_type = hlo_eval.root_types(text)[0]
    if out_type == "f16":
        got_f = got.view(torch.int16).cpu().numpy().view(np.float16).astype(np.float32)
        exp_f = np.asarray(exp).view(np.float16).astype(np.float32)
        step = 2.0 ** -10
    else:
        got_f, exp_f, step = got.cpu().numpy(), np.asarray(exp, np.float32), 2.0 ** -23
    assert got_f.shape == exp_f.shape
    # sum_k |a_k b_k| from the operands as the call sees them (scales sliced to the corner in use)
    a, b, sa, sb = args[:4]
    if a.ndim == 1:                  # CudnnFusionUnsupportedInputs: lhs is a vector broadcast along k inside the module
        a = np.repeat(a[:, None], sa.shape[-1] * 32, axis=1)
    if "rhs_contracting_dims={0}" in text:          # CudnnFusionUnsupportedDimensions: rhs and its scales are [k, n]
        b, sb = np.ascontiguousarray(b.T), np.ascontiguousarray(sb.T)
    if a.ndim > sa.ndim:             # MxFp8ReshapedOperands: [.., k / 32, 32] parameters, flattened inside the module
        a, b = a.reshape(a.shape[: sa.ndim - 1] + (-1,)), b.reshape(b.shape[: sb.ndim - 1] + (-1,))
    kinds = ["e4m3fn" if t == "f8e4m3fn" else "e5m2" for _, t, _ in params[:2]]
    # (Mxfp8_PaddedScales pads inside the module: its parameters are already the corner.)
    sa, sb = sa[..., : a.shape[-2], : a.shape[-1] // 32], sb[..., : b.shape[-2], : b.shape[-1] // 32]
    absdot = np.matmul(np.abs(o.mx_dequantize(a, sa, kinds[0])).astype(np.float64),
                       np.swapaxes(np.abs(o.mx_dequantize(b, sb, kinds[1])).astype(np.float64), -1, -2))
    err = np.abs(got_f.astype(np.float64) - exp_f)
    assert (err <= absdot * 2.0 ** -16 + np.abs(exp_f) * step + 1e-30).all(), float((err / (absdot + 1e-30)).max())
    if case["error_spec"] and out_type == "f32":
        assert o.near_mismatches(exp_f, got_f, *case["error_spec"])[0] == 0
