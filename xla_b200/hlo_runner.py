"""Runs a fixture HLO module on the GPU the way XLA would after its GemmRewriter pass.

The module text goes through `b200sd_rewrite_hlo` (the rewriter-lite in csrc/hlo_rewriter.cc, which
restates xla/backends/gpu/transforms/gemm_rewriter.cc for this path); the resulting custom call is
then executed through the FFI boundary exactly like any other call site.  The only work done
outside the custom call is what the rewritten module itself still contains: the reciprocal of a
scale the original HLO divided by, and scalar constants.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Sequence

from . import _native
from .scaled_dot import FfiCall, XlaFfiError

_TORCH_DTYPE = {}


def _torch_dtype(code: int):
    import torch

    if not _TORCH_DTYPE:
        _TORCH_DTYPE.update({2: torch.int8, 4: torch.int32, 10: torch.float16, 11: torch.float32, 16: torch.bfloat16,
                             19: torch.float8_e5m2, 20: torch.float8_e4m3fn})
    return _TORCH_DTYPE[code]


def rewrite(hlo_text: str):
    """Returns (rewritten module text, plan dict)."""
    out = C.create_string_buffer(max(1 << 16, 4 * len(hlo_text)))
    plan = C.create_string_buffer(1 << 15)
    err = C.create_string_buffer(1024)
    rc = _native.product.b200sd_rewrite_hlo(hlo_text.encode(), out, len(out), plan, len(plan), err, len(err))
    if rc != 0:
        raise XlaFfiError(rc, err.value.decode(errors="replace"))
    return out.value.decode(), json.loads(plan.value.decode())


def run_hlo_module(hlo_text: str, params: Sequence, stream=None):
    """Rewrites `hlo_text` and executes the custom call on `params` (torch CUDA tensors in parameter
    order).  Returns the module's outputs in the order of its ROOT (a tensor, or a tuple)."""
    import torch

    _, plan = rewrite(hlo_text)
    if not plan["rewritten"]:
        raise XlaFfiError(12, "module was not rewritten onto a custom call: " + plan["reason"])
    dev = params[0].device
    operands = []
    for src in plan["operands"]:
        if src["param"] < 0:
            operands.append(torch.full((), float(src["constant"]), dtype=torch.float32, device=dev))
        elif src["reciprocal"]:
            operands.append((1.0 / params[src["param"]].float()).reshape(()))
        else:
            operands.append(params[src["param"]])
        if src.get("reshaped"):
            # a bitcast between the dequantisation and the dot: the same row-major bytes in the shape the dot saw
            if not operands[-1].is_contiguous():
                raise ValueError(f"parameter {src['param']} is viewed in another shape and must be contiguous")
            operands[-1] = operands[-1].reshape(tuple(src["dims"]))
        if src.get("transposed"):
            # a column-major parameter: the same bytes are the row-major matrix with the dimensions swapped
            phys = operands[-1].t()
            if not phys.is_contiguous():
                raise ValueError(f"parameter {src['param']} is declared column-major; pass a tensor whose .t() is contiguous")
            operands[-1] = phys
        if src.get("padded_dims", src["dims"]) != src["dims"]:
            # the `pad` instructions of the rewritten module: zero-fill up to multiples of 16
            t = operands[-1]
            full = torch.zeros(tuple(src["padded_dims"]), dtype=torch.uint8 if t.element_size() == 1 else t.dtype, device=dev)
            view = t.view(torch.uint8) if t.element_size() == 1 else t
            full[tuple(slice(0, d) for d in src["dims"])] = view
            operands[-1] = full.view(t.dtype) if t.element_size() == 1 else full
    results, outputs = [], {}
    for res in plan["results"]:
        alloc = res.get("padded_dims", res["dims"])
        t = torch.empty(tuple(alloc), dtype=_torch_dtype(res["dtype"]), device=dev)
        results.append(t)
        if res["root_index"] >= -1:
            # the `slice` instruction of the rewritten module
            out = t[tuple(slice(0, d) for d in res["dims"])] if alloc != res["dims"] else t
            if res.get("transposed"):
                out = out.t()                                   # a column-major result: D^T was computed
            if res.get("view_dims"):
                out = out.reshape(tuple(res["view_dims"]))      # the bitcast behind the dot
            outputs[res["root_index"]] = out
    attrs = dict(plan["attrs"])
    for key in ("alpha_real", "beta"):                       # f64 attributes, whatever the JSON reader made of them
        attrs[key] = float(attrs[key])
    call = FfiCall(plan["target"], operands, results, attrs)
    s = stream if stream is not None else torch.cuda.current_stream(dev).cuda_stream
    call.run(s, dev.index or 0)
    call.close()
    if -1 in outputs:
        return outputs[-1]
    return tuple(outputs[i] for i in sorted(outputs))
