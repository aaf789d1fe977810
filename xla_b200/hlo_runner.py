"""Runs an HLO module on the GPU the way XLA would after its GemmRewriter pass.

The module text goes through `b200sd_rewrite_hlo` (the rewriter-lite in csrc/hlo_rewriter.cc, which
restates xla/backends/gpu/transforms/gemm_rewriter.cc for this path).  The rewritten module is then
executed instruction by instruction: every `custom-call` to "b200$scaled_dot$f8" / "b200$dot$s8" / "b200$block_scaled_dot$mx" goes
through the FFI boundary exactly like any other call site, and what is left around the calls -- the
ops XLA would hand to its other emitters: data movement in front of a call (pad, slice, transpose,
broadcast, select ...), the reciprocal or the f32 conversion of a scale, arithmetic the rewriter did
not fold -- runs as plain torch ops on the same stream.  A dot that was NOT rewritten is refused
unless `allow_residual_dots` is set: this library is not a general dot emitter.

Values are torch tensors in their logical shape; the layout an instruction declares matters only
to `bitcast`, which reinterprets the bytes as they lie in memory.
"""
from __future__ import annotations

import ctypes as C
import json
import re
from typing import Sequence

from . import _native
from .scaled_dot import FfiCall, XlaFfiError

_TARGETS = ("b200$scaled_dot$f8", "b200$dot$s8", "b200$block_scaled_dot$mx")


def rewrite(hlo_text: str):
    """Returns (rewritten module text, plan dict)."""
    out = C.create_string_buffer(max(1 << 16, 6 * len(hlo_text)))
    plan = C.create_string_buffer(1 << 17)
    err = C.create_string_buffer(1024)
    rc = _native.product.b200sd_rewrite_hlo(hlo_text.encode(), out, len(out), plan, len(plan), err, len(err))
    if rc != 0:
        raise XlaFfiError(rc, err.value.decode(errors="replace"))
    return out.value.decode(), json.loads(plan.value.decode())


# ------------------------------------------------------------------------------------------- text
def _split_top(s: str):
    out, cur, depth = [], "", 0
    for ch in s:
        depth += ch in "([{"
        depth -= ch in ")]}"
        if ch == "," and depth == 0:
            out.append(cur.strip())
            cur = ""
        else:
            cur += ch
    if cur.strip():
        out.append(cur.strip())
    return out


def _parse_shape(text: str):
    """"f32[2,3]{0,1}" -> ("f32", (2, 3), (0, 1)); "(a, b)" -> ("tuple", [shapes])."""
    text = text.strip()
    if text.startswith("("):
        return ("tuple", [_parse_shape(p) for p in _split_top(text[1:-1])], None)
    m = re.match(r"([a-z0-9]+)\[([0-9, ]*)\](?:\{([0-9, ]*)[^}]*\})?", text)
    dims = tuple(int(x) for x in m.group(2).split(",") if x.strip())
    layout = tuple(int(x) for x in m.group(3).split(",") if x.strip()) if m.group(3) else None
    if layout is not None and len(layout) != len(dims):
        layout = None
    return (m.group(1), dims, layout)


def parse_module(text: str):
    """{computation name: [instruction dicts]}, name of the entry computation."""
    lines = []
    for raw in text.splitlines():
        t = raw.split("//")[0].strip()
        if not t:
            continue
        eq, paren = t.find(" = "), t.find("(")
        starts = eq >= 0 and (paren < 0 or eq < paren)
        if t.startswith("HloModule") or t == "}" or starts or (t.endswith("{") and not starts) or not lines:
            lines.append(t)
        else:
            lines[-1] += " " + t
    comps, cur, entry, last = {}, None, None, None
    for t in lines:
        if t.startswith("HloModule"):
            continue
        if cur is None:
            head = t[:-1].strip()
            is_entry = head.startswith("ENTRY ")
            name = re.split(r"[ (]", head[6:].strip() if is_entry else head)[0].lstrip("%")
            cur = comps.setdefault(name, [])
            last = name
            if is_entry:
                entry = name
            continue
        if t == "}":
            cur = None
            continue
        closes = t.endswith("}") and t.count("{") < t.count("}")
        if closes:
            t = t[:-1].strip()
        root = t.startswith("ROOT ")
        if root:
            t = t[5:].strip()
        name, rest = t.split(" = ", 1)
        m = re.match(r"(\(.*?\)\s|[a-z0-9]+\[[0-9, ]*\](?:\{[^}]*\})?\s)?\s*([a-z\-]+)\((.*)$", rest)
        shape_text, opcode, tail = m.group(1), m.group(2), m.group(3)
        depth, i = 1, 0
        while depth:
            depth += {"(": 1, ")": -1}.get(tail[i], 0)
            i += 1
        args, attrs = tail[: i - 1], tail[i:].lstrip(", ")
        operands = [] if opcode in ("constant", "parameter") else [a.split(" ")[-1].lstrip("%") for a in _split_top(args)]
        cur.append(dict(name=name.strip().lstrip("%"), shape=_parse_shape(shape_text) if shape_text else None, opcode=opcode,
                        operands=operands, literal=args.strip(), attrs=attrs, root=root))
        if closes:
            cur = None
    return comps, entry or last


def _int_list(attrs: str, key: str):
    m = re.search(key + r"=\{([0-9, ]*)\}", attrs)
    return tuple(int(x) for x in m.group(1).split(",") if x.strip()) if m else None


def _backend_config(attrs: str) -> dict:
    m = re.search(r"backend_config=\{(.*)\}", attrs)
    out = {}
    for item in _split_top(m.group(1)):
        key, value = (s.strip() for s in item.split("=", 1))
        arr = re.match(r"array<i64:\s*([0-9, -]*)>", value)
        if arr:
            out[key] = [int(x) for x in arr.group(1).split(",") if x.strip()]
        elif value in ("true", "false"):
            out[key] = value == "true"
        else:
            v, _, kind = (s.strip() for s in value.partition(":"))
            out[key] = (kind, float(v) if kind.startswith("f") else int(v)) if kind else (float(v) if "." in v else int(v))
    return out


# ------------------------------------------------------------------------------------------- values
def _torch():
    import torch

    return torch


def _dtype(name: str):
    torch = _torch()
    table = {"pred": torch.bool, "s8": torch.int8, "s32": torch.int32, "s64": torch.int64, "u8": torch.uint8, "f16": torch.float16,
             "f32": torch.float32, "bf16": torch.bfloat16, "f8e5m2": torch.float8_e5m2, "f8e4m3fn": torch.float8_e4m3fn}
    if hasattr(torch, "float8_e8m0fnu"):
        table["f8e8m0fnu"] = torch.float8_e8m0fnu
    return table[name]


def _is_f8(t) -> bool:
    torch = _torch()
    return t.dtype in (torch.float8_e5m2, torch.float8_e4m3fn) or t.dtype == getattr(torch, "float8_e8m0fnu", None)


def _moved(t, fn):
    """Applies a data-movement function; FP8 tensors go through their bytes (torch moves bytes of any type)."""
    torch = _torch()
    if _is_f8(t):
        return fn(t.view(torch.uint8)).view(t.dtype)
    return fn(t)


def _physical_order(dims, layout):
    return tuple(reversed(layout)) if layout is not None else tuple(range(len(dims)))


def _bitcast(t, src_shape, dst_shape):
    """The bytes of `t` as they lie in memory under src_shape's layout, read under dst_shape's."""
    _, sdims, slayout = src_shape
    _, ddims, dlayout = dst_shape
    sp, dp = _physical_order(sdims, slayout), _physical_order(ddims, dlayout)

    def move(x):
        flat = x.permute(sp).contiguous().reshape(-1)
        phys = flat.reshape(tuple(ddims[d] for d in dp))
        inverse = [dp.index(i) for i in range(len(dp))]
        return phys.permute(inverse).contiguous()

    return _moved(t, move)


class _Evaluator:
    def __init__(self, comps, entry, params, stream, allow_residual_dots):
        self.comps, self.entry, self.params = comps, entry, params
        self.stream, self.allow_residual_dots = stream, allow_residual_dots
        self.torch = _torch()
        self.dev = params[0].device
        self.calls = 0

    def run(self):
        env, shapes, result = {}, {}, None
        for ins in self.comps[self.entry]:
            shape = ins["shape"] or shapes[ins["operands"][0]]
            val = self.eval(ins, shape, [env[o] for o in ins["operands"]], [shapes[o] for o in ins["operands"]])
            env[ins["name"]], shapes[ins["name"]] = val, shape
            if ins["root"]:
                result = val
        return result if result is not None else env[self.comps[self.entry][-1]["name"]]

    def eval(self, ins, shape, a, a_shapes):
        torch, op, attrs = self.torch, ins["opcode"], ins["attrs"]
        t, dims = (shape[0], shape[1]) if shape[0] != "tuple" else ("tuple", None)
        if op == "parameter":
            p = self.params[int(ins["literal"])]
            return p.reshape(dims) if tuple(p.shape) != tuple(dims) else p
        if op == "constant":
            lit = ins["literal"]
            v = {"inf": float("inf"), "-inf": float("-inf"), "nan": float("nan"), "true": 1.0, "false": 0.0}.get(lit)
            v = float(lit) if v is None else v
            base = torch.full(dims, v, dtype=torch.float32, device=self.dev)
            return base.to(_dtype(t))
        if op == "convert":
            x = a[0]
            if _is_f8(x):
                x = x.to(torch.float32)
            return x.to(_dtype(t))
        if op in ("copy", "optimization-barrier"):
            return a[0]
        if op == "reshape":
            return _moved(a[0], lambda x: x.reshape(dims))
        if op == "bitcast":
            return _bitcast(a[0], a_shapes[0], shape)
        if op == "transpose":
            perm = _int_list(attrs, "dimensions")
            return _moved(a[0], lambda x: x.permute(perm).contiguous())
        if op == "broadcast":
            bd = _int_list(attrs, "dimensions") or ()
            view = [1] * len(dims)
            for i, d in enumerate(bd):
                view[d] = dims[d]
            return _moved(a[0], lambda x: x.reshape(view).expand(dims).contiguous())
        if op == "slice":
            spec = re.search(r"slice=\{(.*?)\}", attrs).group(1)
            idx = []
            for part in re.findall(r"\[([0-9:]+)\]", spec):
                nums = [int(x) for x in part.split(":")]
                idx.append(slice(nums[0], nums[1], nums[2] if len(nums) > 2 else 1))
            return _moved(a[0], lambda x: x[tuple(idx)].contiguous())
        if op == "dynamic-slice":
            sizes = _int_list(attrs, "dynamic_slice_sizes")
            starts = [int(s.item()) for s in a[1:]]
            src = a[0].shape
            starts = [min(max(s, 0), src[i] - sizes[i]) for i, s in enumerate(starts)]        # clamped, as XLA does
            idx = tuple(slice(s, s + n) for s, n in zip(starts, sizes))
            return _moved(a[0], lambda x: x[idx].contiguous())
        if op == "pad":
            cfg = re.search(r"padding=([0-9_x\-]+)", attrs).group(1)
            lo_hi = [tuple(int(v) for v in part.split("_")) for part in cfg.split("x")]
            if any(len(p) > 2 and p[2] != 0 for p in lo_hi):
                raise XlaFfiError(12, "interior padding is not handled by the runner")
            x, pv = a[0], a[1]

            def move(xx, pp):
                out = pp.reshape([1] * xx.dim()).expand([lo + n + hi for n, (lo, hi, *_) in zip(xx.shape, lo_hi)]).clone()
                out[tuple(slice(lo, lo + n) for n, (lo, hi, *_) in zip(xx.shape, lo_hi))] = xx
                return out

            if _is_f8(x):
                return move(x.view(torch.uint8), pv.view(torch.uint8)).view(x.dtype)
            return move(x, pv)
        if op == "concatenate":
            d = _int_list(attrs, "dimensions")[0]
            if _is_f8(a[0]):
                return torch.cat([x.view(torch.uint8) for x in a], dim=d).view(a[0].dtype)
            return torch.cat(list(a), dim=d)
        if op == "select":
            if _is_f8(a[1]):
                return torch.where(a[0], a[1].view(torch.uint8), a[2].view(torch.uint8)).view(a[1].dtype)
            return torch.where(a[0], a[1], a[2])
        if op == "compare":
            direction = re.search(r"direction=([A-Z]+)", attrs).group(1)
            fn = {"EQ": torch.eq, "NE": torch.ne, "LT": torch.lt, "LE": torch.le, "GT": torch.gt, "GE": torch.ge}[direction]
            return fn(a[0], a[1])
        if op in ("add", "subtract", "multiply", "divide", "maximum", "minimum", "tanh", "abs", "negate", "exponential", "sqrt",
                  "rsqrt", "logistic", "clamp"):
            # Floating-point element-wise ops are computed in f32 and rounded once to the instruction's type
            # (FP8 tensors have no arithmetic of their own in torch); integers stay integers.
            floating = a[0].dtype.is_floating_point
            v = [x.float() for x in a] if floating else list(a)
            if op in ("maximum", "minimum"):                   # NaN propagates, as XLA's maximum / minimum do
                r = (torch.maximum if op == "maximum" else torch.minimum)(v[0], v[1])
            elif op == "clamp":
                r = torch.minimum(torch.maximum(v[1], v[0]), v[2])      # NaN in x stays NaN
            elif len(v) == 2:
                r = {"add": torch.add, "subtract": torch.sub, "multiply": torch.mul, "divide": torch.div}[op](v[0], v[1])
            else:
                r = {"tanh": torch.tanh, "abs": torch.abs, "negate": torch.neg, "exponential": torch.exp, "sqrt": torch.sqrt,
                     "rsqrt": torch.rsqrt, "logistic": torch.sigmoid}[op](v[0])
            return r.to(_dtype(t)) if floating else r
        if op == "reduce":
            body = self.comps[re.search(r"to_apply=%?([A-Za-z0-9_.\-]+)", attrs).group(1)]
            kind = next(i["opcode"] for i in body if i["root"] or i is body[-1])
            rd = _int_list(attrs, "dimensions")
            x, init = a[0], a[1]
            if kind == "maximum":
                r = torch.amax(x.float(), dim=rd) if rd else x.float()
                r = torch.where(torch.isnan(x.float()).any() if not rd else torch.isnan(x.float()).any(dim=rd).reshape(r.shape),
                                torch.full_like(r, float("nan")), torch.maximum(r, init.float()))
            elif kind == "add":
                r = (torch.sum(x.float(), dim=rd) if rd else x.float()) + init.float()
            else:
                raise XlaFfiError(12, f"reduce with {kind} is not handled by the runner")
            return r.to(_dtype(t)).reshape(dims)
        if op == "tuple":
            return tuple(a)
        if op == "get-tuple-element":
            return a[0][int(re.search(r"index=(\d+)", attrs).group(1))]
        if op == "custom-call":
            return self.custom_call(ins, shape, a)
        if op == "dot":
            if not self.allow_residual_dots:
                raise XlaFfiError(12, f"dot {ins['name']} was not rewritten onto a custom call and this library emits no other dots")
            return self.residual_dot(ins, shape, a)
        raise XlaFfiError(12, f"opcode {op} is not handled by the runner")

    def custom_call(self, ins, shape, operands):
        torch = self.torch
        target = re.search(r'custom_call_target="([^"]+)"', ins["attrs"]).group(1)
        if target not in _TARGETS:
            raise XlaFfiError(12, f"custom call target {target} is not one of this library's")
        results = [torch.empty(s[1], dtype=_dtype(s[0]), device=self.dev) for s in shape[1]]
        call = FfiCall(target, [o.contiguous() for o in operands], results, _backend_config(ins["attrs"]))
        s = self.stream if self.stream is not None else torch.cuda.current_stream(self.dev).cuda_stream
        call.run(s, self.dev.index or 0)
        call.close()
        self.calls += 1
        return tuple(results)

    def residual_dot(self, ins, shape, a):
        torch = self.torch
        lc, rc = _int_list(ins["attrs"], "lhs_contracting_dims"), _int_list(ins["attrs"], "rhs_contracting_dims")
        lb, rb = _int_list(ins["attrs"], "lhs_batch_dims") or (), _int_list(ins["attrs"], "rhs_batch_dims") or ()
        x, y = a[0].float(), a[1].float()
        letters = "abcdefghijklmnop"
        xs, ys = list(letters[: x.dim()]), list(letters[x.dim(): x.dim() + y.dim()])
        for i, j in zip(lc, rc):
            ys[j] = xs[i]
        for i, j in zip(lb, rb):
            ys[j] = xs[i]
        out = [xs[i] for i in lb] + [c for i, c in enumerate(xs) if i not in lc and i not in lb] + \
              [c for j, c in enumerate(ys) if j not in rc and j not in rb]
        r = torch.einsum(f"{''.join(xs)},{''.join(ys)}->{''.join(out)}", x, y)
        return r.to(_dtype(shape[0]))


def run_hlo_module(hlo_text: str, params: Sequence, stream=None, allow_residual_dots: bool = False, return_stats: bool = False):
    """Rewrites `hlo_text` and executes the rewritten module on `params` (torch CUDA tensors in parameter
    order, logical shapes).  Returns the module's root value: a tensor, or a tuple of tensors."""
    rewritten, plan = rewrite(hlo_text)
    if not plan["rewritten"] and not allow_residual_dots:
        raise XlaFfiError(12, "module was not rewritten onto a custom call: " + plan["reason"])
    comps, entry = parse_module(rewritten)
    ev = _Evaluator(comps, entry, list(params), stream, allow_residual_dots)
    out = ev.run()
    if return_stats:
        return out, {"custom_calls": ev.calls, "plan": plan}
    return out
