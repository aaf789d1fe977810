"""Mini HLO interpreter for the fixture modules.  TEST INFRASTRUCTURE ONLY.

Evaluates the small subset of HLO text the fixtures under tests/golden/hlo use (parameter,
constant, convert, broadcast, multiply, divide, add, dot, tanh, maximum, abs, reduce with a max
computation, clamp, copy, bitcast, reshape, tuple, get-tuple-element) with the interpreter's rules
(xla/hlo/evaluator/hlo_evaluator_typed_visitor.h: element-wise ops in the operand type, dot with
f32 accumulation :1271-1340, maximum / clamp propagating NaN :594-613, :843-865), using the
conversions of scaled_dot_oracle.py.  It lets the SAME module text drive both the expected values
and, through the rewriter, the CUDA path.  Parity status: as for scaled_dot_oracle.py (conversions
pinned by the reference's tables; the dot itself not pinned by stored outputs).

Values are kept as (type, array): FP8 as uint8 code points, bf16 / f16 as uint16 bit patterns,
f32 as float32, s8 / s32 as integers -- the same representation the parity tests compare in.
"""
from __future__ import annotations

import re

import numpy as np

from . import scaled_dot_oracle as o

_KIND = {"f8e4m3fn": "e4m3fn", "f8e5m2": "e5m2"}


def _to_f32(t, v):
    if t in _KIND:
        return o.fp8_decode(v, _KIND[t])
    if t == "bf16":
        return o.bf16_bits_to_f32(v)
    if t == "f16":
        return np.asarray(v, np.uint16).view(np.float16).astype(np.float32)
    return np.asarray(v).astype(np.float32)


def _from_f32(t, x):
    x = np.asarray(x, np.float32)
    if t in _KIND:
        return o.fp8_encode(x, _KIND[t])
    if t == "bf16":
        return o.f32_to_bf16_bits(x)
    if t == "f16":
        return o.f32_to_f16_bits(x)
    if t == "f32":
        return x
    if t == "s32":
        return x.astype(np.int32)
    raise ValueError(f"convert to {t}")


def _parse(text):
    comps, cur = {}, None
    entry = None
    for line in text.splitlines():
        t = line.strip()
        if not t or t.startswith("//") or t.startswith("HloModule"):
            continue
        if cur is None:
            assert t.endswith("{"), t
            head = t[:-1].strip()
            is_entry = head.startswith("ENTRY ")
            name = re.split(r"[ (]", head[6:].strip() if is_entry else head)[0].lstrip("%")
            cur = comps.setdefault(name, [])
            if is_entry:
                entry = name
            continue
        if t == "}":
            cur = None
            continue
        root = t.startswith("ROOT ")
        if root:
            t = t[5:].strip()
        name, rest = t.split(" = ", 1)
        m = re.match(r"(\(.*?\)|[a-z0-9]+\[[0-9, ]*\](?:\{[0-9,]*\})?)\s+([a-z\-]+)\((.*)$", rest)
        assert m, rest
        shape, opcode, tail = m.group(1), m.group(2), m.group(3)
        depth, i = 1, 0
        while depth:
            depth += {"(": 1, ")": -1}.get(tail[i], 0)
            i += 1
        args, attrs = tail[: i - 1], tail[i:].lstrip(", ")
        operands = [a.strip().split(" ")[-1].lstrip("%") for a in _split(args)] if opcode not in ("constant", "parameter") else []
        cur.append(dict(name=name.strip().lstrip("%"), shape=shape, opcode=opcode, operands=operands, literal=args.strip(),
                        attrs=attrs, root=root))
    return comps, entry


def _split(s):
    out, cur, d = [], "", 0
    for c in s:
        d += c in "([{"
        d -= c in ")]}"
        if c == "," and d == 0:
            out.append(cur)
            cur = ""
        else:
            cur += c
    if cur.strip():
        out.append(cur)
    return out


def _shape(s):
    m = re.match(r"([a-z0-9]+)\[([0-9, ]*)\]", s)
    dims = tuple(int(x) for x in m.group(2).split(",") if x.strip())
    return m.group(1), dims


def _attr_dims(attrs, key):
    m = re.search(key + r"=\{([0-9, ]*)\}", attrs)
    return tuple(int(x) for x in m.group(1).split(",") if x.strip()) if m else None


def evaluate(text, params):
    """Runs the ENTRY computation on `params` (list, in parameter order, in the representation
    described in the module docstring).  Returns the root value, or a tuple of values."""
    comps, entry = _parse(text)
    env = {}
    result = None
    for ins in comps[entry]:
        op, name = ins["opcode"], ins["name"]
        if ins["shape"].startswith("("):
            t, dims = "tuple", ()
        else:
            t, dims = _shape(ins["shape"])
        a = [env[x] for x in ins["operands"]]
        if op == "parameter":
            val = (t, np.asarray(params[int(ins["literal"])]).reshape(dims))
        elif op == "constant":
            lit = ins["literal"]
            v = {"inf": np.inf, "-inf": -np.inf, "nan": np.nan}.get(lit)
            v = float(lit) if v is None else v
            val = (t, _from_f32(t, np.full(dims, v, np.float32)) if t != "s32" else np.full(dims, int(v), np.int32))
        elif op == "convert":
            st, sv = a[0]
            if st in ("s32", "s8") and t == "f32":
                val = (t, sv.astype(np.float32))
            else:
                val = (t, _from_f32(t, _to_f32(st, sv)))
        elif op in ("copy",):
            val = a[0]
        elif op in ("bitcast", "reshape"):            # default layouts only: a row-major reinterpretation of the shape
            val = (t, np.asarray(a[0][1]).reshape(dims))
        elif op == "broadcast":
            bd = _attr_dims(ins["attrs"], "dimensions") or ()
            st, sv = a[0]
            shape = [1] * len(dims)
            for i, d in enumerate(bd):
                shape[d] = dims[d]
            val = (t, np.broadcast_to(np.asarray(sv).reshape(shape), dims).copy())
        elif op in ("multiply", "divide", "add", "maximum"):
            x, y = _to_f32(*a[0]), _to_f32(*a[1])
            with np.errstate(all="ignore"):
                if op == "multiply":
                    r = x * y
                elif op == "divide":
                    r = x / y
                elif op == "add":
                    r = x + y
                else:
                    r = np.where(np.isnan(x) | np.isnan(y), np.float32(np.nan), np.maximum(x, y))
            val = (t, _from_f32(t, r.astype(np.float32)))
        elif op == "tanh":
            val = (t, _from_f32(t, np.tanh(_to_f32(*a[0])).astype(np.float32)))
        elif op == "abs":
            val = (t, _from_f32(t, np.abs(_to_f32(*a[0]))))
        elif op == "clamp":
            lo, x, hi = (_to_f32(*v) for v in a)
            with np.errstate(invalid="ignore"):
                r = np.where(np.isnan(x), x, np.minimum(np.maximum(x, lo), hi))
            val = (t, _from_f32(t, r))
        elif op == "reduce":
            x, init = _to_f32(*a[0]), _to_f32(*a[1])
            body = comps[re.search(r"to_apply=%?([A-Za-z0-9_.]+)", ins["attrs"]).group(1)]
            assert any(i["opcode"] == "maximum" for i in body), "only max reductions are supported"
            r = np.float32(np.nan) if np.isnan(x).any() else np.maximum(np.float32(init), x.max() if x.size else init)
            val = (t, _from_f32(t, np.asarray(r, np.float32).reshape(dims)))
        elif op == "dot":
            lc = _attr_dims(ins["attrs"], "lhs_contracting_dims")[0]
            rc = _attr_dims(ins["attrs"], "rhs_contracting_dims")[0]
            (lt, lv), (rt, rv) = a
            if "lhs_batch_dims" in ins["attrs"]:
                # one leading batch dimension on both operands: independent dots, stacked
                assert _attr_dims(ins["attrs"], "lhs_batch_dims") == (0,) and _attr_dims(ins["attrs"], "rhs_batch_dims") == (0,)
                fl, fr = _to_f32(lt, lv), _to_f32(rt, rv)
                parts = [o.dot_f32(fl[i], fr[i], lc - 1, rc - 1) for i in range(fl.shape[0])]
                val = (t, _from_f32(t, np.stack(parts)))
            elif lt == "s8":
                val = (t, o.dot_s8(lv, rv, lc, rc))
            else:
                val = (t, _from_f32(t, o.dot_f32(_to_f32(lt, lv), _to_f32(rt, rv), lc, rc)))
        elif op == "tuple":
            val = ("tuple", tuple(v for _, v in a))
        elif op == "get-tuple-element":
            idx = int(re.search(r"index=(\d+)", ins["attrs"]).group(1))
            val = ("?", a[0][1][idx])
        else:
            raise NotImplementedError(op)
        env[name] = val
        if ins["root"]:
            result = val
    if result is None:
        result = env[comps[entry][-1]["name"]]
    return result[1]
