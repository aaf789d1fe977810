"""Mini HLO interpreter for test modules.  TEST INFRASTRUCTURE ONLY.

Evaluates the subset of HLO text that the fixtures under tests/golden/hlo and the modules of the
reference's own GemmRewriter tests (tests/golden/ref_rewrites.json) use -- parameter, constant,
convert, broadcast, the element-wise arithmetic, compare, select, clamp, dot, reduce (max / add), pad,
slice, dynamic-slice, concatenate, reshape, bitcast, transpose, copy, tuple, get-tuple-element --
with the interpreter's rules (xla/hlo/evaluator/hlo_evaluator_typed_visitor.h: element-wise ops
computed in f32 and rounded to the instruction's type, dot with f32 accumulation and one final
rounding :1271-1340, maximum / clamp propagating NaN :594-613, :843-865), using the conversions of
scaled_dot_oracle.py.  It lets the SAME module text drive both the expected values and, through
the rewriter, the CUDA path.  Parity status: as for scaled_dot_oracle.py (conversions pinned by the
reference's tables; the dot itself not pinned by stored outputs).

Values are kept as (type, array): FP8 as uint8 code points, bf16 / f16 as uint16 bit patterns,
f32 as float32, s8 / s32 as integers, pred as bool -- the representation the parity tests compare in.
Arrays hold the LOGICAL value; the layout an instruction declares matters only to `bitcast`.
"""
from __future__ import annotations

import re

import numpy as np

from . import scaled_dot_oracle as o

_KIND = {"f8e4m3fn": "e4m3fn", "f8e5m2": "e5m2"}
_INT = {"s8": np.int8, "s32": np.int32, "s64": np.int64, "u8": np.uint8, "u32": np.uint32}


def _to_f32(t, v):
    if t in _KIND:
        return o.fp8_decode(v, _KIND[t])
    if t == "f8e8m0fnu":
        return o.e8m0_decode(v)
    if t == "bf16":
        return o.bf16_bits_to_f32(v)
    if t == "f16":
        return np.asarray(v, np.uint16).view(np.float16).astype(np.float32)
    return np.asarray(v).astype(np.float32)


def _from_f32(t, x):
    x = np.asarray(x, np.float32)
    if t in _KIND:
        return o.fp8_encode(x, _KIND[t])
    if t == "f8e8m0fnu":
        return o.e8m0_encode(x)
    if t == "bf16":
        return o.f32_to_bf16_bits(x)
    if t == "f16":
        return o.f32_to_f16_bits(x)
    if t == "f32":
        return x
    if t in _INT:
        return x.astype(_INT[t])
    if t == "pred":
        return x != 0
    raise ValueError(f"convert to {t}")


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
    """"f32[2,3]{0,1}" -> ("f32", (2, 3), (0, 1) or None)."""
    m = re.match(r"\s*([a-z0-9]+)\[([0-9, ]*)\](?:\{([0-9, ]*)[^}]*\})?", s)
    dims = tuple(int(x) for x in m.group(2).split(",") if x.strip())
    layout = tuple(int(x) for x in m.group(3).split(",") if x.strip()) if m.group(3) else None
    if layout is not None and len(layout) != len(dims):
        layout = None
    return m.group(1), dims, layout


def _parse(text):
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
            lines[-1] += " " + t          # an instruction written over several lines
    comps, cur, entry, last = {}, None, None, None
    for t in lines:
        if t.startswith("HloModule"):
            continue
        if cur is None:
            assert t.endswith("{"), t
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

        def add(line, is_root):
            name, rest = line.split(" = ", 1)
            name = name.strip().lstrip("%")
            m = re.match(r"(\(.*?\)\s|[a-z0-9]+\[[0-9, ]*\](?:\{[^}]*\})?\s)?\s*([a-z\-]+)\((.*)$", rest)
            assert m, rest
            shape, opcode, tail = m.group(1), m.group(2), m.group(3)
            depth, i = 1, 0
            while depth:
                depth += {"(": 1, ")": -1}.get(tail[i], 0)
                i += 1
            args, attrs = tail[: i - 1], tail[i:].lstrip(", ")
            operands = []
            if opcode not in ("constant", "parameter"):
                for k, a in enumerate(_split(args)):
                    a = a.strip()
                    if a.endswith(")"):          # an operand written as an instruction of its own: evaluated first, under a made-up name
                        nested = f"{name}.operand{k}"
                        add(f"{nested} = {a}", False)
                        a = nested
                    operands.append(a.split(" ")[-1].lstrip("%"))
            cur.append(dict(name=name, shape=shape.strip() if shape else None, opcode=opcode, operands=operands,
                            literal=args.strip(), attrs=attrs, root=is_root))

        add(t, root)
        if closes:
            cur = None
    return comps, entry or last


def _attr_dims(attrs, key):
    m = re.search(key + r"=\{([0-9, ]*)\}", attrs)
    return tuple(int(x) for x in m.group(1).split(",") if x.strip()) if m else None


def _physical(dims, layout):
    return tuple(reversed(layout)) if layout is not None else tuple(range(len(dims)))


def _bitcast(v, src, dst):
    """The bytes of `v` as they lie in memory under `src`'s layout, read under `dst`'s (same element size)."""
    _, sdims, slayout = src
    _, ddims, dlayout = dst
    sp, dp = _physical(sdims, slayout), _physical(ddims, dlayout)
    flat = np.ascontiguousarray(np.transpose(np.asarray(v).reshape(sdims), sp)).reshape(-1)
    phys = flat.reshape(tuple(ddims[d] for d in dp))
    inverse = [dp.index(i) for i in range(len(dp))]
    return np.ascontiguousarray(np.transpose(phys, inverse))


def _dot(lhs, rhs, lc, rc, lb, rb):
    """f32 values; batch dims lb / rb; one contracting dim each.  Result dims: batch..., lhs free, rhs free."""
    if lb:
        lperm = list(lb) + [d for d in range(lhs.ndim) if d not in lb]
        rperm = list(rb) + [d for d in range(rhs.ndim) if d not in rb]
        l2, r2 = np.transpose(lhs, lperm), np.transpose(rhs, rperm)
        nb = len(lb)
        lc2, rc2 = lperm.index(lc) - nb, rperm.index(rc) - nb
        bshape = l2.shape[:nb]
        l3, r3 = l2.reshape((-1,) + l2.shape[nb:]), r2.reshape((-1,) + r2.shape[nb:])
        parts = [o.dot_f32(np.ascontiguousarray(l3[i]), np.ascontiguousarray(r3[i]), lc2, rc2) for i in range(l3.shape[0])]
        out = np.stack(parts)
        return out.reshape(bshape + out.shape[1:])
    return o.dot_f32(lhs, rhs, lc, rc)


def _scaled_dot(t, lhs, rhs, lhs_scale, rhs_scale, lc, rc, lb, rb):
    """The `scaled-dot` instruction as the interpreter defines it (HandleScaledDot,
    hlo_evaluator_typed_visitor.h:1783-1990).  All four operands are first converted to the result type; a scale of
    rank 0 counts as 1; a scale entry covers dim / scale_dim consecutive indices in every dimension; each result
    element is the sum over k, in order, of ((lhs * lhs_scale) * rhs) * rhs_scale in f32.  `lhs` .. `rhs_scale` are
    (type, value) pairs; returns f32 values [batch..., lhs free, rhs free]."""
    def prepared(v, sc):
        x = _to_f32(t, _from_f32(t, _to_f32(*v)))
        if np.ndim(sc[1]) == 0:
            return x, np.ones_like(x)
        y = _to_f32(t, _from_f32(t, _to_f32(*sc)))
        assert y.ndim == x.ndim and all(d % e == 0 for d, e in zip(x.shape, y.shape)), (x.shape, y.shape)
        for axis, (d, e) in enumerate(zip(x.shape, y.shape)):
            if d != e:
                y = np.repeat(y, d // e, axis=axis)
        return x, y

    (a, sa), (b, sb) = prepared(lhs, lhs_scale), prepared(rhs, rhs_scale)
    nb = len(lb)
    lfree = [d for d in range(a.ndim) if d not in lb and d != lc]
    rfree = [d for d in range(b.ndim) if d not in rb and d != rc]
    lperm, rperm = list(lb) + lfree + [lc], list(rb) + rfree + [rc]
    a, sa, b, sb = a.transpose(lperm), sa.transpose(lperm), b.transpose(rperm), sb.transpose(rperm)
    bshape, mshape, nshape, k = a.shape[:nb], a.shape[nb:-1], b.shape[nb:-1], a.shape[-1]
    a, sa = a.reshape(bshape + (-1, 1, k)), sa.reshape(bshape + (-1, 1, k))
    b, sb = b.reshape(bshape + (1, -1, k)), sb.reshape(bshape + (1, -1, k))
    acc = np.zeros(bshape + (a.shape[-3], b.shape[-2]), np.float32)
    with np.errstate(over="ignore", invalid="ignore", under="ignore"):
        for i in range(k):
            acc += ((a[..., i] * sa[..., i]) * b[..., i]) * sb[..., i]
    return acc.reshape(bshape + mshape + nshape)


def evaluate(text, params):
    """Runs the ENTRY computation on `params` (list, in parameter order, in the representation
    described in the module docstring).  Returns the root value, or a tuple of values."""
    comps, entry = _parse(text)
    env, shapes = {}, {}
    result = None
    for ins in comps[entry]:
        op, name, attrs = ins["opcode"], ins["name"], ins["attrs"]
        shape_text = ins["shape"]
        if shape_text is None:
            shp = shapes[ins["operands"][0]]                  # a shape left out is the first operand's
        elif shape_text.startswith("("):
            shp = ("tuple", (), None)
        else:
            shp = _shape(shape_text)
        t, dims = shp[0], shp[1]
        a = [env[x] for x in ins["operands"]]
        a_shapes = [shapes[x] for x in ins["operands"]]
        if op == "parameter":
            val = (t, np.asarray(params[int(ins["literal"])]).reshape(dims))
        elif op == "constant":
            lit = ins["literal"]
            v = {"inf": np.inf, "-inf": -np.inf, "nan": np.nan, "true": 1.0, "false": 0.0}.get(lit)
            v = float(lit) if v is None else v
            val = (t, _from_f32(t, np.full(dims, v, np.float32)) if t not in _INT else np.full(dims, int(v), _INT[t]))
        elif op == "convert":
            st, sv = a[0]
            if st in _INT and t == "f32":
                val = (t, np.asarray(sv).astype(np.float32))
            elif st == "pred":
                val = (t, _from_f32(t, np.asarray(sv).astype(np.float32)))
            else:
                val = (t, _from_f32(t, _to_f32(st, sv)))
        elif op == "copy":
            val = a[0]
        elif op == "reshape":
            val = (t, np.asarray(a[0][1]).reshape(dims))
        elif op == "bitcast":
            val = (t, _bitcast(a[0][1], a_shapes[0], shp))
        elif op == "transpose":
            val = (t, np.ascontiguousarray(np.transpose(np.asarray(a[0][1]), _attr_dims(attrs, "dimensions"))))
        elif op == "broadcast":
            bd = _attr_dims(attrs, "dimensions") or ()
            st, sv = a[0]
            view = [1] * len(dims)
            for i, d in enumerate(bd):
                view[d] = dims[d]
            val = (t, np.broadcast_to(np.asarray(sv).reshape(view), dims).copy())
        elif op == "slice":
            spec = re.search(r"slice=\{(.*?)\}", attrs).group(1)
            idx = []
            for part in re.findall(r"\[([0-9:]+)\]", spec):
                nums = [int(x) for x in part.split(":")]
                idx.append(slice(nums[0], nums[1], nums[2] if len(nums) > 2 else 1))
            val = (t, np.ascontiguousarray(np.asarray(a[0][1])[tuple(idx)]))
        elif op == "dynamic-slice":
            sizes = _attr_dims(attrs, "dynamic_slice_sizes")
            src = np.asarray(a[0][1])
            starts = [int(np.asarray(s[1]).reshape(())) for s in a[1:]]
            starts = [min(max(s, 0), src.shape[i] - sizes[i]) for i, s in enumerate(starts)]     # clamped, as XLA does
            val = (t, np.ascontiguousarray(src[tuple(slice(s, s + n) for s, n in zip(starts, sizes))]))
        elif op == "pad":
            cfg = re.search(r"padding=([0-9_x\-]+)", attrs).group(1)
            lo_hi = [tuple(int(v) for v in part.split("_")) for part in cfg.split("x")]
            assert all(len(p) == 2 or p[2] == 0 for p in lo_hi), "interior padding"
            src = np.asarray(a[0][1])
            out = np.empty(dims, src.dtype)
            out[...] = np.asarray(a[1][1]).reshape(())
            out[tuple(slice(lo, lo + n) for n, (lo, *_rest) in zip(src.shape, lo_hi))] = src
            val = (t, out)
        elif op == "concatenate":
            val = (t, np.concatenate([np.asarray(x[1]) for x in a], axis=_attr_dims(attrs, "dimensions")[0]))
        elif op == "select":
            val = (t, np.where(np.asarray(a[0][1]).astype(bool), np.asarray(a[1][1]), np.asarray(a[2][1])))
        elif op == "compare":
            direction = re.search(r"direction=([A-Z]+)", attrs).group(1)
            x, y = _to_f32(*a[0]), _to_f32(*a[1])
            fn = {"EQ": np.equal, "NE": np.not_equal, "LT": np.less, "LE": np.less_equal, "GT": np.greater, "GE": np.greater_equal}[direction]
            val = ("pred", fn(x, y))
        elif op in ("multiply", "divide", "add", "subtract", "maximum", "minimum"):
            if a[0][0] in _INT:
                x, y = np.asarray(a[0][1]), np.asarray(a[1][1])
                r = {"multiply": x * y, "add": x + y, "subtract": x - y, "maximum": np.maximum(x, y), "minimum": np.minimum(x, y),
                     "divide": None}[op]
                val = (t, r.astype(_INT[t]))
            else:
                x, y = _to_f32(*a[0]), _to_f32(*a[1])
                with np.errstate(all="ignore"):
                    if op == "multiply":
                        r = x * y
                    elif op == "divide":
                        r = x / y
                    elif op == "add":
                        r = x + y
                    elif op == "subtract":
                        r = x - y
                    else:
                        pick = np.maximum if op == "maximum" else np.minimum
                        r = np.where(np.isnan(x) | np.isnan(y), np.float32(np.nan), pick(x, y))
                val = (t, _from_f32(t, r.astype(np.float32)))
        elif op in ("tanh", "abs", "negate", "exponential", "sqrt", "rsqrt", "logistic"):
            x = _to_f32(*a[0])
            with np.errstate(all="ignore"):
                r = {"tanh": np.tanh, "abs": np.abs, "negate": np.negative, "exponential": np.exp, "sqrt": np.sqrt,
                     "rsqrt": lambda v: 1.0 / np.sqrt(v), "logistic": lambda v: 1.0 / (1.0 + np.exp(-v))}[op](x)
            val = (t, _from_f32(t, np.asarray(r, np.float32)))
        elif op == "clamp":
            lo, x, hi = (_to_f32(*v) for v in a)
            with np.errstate(invalid="ignore"):
                r = np.where(np.isnan(x), x, np.minimum(np.maximum(x, lo), hi))
            val = (t, _from_f32(t, r))
        elif op == "reduce":
            x, init = _to_f32(*a[0]), _to_f32(*a[1])
            body = comps[re.search(r"to_apply=%?([A-Za-z0-9_.\-]+)", attrs).group(1)]
            kind = next((i["opcode"] for i in body if i["root"]), body[-1]["opcode"])
            rd = _attr_dims(attrs, "dimensions")
            axes = tuple(rd) if rd else None
            if kind == "maximum":
                with np.errstate(invalid="ignore"):
                    r = np.maximum(np.float32(init), x.max(axis=axes) if x.size else init)
                r = np.where(np.isnan(x).any(axis=axes), np.float32(np.nan), r)
            elif kind == "add":
                r = x.sum(axis=axes, dtype=np.float32) + np.float32(init)
            else:
                raise NotImplementedError(f"reduce with {kind}")
            val = (t, _from_f32(t, np.asarray(r, np.float32).reshape(dims)))
        elif op == "dot":
            lc = _attr_dims(attrs, "lhs_contracting_dims")[0]
            rc = _attr_dims(attrs, "rhs_contracting_dims")[0]
            lb, rb = _attr_dims(attrs, "lhs_batch_dims") or (), _attr_dims(attrs, "rhs_batch_dims") or ()
            (lt, lv), (rt, rv) = a
            if lt in _INT and t not in _INT:
                # integer operands, floating-point result: the interpreter converts the operands to the result type
                # and accumulates there (hlo_evaluator_typed_visitor.h:1271-1340); sums stay exact below 2^24
                val = (t, _from_f32(t, _dot(np.asarray(lv).astype(np.float32), np.asarray(rv).astype(np.float32), lc, rc, lb, rb)))
            elif lt == "s8" and not lb and np.asarray(lv).ndim == 2 and np.asarray(rv).ndim == 2:
                val = (t, o.dot_s8(lv, rv, lc, rc))
            elif lt in _INT and not lb:        # several free dimensions: exact integer contraction
                val = (t, np.tensordot(np.asarray(lv, np.int64), np.asarray(rv, np.int64), axes=([lc], [rc])).astype(_INT[t]))
            elif lt in _INT:
                val = (t, _dot(np.asarray(lv, np.float64).astype(np.float32), np.asarray(rv, np.float64).astype(np.float32), lc, rc, lb, rb).astype(_INT[t]))
            else:
                val = (t, _from_f32(t, _dot(_to_f32(lt, lv), _to_f32(rt, rv), lc, rc, lb, rb)))
        elif op == "scaled-dot":
            lc = _attr_dims(attrs, "lhs_contracting_dims")[0]
            rc = _attr_dims(attrs, "rhs_contracting_dims")[0]
            lb, rb = _attr_dims(attrs, "lhs_batch_dims") or (), _attr_dims(attrs, "rhs_batch_dims") or ()
            val = (t, _from_f32(t, _scaled_dot(t, a[0], a[1], a[2], a[3], lc, rc, lb, rb)))
        elif op == "custom-call" and '"__op$block_scaled_dot"' in attrs:
            # block_scaling_rewriter.h:30-77; evaluated as the expansion of block_scaling_rewriter.cc:194-262
            (lt, lv), (rt, rv), (st, sv), (ut, uv) = a[:4]
            assert len(a) == 4 and st == ut == "f8e8m0fnu", "only the MX form (f8e8m0fnu scales, no global scale) is evaluated"
            code = {"f32": o.F32, "bf16": o.BF16, "f16": o.F16}[t]
            bs = re.search(r"block_size\W*(\d+)", attrs)          # explicit block size (block_scaling_rewriter.cc:613-621)
            val = (t, o.block_scaled_dot(lv, rv, sv, uv, a_kind=_KIND[lt], b_kind=_KIND[rt], out_dtype=code,
                                         block_size=int(bs.group(1)) if bs else None))
        elif op == "tuple":
            val = ("tuple", tuple(v for _, v in a))
        elif op == "get-tuple-element":
            idx = int(re.search(r"index=(\d+)", attrs).group(1))
            val = ("?", a[0][1][idx])
        else:
            raise NotImplementedError(op)
        env[name], shapes[name] = val, shp
        if ins["root"]:
            result = val
    if result is None:
        result = env[comps[entry][-1]["name"]]
    return result[1]


def root_types(text):
    """Element types of the module's result: a list (one entry per tuple element)."""
    comps, entry = _parse(text)
    ins = next((i for i in comps[entry] if i["root"]), comps[entry][-1])
    s = ins["shape"]
    if s is None:
        return None
    if s.startswith("("):
        return [_shape(p)[0] for p in _split(s[1:-1])]
    return [_shape(s)[0]]
