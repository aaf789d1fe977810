"""The reference's GemmRewriter test modules (tests/golden/ref_rewrites.json) and seeded inputs for them."""
import json
import os
import re

import numpy as np

from oracle import scaled_dot_oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
EPILOGUE_NUMBER = {"DEFAULT": 0, "BIAS": 1, "RELU": 2, "BIAS_RELU": 3, "GELU": 4, "GELU_AUX": 5, "BIAS_GELU": 6, "BIAS_GELU_AUX": 7}


def load():
    with open(os.path.join(HERE, "golden", "ref_rewrites.json")) as f:
        d = json.load(f)
    return d["fp8"], d["int8"]


def applies_to_blackwell(case) -> bool:
    """Tests the reference skips on a Blackwell CUDA GPU (pre-Ada expectations, ROCm-only types)."""
    notes = " ".join(case["skip_notes"])
    return not ("pre-Ada" in notes or case["test"] in ("FnuzTypeF8",))


def parameters(hlo: str):
    """[(number, type, dims)] of the entry computation's parameters."""
    entry = hlo[hlo.rfind("ENTRY"):] if "ENTRY" in hlo else hlo
    found = {}
    for m in re.finditer(r"=\s*([a-z0-9]+)\[([0-9, ]*)\](?:\{[0-9, ]*\})?\s+parameter\((\d+)\)", entry):
        found[int(m.group(3))] = (m.group(1), tuple(int(x) for x in m.group(2).split(",") if x.strip()))
    return [(i,) + found[i] for i in sorted(found)]


def make_inputs(hlo: str, seed: int):
    """Seeded inputs in the oracle's representation (FP8 code points, bf16 / f16 bit patterns ...).  Values are kept
    small (|x| <= 0.25, scales in [0.5, 1]) so that results over the short contracting dimensions of these modules
    stay of order one or below: several of the reference's bounds are absolute (ErrorSpec{2e-3, 0}), and its tests
    draw their random arguments from a small range too."""
    rng = np.random.default_rng(seed)
    out = []
    for _, t, dims in parameters(hlo):
        if t in ("f8e4m3fn", "f8e5m2"):
            v = rng.uniform(-0.25, 0.25, size=dims).astype(np.float32)
            out.append(o.fp8_encode(v, "e4m3fn" if t == "f8e4m3fn" else "e5m2"))
        elif t == "f8e8m0fnu":
            out.append(rng.integers(121, 132, size=dims, dtype=np.uint8))        # block scales 2^-6 .. 2^4
        elif t == "s8":
            out.append(rng.integers(-127, 128, size=dims, dtype=np.int8))
        elif t == "pred":
            out.append(rng.integers(0, 2, size=dims).astype(bool))
        elif t in ("s32", "s64"):
            out.append(np.zeros(dims, np.int32))
        else:
            v = (rng.uniform(0.5, 1.0, size=dims) if len(dims) == 0 else rng.uniform(-0.25, 0.25, size=dims)).astype(np.float32)
            out.append({"f32": lambda x: x, "bf16": o.f32_to_bf16_bits, "f16": o.f32_to_f16_bits}[t](v))
    return out


def to_f32(t: str, v):
    if t in ("f8e4m3fn", "f8e5m2"):
        return o.fp8_decode(v, "e4m3fn" if t == "f8e4m3fn" else "e5m2")
    if t == "f8e8m0fnu":
        return o.e8m0_decode(v)
    if t == "bf16":
        return o.bf16_bits_to_f32(v)
    if t == "f16":
        return np.asarray(v, np.uint16).view(np.float16).astype(np.float32)
    return np.asarray(v).astype(np.float32)
