"""Times the kernel variants on given shapes and writes the table `b200sd_load_config_table` reads.

    python -m xla_b200.autotune --out table.txt [--shape f8:8192x8192x8192 ...] [--iters 20]

The offline counterpart of the reference's cuBLASLt autotuner backend
(xla/backends/gpu/autotuner/cublaslt.cc:84-189: enumerate the algorithms of a GEMM, time each, keep the
best) and of its persisted result (docs/persisted_autotuning.md).  Shapes are `f8:MxNxK` or `s8:MxNxK`
(A is [M,K], B is [K,N], row-major), or `mx:MxNxK` for the MX block-scaled dot (A is [M,K], B is [N,K], one
f8e8m0fnu scale per 32 values; the candidates are its two tile forms).  Point B200SD_CONFIG_TABLE at the file, or load it with
`xla_b200.load_config_table(path)`, and B200SD_KERNEL_AUTO / selected_config = 0 follows it.
"""
from __future__ import annotations

import argparse
import ctypes as C
import sys

from . import _native

# Configs of the benchmark plus their per-GPU shards.
DEFAULT_SHAPES = ["f8:8192x8192x8192", "f8:8192x4096x8192", "f8:8192x2048x8192", "f8:8192x1024x8192", "f8:4096x4096x4096",
                  "f8:16x28672x8192", "f8:64x28672x8192", "f8:128x28672x8192", "f8:8192x8192x14336", "f8:8192x8192x7168",
                  "s8:4096x4096x4096", "mx:8192x8192x8192", "mx:4096x4096x4096", "mx:2048x8192x4096"]
KERNEL_NAMES = {1: "dense", 2: "split-K", 3: "dense single-CTA", 4: "dense CTA pair", 5: "CTA pair + stream-K tail",
                6: "MX, one 256-column accumulator", 7: "MX, two 224-column accumulators"}


def candidates(kind: str, m: int, n: int, k: int):
    if kind == "mx":
        return [6, 7]
    out = [3, 4, 5] if m > 128 else [3]
    if kind == "f8" and m <= 128 and _native.product.b200sd_workspace_bytes(m, n, k) > 0:
        out.append(2)
    return out


def time_variants(kind: str, m: int, n: int, k: int, kernels, iters: int, rounds: int = 5):
    """Returns {kernel: ms per launch}.  The variants are timed in turn, `rounds` times over, and the
    best round of each is kept, so that clock and temperature drift hits all of them alike."""
    import torch

    from .scaled_dot import F8E8M0FNU, BlockScaledDotCall, Buffer, GemmBackendConfig, Int8DotCall, ScaledDotCall

    dev = torch.device("cuda", torch.cuda.current_device())
    operand_sets = []
    for i in range(2):                                   # two operand sets, so a launch never finds its inputs in L2
        ws = torch.empty(32 << 20, dtype=torch.int8, device=dev)
        if kind == "s8":
            a = torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev)
            b = torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev)
            operand_sets.append(([a, b], [torch.empty((m, n), dtype=torch.int32, device=dev), ws]))
        elif kind == "mx":
            a = torch.randn((m, k), device=dev).to(torch.float8_e4m3fn)
            b = torch.randn((n, k), device=dev).to(torch.float8_e4m3fn)
            sa = torch.randint(120, 135, (m, k // 32), dtype=torch.uint8, device=dev)
            sb = torch.randint(120, 135, (n, k // 32), dtype=torch.uint8, device=dev)
            keep = (sa, sb)                              # the Buffers below hold addresses only
            operand_sets.append(([a, b, Buffer(F8E8M0FNU, tuple(sa.shape), sa.data_ptr()), Buffer(F8E8M0FNU, tuple(sb.shape), sb.data_ptr())],
                                 [torch.empty((m, n), dtype=torch.bfloat16, device=dev), ws], keep))
        else:
            a = torch.randn((m, k), device=dev).to(torch.float8_e4m3fn)
            b = torch.randn((k, n), device=dev).to(torch.float8_e4m3fn)
            one = torch.ones((), device=dev)
            operand_sets.append(([a, b, one, one], [torch.empty((m, n), dtype=torch.bfloat16, device=dev), ws]))
    stream = torch.cuda.current_stream(dev).cuda_stream
    ordinal = dev.index or 0
    calls = {}
    for kern in kernels:
        if kind == "s8":
            calls[kern] = [Int8DotCall(s[0], s[1], selected_algorithm=kern) for s in operand_sets]
        elif kind == "mx":
            calls[kern] = [BlockScaledDotCall(s[0], s[1], selected_algorithm=kern) for s in operand_sets]
        else:
            calls[kern] = [ScaledDotCall(s[0], s[1], GemmBackendConfig(selected_algorithm=kern)) for s in operand_sets]
        for c in calls[kern]:
            c.run(stream, ordinal)
    best = {kern: float("inf") for kern in kernels}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for r in range(rounds + 1):                          # round 0 warms up and is not counted
        for kern in kernels:
            e0.record()
            for i in range(iters):
                calls[kern][i & 1].execute(stream, ordinal)
            e1.record()
            torch.cuda.synchronize()
            if r > 0:
                best[kern] = min(best[kern], e0.elapsed_time(e1) / iters)
    for kern in kernels:
        for c in calls[kern]:
            c.close()
    return best


def parse_shape(text: str):
    kind, dims = text.split(":")
    m, n, k = (int(x) for x in dims.lower().split("x"))
    if kind not in ("f8", "s8", "mx"):
        raise ValueError(f"shape {text}: type must be f8, s8 or mx")
    if kind == "mx" and k % 32:
        raise ValueError(f"shape {text}: k must be a multiple of 32")
    return kind, m, n, k


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--out", required=True)
    ap.add_argument("--shape", action="append", default=None, help="f8:MxNxK, s8:MxNxK or mx:MxNxK; may repeat")
    ap.add_argument("--iters", type=int, default=30)
    args = ap.parse_args(argv)
    lines = ["# type m n k kernel   (written by python -m xla_b200.autotune; times in ms per launch)"]
    for text in args.shape or DEFAULT_SHAPES:
        kind, m, n, k = parse_shape(text)
        timings = time_variants(kind, m, n, k, candidates(kind, m, n, k), args.iters)
        best = min(timings, key=timings.get)
        detail = ", ".join(f"{KERNEL_NAMES[kk]} {t:.4f}" for kk, t in sorted(timings.items()))
        lines.append(f"{kind} {m} {n} {k} {best}   # {detail}")
        print(lines[-1], flush=True)
    with open(args.out, "w") as f:
        f.write("\n".join(lines) + "\n")
    err = C.create_string_buffer(512)
    n_entries = C.c_int32(0)
    rc = _native.product.b200sd_load_config_table(args.out.encode(), C.byref(n_entries), err, len(err))
    if rc != 0:
        print(f"the written table does not load: {err.value.decode()}", file=sys.stderr)
        return 1
    print(f"{args.out}: {n_entries.value} entries")
    return 0


if __name__ == "__main__":
    sys.exit(main())
