#!/usr/bin/env python
"""Benchmark of the quantized scaled-dot hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|cublaslt] [--workload c1|...]

A "step" is one pass of the hot path over one batch of synthetic input: one custom call through
the XLA FFI boundary of libb200_scaled_dot.so.  Default workload `c1` is BASELINE config 1:
M=N=K=8192 e4m3fn operands (values from N(0,1) scaled to amax 448), per-tensor f32 scales, bf16
bias ~N(0,0.02), GELU, scaled e4m3fn output (out_scale 1.0) and an f32 amax.  On N>1 GPUs B, bias
and D are N-split column-parallel (A replicated) with no collective: total work is fixed, so
scaling is "strong".

Timing: W (>=3) untimed warm-up steps, then exactly K steps between two CUDA events on the
launching stream, bracketed by barrier + synchronize; max over ranks.  Two operand/result sets
are used alternately and together exceed the 126 MB L2, so no step finds its inputs in cache.

The one JSON line carries, besides the contract's keys:
  e2e          the same call with HOST buffers: pinned host -> device copies of every input and
               device -> host copies of every result inside the timed region (upload, call and
               download of consecutive steps overlapped on three streams)
  roofline     for the dominant kernel of the headline workload
  sustained    the headline workload launched back to back for at least two seconds with the
               clock sampler running: TFLOP/s, median SM MHz, fraction of the tensor rate at
               that clock and of twice the sustained bf16 figure
  secondary    the other BASELINE configurations, a few hundred launches each: config 2 (decode,
               GB/s at M = 16 / 64 / 128, and N-split at N > 1), config 3 (int8, TOP/s and the
               number of s32 mismatches against the oracle on a block of rows), and at N > 1
               config 4 (K-split dot + sum across ranks, ms, max over ranks)
  cpu_baseline the CPU oracle timed on a bounded sample, all host threads
  clocks, gpu_launches

`--impl cublaslt` times the library the reference's GPU path calls on the same shapes (one GPU).
`--impl reference` times the reference arithmetic on the host cores (XLA's own CPU backend cannot
be built offline, so this is the NumPy/BLAS port in oracle/), on a bounded sample of the same
workload, and prints the same line with "impl": "reference".  `--workload`, `--m/--n/--k` and
`--kernel` select other workloads / sizes / kernel variants for profiler captures.
"""
import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FP8 scaled-dot TFLOP/s at 8192^3 per B200 and at 2/4/8 GPUs; % of FP8 dense peak"
WORKLOAD_NAME = {
    "c1": "config 1: dense FP8 linear 8192^3, bias + GELU + scaled e4m3 output + amax",
    "plain": "scaled dot, bf16 output, no epilogue",
    "c2": "config 2: decode-shape FP8 dot, bf16 output",
    "c3": "config 3: int8 dot + per-row x per-column dequant to bf16",
    "c4": "config 4: row-parallel FP8 dot + sum of the bf16 partials across ranks",
    "mx": "MX block-scaled FP8 dot (one e8m0 scale per 32 values along K), bf16 output",
}
DEFAULT_DIMS = {"c1": (8192, 8192, 8192), "plain": (8192, 8192, 8192), "c2": (64, 28672, 8192),
                "c3": (4096, 4096, 4096), "c4": (8192, 8192, 28672), "mx": (8192, 8192, 8192)}
FLOP_PER_CLK_PER_SM = 16384.0      # dense 8-bit tensor rate of one SM: 8192 multiply-adds per clock
# dram__bytes_read.sum + dram__bytes_write.sum per launch, each from one ncu capture of that kernel at
# that size on one GPU (bytes).
NCU_DRAM_BYTES_PER_LAUNCH = {("c1", 8192, 8192, 8192): 396.0e6, ("c2", 64, 28672, 8192): 240.06e6,
                             ("c3", 4096, 4096, 4096): 33.8e6}


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "cublaslt"])
    p.add_argument("--workload", default="c1", choices=sorted(WORKLOAD_NAME))
    p.add_argument("--overlap", type=int, default=-1, help="c4, N>1: 2 = sum formed inside the dot's kernel over peer memory (default), 1 = NCCL all-reduce of "
                   "finished row blocks on a second stream, 0 = dot then one NCCL all-reduce")
    p.add_argument("--multicast", type=int, default=-1, help="c4 fused: use the NVSwitch multicast mappings (finished rows by multimem.st, pulled sums by "
                   "multimem.ld_reduce); default: on with the pull forms")
    p.add_argument("--pull", type=int, default=-1, help="c4 fused: 1 / 2 = partials stay with their producer and the owner of the rows fetches their sum "
                   "(in the switch with --multicast 1; 2 = piecewise during the next round), 0 = partials are pushed to the owner; "
                   "default: measured best per GPU count")
    p.add_argument("--ar-rows", type=int, default=2048, help="c4 overlap: rows of D per all-reduce")
    p.add_argument("--gemm-ctas", type=int, default=132, help="c4 overlap: SMs the dot may occupy")
    p.add_argument("--nccl-ctas", type=int, default=16, help="c4 overlap: CTAs the collective may use (0 = NCCL's choice)")
    p.add_argument("--m", type=int, default=0)
    p.add_argument("--n", type=int, default=0)
    p.add_argument("--k", type=int, default=0)
    p.add_argument("--kernel", type=int, default=0, help="0 auto, 1 dense, 2 split-K, 3 dense single-CTA, 4 dense CTA pair, 5 CTA pair with a stream-K tail")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-secondary", action="store_true", help="headline workload only (profiler captures)")
    p.add_argument("--no-sustained", action="store_true")
    p.add_argument("--secondary-steps", type=int, default=200, help="timed launches per secondary configuration (launch-list captures use fewer)")
    p.add_argument("--sustained-seconds", type=float, default=2.2)
    p.add_argument("--counters", action="store_true", help="print the kernels' own wait counters of the last launch "
                   "(needs the tuning build: B200SD_LIBRARY=xla_b200/lib/libb200_scaled_dot_tuning.so B200SD_TIMING=1)")
    return p.parse_args()


def workload_dims(args):
    dflt = DEFAULT_DIMS[args.workload]
    return (args.m or dflt[0], args.n or dflt[1], args.k or dflt[2])


def config_block(kind, m, n, k, parallelism):
    return {"workload": WORKLOAD_NAME[kind], "m": m, "n": n, "k": k, "parallelism": parallelism,
            "l2": "two operand/result sets used alternately; together larger than the 126 MB L2"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def c4_link_bytes(world, m, n, in_switch):
    """Bytes every rank must send over NVLink (per direction) to sum the bf16 [m, n] partials of a K-split and leave the sum
    on every rank.  Without the switch's help: reduce-scatter + all-gather, 2 (N-1)/N of the result.  With the in-switch sum
    (multimem.ld_reduce / multimem.st): every partial block leaves its producer once -- the own block too, it is added in
    the switch like the others -- and every finished block once: (N + 1)/N of the result."""
    full = float(m) * n * 2
    return full * (world + 1) / world if in_switch else 2.0 * (world - 1) / world * full


def algorithmic_bytes(kind, m, n, k):
    if kind == "c2":
        return k * n + m * k + 2 * m * n
    if kind == "c3":
        return m * k + k * n + 2 * m * n + 4 * (m + n)
    if kind == "c1":
        return m * k + k * n + m * n + 2 * n    # e4m3 in, e4m3 out, bf16 bias
    if kind == "mx":
        return m * k + k * n + (m + n) * (k // 32) + 2 * m * n
    return m * k + k * n + 2 * m * n            # bf16 out


# --------------------------------------------------------------------------------------------- CPU arm
def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_block(kind, a, b, extra):
    """The oracle on one block of rows: dequantise + dot + epilogue, exactly the workload's arithmetic."""
    from oracle import scaled_dot_oracle as o

    if kind == "c3":
        rs, cs = extra
        return o.dequant_s32_to_bf16(o.dot_s8(a, b), rs, cs)
    if kind == "c1":
        return o.scaled_dot_f8(a, b, 0.01, 0.01, bias=extra, epilogue=o.EPI_BIAS_GELU, d_scale=1.0, out_dtype=o.F8E4M3FN,
                               want_amax=True)
    return o.scaled_dot_f8(a, b, 0.01, 0.01, out_dtype=o.BF16)


def cpu_sample_step(wl, m_rows, n_cols, pool, threads, seed=0):
    """One pass of the oracle over an [m_rows, K] x [K, n_cols] sample of the workload, the work dealt out to
    `threads` workers by columns (NumPy releases the interpreter lock inside its loops and in BLAS, whose own
    threading is switched off meanwhile).  Returns (seconds, algorithmic units): flops, or bytes for c2."""
    import numpy as np

    kind, (m, n, k) = wl
    rng = np.random.default_rng(seed)
    if kind == "c3":
        a = rng.integers(-127, 128, size=(m_rows, k), dtype=np.int8)
        b = rng.integers(-127, 128, size=(k, n_cols), dtype=np.int8)
        rs = rng.uniform(0.001, 0.02, size=m_rows).astype(np.float32)
        cs = rng.uniform(0.001, 0.02, size=n_cols).astype(np.float32)
    else:
        a = rng.integers(0, 0x7F, size=(m_rows, k), dtype=np.uint8)       # finite e4m3 code points
        b = rng.integers(0, 0x7F, size=(k, n_cols), dtype=np.uint8)
        bias = rng.standard_normal(n_cols).astype(np.float32) * np.float32(0.02)
    # Column blocks: every worker dequantises its own columns of B once and the (few) rows of A.
    parts = max(1, min(threads, n_cols // 64))
    bounds = [n_cols * i // parts for i in range(parts + 1)]
    t0 = time.perf_counter()
    futures = []
    for i in range(parts):
        cols = slice(bounds[i], bounds[i + 1])
        extra = (rs, cs[cols]) if kind == "c3" else (bias[cols] if kind == "c1" else None)
        futures.append(pool.submit(cpu_block, kind, a, np.ascontiguousarray(b[:, cols]), extra))
    for f in futures:
        f.result()
    dt = time.perf_counter() - t0
    units = (k * n_cols + m_rows * k + 2 * m_rows * n_cols) if kind == "c2" else 2.0 * m_rows * n_cols * k
    return dt, units


def cpu_arm(wl, budget_s, steps, warmup):
    """Times `steps` oracle passes on a sample sized so that everything fits in `budget_s`."""
    from concurrent.futures import ThreadPoolExecutor

    kind, (m, n, k) = wl
    threads = host_threads()
    try:
        from threadpoolctl import threadpool_limits
        blas_guard = threadpool_limits(limits=1)          # one BLAS thread per worker: the workers are the parallelism
    except Exception:
        blas_guard = None
    pool = ThreadPoolExecutor(max_workers=threads)
    try:
        m_rows, n_cols = min(m, max(64, 16 * threads)), min(n, 1024)
        dt, _ = cpu_sample_step(wl, m_rows, n_cols, pool, threads)           # calibration (also starts the workers)
        per_step_budget = budget_s / max(1, steps + warmup)
        while dt * 3.0 < per_step_budget and (m_rows < m or n_cols < n):
            if n_cols < n:
                n_cols = min(n, n_cols * 2)
            else:
                m_rows = min(m, m_rows * 2)
            dt, _ = cpu_sample_step(wl, m_rows, n_cols, pool, threads)
        for _ in range(warmup):
            cpu_sample_step(wl, m_rows, n_cols, pool, threads)
        total_t, total_u = 0.0, 0.0
        for i in range(steps):
            t, u = cpu_sample_step(wl, m_rows, n_cols, pool, threads, seed=i)
            total_t += t
            total_u += u
    finally:
        pool.shutdown()
        if blas_guard is not None:
            blas_guard.restore_original_limits()
    scale = 1e-9 if kind == "c2" else 1e-12
    return {"value": total_u / total_t * scale, "unit": "GB/s" if kind == "c2" else "TFLOP/s", "cores": threads,
            "kind": "port", "ms_per_step": 1e3 * total_t / steps,
            "sample": f"{steps} passes of the NumPy/BLAS oracle over A[{m_rows},{k}] x B[{k},{n_cols}] "
                      f"(a {m_rows}x{n_cols} block of the {m}x{n} output), dequantise + dot + epilogue, columns dealt out to "
                      f"{threads} worker threads"}


# --------------------------------------------------------------------------------------------- clocks
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, device_index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            uuid_index = device_index
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                try:
                    uuid_index = int(vis.split(",")[device_index])
                except ValueError:
                    uuid_index = device_index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(uuid_index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def finish(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------------------------- GPU arm
class Bench:
    """Per-process state of the GPU arm: device, rank, and the timing loop shared by every workload."""

    def __init__(self, args):
        import torch
        import torch.distributed as dist

        import xla_b200

        self.torch, self.dist, self.lib, self.args = torch, dist, xla_b200, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(self.local_rank)
        self.dev = torch.device("cuda", self.local_rank)
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.stream = torch.cuda.current_stream().cuda_stream

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x):
        t = self.torch.tensor([x], device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def time_steps(self, step, steps, warmup, sample_clocks=False):
        """`warmup` untimed steps, then exactly `steps` between two events; ms per step, max over ranks."""
        torch = self.torch
        for i in range(warmup):
            step(i)
        self.barrier()
        launches0 = self.lib.launch_count()
        sampler = ClockSampler(self.local_rank) if sample_clocks else None
        if sampler:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        clocks = sampler.finish() if sampler else None
        self.barrier()
        launches = self.lib.launch_count() - launches0
        ms = self.max_over_ranks(e0.elapsed_time(e1) / steps)
        status = self.lib.device_status()
        assert status == 0, f"device status word {status:#x}"
        return ms, clocks, launches

    # ---- problems ---------------------------------------------------------------------------
    def shard(self, kind, m, n, k):
        from xla_b200 import sharding

        if kind == "c4":
            ks = sharding.row_parallel_slices(k, self.world, self.rank)
            return m, n, ks.stop - ks.start
        cols = sharding.column_parallel_slices(n, self.world, self.rank)
        return m, cols.stop - cols.start, k

    def f8_operand(self, shape, seed):
        torch = self.torch
        g = torch.Generator(device=self.dev).manual_seed(seed)
        v = torch.randn(shape, device=self.dev, generator=g)
        s = (v.abs().max() / 448.0).reshape(()).float()
        return (v / s).to(torch.float8_e4m3fn), s

    def make_sets(self, kind, lm, ln, lk, kernel=0, emit_s32=False):
        """Two rotating operand/result sets of one workload, each bound to its own call site."""
        torch = self.torch
        from xla_b200.scaled_dot import (BlockScaledDotCall, Buffer, Epilogue, F8E8M0FNU, GemmBackendConfig, Int8DotCall,
                                         ScaledDotCall)

        dev, sets = self.dev, []
        for i in range(2):
            ws = torch.empty(32 << 20, dtype=torch.int8, device=dev)       # the s8[] scratch XLA appends to the call
            if kind == "c3":
                g = torch.Generator(device=dev).manual_seed(3000 + i)
                a = torch.randint(-127, 128, (lm, lk), dtype=torch.int8, device=dev, generator=g)
                b = torch.randint(-127, 128, (lk, ln), dtype=torch.int8, device=dev, generator=g)
                rs = torch.rand(lm, device=dev, generator=g) * 0.019 + 0.001
                cs = torch.rand(ln, device=dev, generator=g) * 0.019 + 0.001
                d = torch.empty((lm, ln), dtype=torch.bfloat16, device=dev)
                ops, res = [a, b, rs, cs], [d, ws]
                if emit_s32:
                    res = [d, torch.empty((lm, ln), dtype=torch.int32, device=dev), ws]
                call = Int8DotCall(ops, res, selected_algorithm=kernel, emit_s32=emit_s32)
            elif kind == "mx":
                g = torch.Generator(device=dev).manual_seed(7000 + i)
                a = torch.randn((lm, lk), device=dev, generator=g).mul_(4).to(torch.float8_e4m3fn)
                b = torch.randn((ln, lk), device=dev, generator=g).mul_(4).to(torch.float8_e4m3fn)        # [n, k]: K minor on both
                sa = torch.randint(121, 132, (lm, lk // 32), dtype=torch.uint8, device=dev, generator=g)
                sb = torch.randint(121, 132, (ln, lk // 32), dtype=torch.uint8, device=dev, generator=g)
                d = torch.empty((lm, ln), dtype=torch.bfloat16, device=dev)
                ops, res = [a, b, sa, sb], [d, ws]
                call = BlockScaledDotCall([a, b, Buffer(F8E8M0FNU, tuple(sa.shape), sa.data_ptr()),
                                           Buffer(F8E8M0FNU, tuple(sb.shape), sb.data_ptr())], res)
            else:
                a, sa = self.f8_operand((lm, lk), 1000 * i + 1)           # A replicated (same seed on every rank) unless K-split
                b, sb = self.f8_operand((lk, ln), 1000 * i + 2 + 17 * self.rank)
                if kind == "c1":
                    bias = (torch.randn(ln, device=dev) * 0.02).bfloat16()
                    d = torch.empty((lm, ln), dtype=torch.float8_e4m3fn, device=dev)
                    amax = torch.zeros((), dtype=torch.float32, device=dev)
                    ops, res = [a, b, sa, sb, bias, torch.ones((), device=dev)], [d, amax, ws]
                    cfg = GemmBackendConfig(epilogue=Epilogue.BIAS_GELU, damax_output=True, selected_algorithm=kernel)
                else:
                    d = torch.empty((lm, ln), dtype=torch.bfloat16, device=dev)
                    ops, res = [a, b, sa, sb], [d, ws]
                    cfg = GemmBackendConfig(selected_algorithm=kernel)
                call = ScaledDotCall(ops, res, cfg)
            call.run(self.stream, self.local_rank)                        # instantiate + initialize + first execute
            sets.append((call, ops, res))
        torch.cuda.synchronize()
        assert self.lib.device_status() == 0
        return sets

    def c4_runner(self, sets, lm, ln, overlap, multicast=False):
        """How the K-split dot and its sum run on N > 1 ranks.  Returns (per-set callables or None, description)."""
        from xla_b200 import sharding

        args, dist = self.args, self.dist
        if overlap < 0:
            overlap = 2
        if overlap == 2:
            # Measured on 8192 x 28672 x 8192: 2 GPUs -- pull by the own tile's warp 0.73 ms, push 0.73, reducer warps 0.76;
            # 4 GPUs -- reducer warps 0.40, push 0.44, own tile's warp 0.51; 8 GPUs -- reducer warps 0.36, push 0.41, own tile's
            # warp 0.42 (one NCCL all-reduce behind the dot: 0.92 / 0.66 / 0.54).
            pull = args.pull if args.pull >= 0 else (1 if self.world == 2 else 2)
            multicast = multicast if multicast >= 0 else (1 if pull else 0)
            fused = [sharding.PeerReducedRowParallelScaledDot(lm, ln, device=self.dev, multicast=bool(multicast), pull=int(pull))
                     for _ in sets]
            runners = [(lambda f=f, ops=ops: f(ops[0], ops[1], ops[2], ops[3])) for f, (_, ops, _) in zip(fused, sets)]
            for i, f in enumerate(fused):                            # results now land in the symmetric buffers
                sets[i] = (sets[i][0], sets[i][1], [f.out] + list(sets[i][2][1:]))
            how = "formed inside the dot's kernel over peer memory (no collective launch"
            if pull:
                how += (", partials fetched by the rows' owner" if pull == 1 else ", partials fetched by the reducer warps of the rows' owner") + \
                    (" and added in the NVSwitch" if fused[0].in_switch_sum else " with peer loads")
            return runners, how + (", finished rows via NVSwitch multicast)" if fused[0].multicast else ")")
        if overlap == 1:
            group = None
            if args.nccl_ctas > 0:
                opts = dist.ProcessGroupNCCL.Options()
                opts.config.max_ctas = args.nccl_ctas
                opts.config.min_ctas = min(args.nccl_ctas, 4)
                group = dist.new_group(backend="nccl", pg_options=opts)
            runners = [sharding.OverlappedRowParallelScaledDot(ops[0], ops[1], ops[2], ops[3], res[0], rows_per_block=args.ar_rows,
                                                               gemm_ctas=args.gemm_ctas, group=group)
                       for _, ops, res in sets]
            return runners, (f"of {args.ar_rows}-row blocks overlapped with the dot ({args.gemm_ctas} SMs dot, "
                             f"{args.nccl_ctas} CTAs NCCL)")
        return None, "by one NCCL all-reduce behind the dot"

    def make_step(self, kind, sets, runners, stream=None):
        dist, world = self.dist, self.world

        def step(i):
            call, ops, res = sets[i & 1]
            if runners is not None:
                runners[i & 1]()
                return
            call.execute(stream if stream is not None else self.stream, self.local_rank)
            if kind == "c4" and world > 1:
                dist.all_reduce(res[0], op=dist.ReduceOp.SUM)        # bf16 partials, one NCCL all-reduce
        return step

    # ---- end to end with host buffers ---------------------------------------------------------
    def e2e(self, kind, sets, runners, steps):
        """Host buffers in pinned memory; every step copies ALL inputs to the device, runs the call through the
        FFI boundary and copies ALL results back.  The three legs run on three streams and the two device
        operand/result sets alternate, so step i+1's upload and step i-1's download overlap step i's kernel
        (PCIe is full duplex); every byte still moves inside the timed region."""
        torch, dev, dist, world = self.torch, self.dev, self.dist, self.world
        host_in = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in sets[0][1]]
        for hbuf, o in zip(host_in, sets[0][1]):
            hbuf.copy_(o)
        host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in sets[0][2][:-1]]   # the workspace is scratch, not a result
        h2d = sum(hb.numel() * hb.element_size() for hb in host_in)
        d2h = sum(hb.numel() * hb.element_size() for hb in host_out)
        e2e_steps = max(4, min(steps, 20))
        s_in, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        in_ready = [torch.cuda.Event() for _ in range(2)]
        computed = [torch.cuda.Event() for _ in range(2)]
        downloaded = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            j = i & 1
            call, ops, res = sets[j]
            with torch.cuda.stream(s_in):
                if i >= 2:
                    s_in.wait_event(computed[j])                 # set j's operands were last read by step i-2
                for hbuf, o in zip(host_in, ops):
                    o.copy_(hbuf, non_blocking=True)
                in_ready[j].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(in_ready[j])
                if i >= 2:
                    s_cmp.wait_event(downloaded[j])              # set j's results were last read by step i-2's download
                if runners is not None:
                    runners[j]()
                else:
                    call.execute(s_cmp.cuda_stream, self.local_rank)
                    if kind == "c4" and world > 1:
                        dist.all_reduce(res[0], op=dist.ReduceOp.SUM)
                computed[j].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed[j])
                for hbuf, o in zip(host_out, res[:-1]):
                    hbuf.copy_(o, non_blocking=True)
                downloaded[j].record(s_out)

        def e2e_run(n):
            for st in (s_in, s_cmp, s_out):
                st.wait_stream(torch.cuda.current_stream(dev))
            for i in range(n):
                e2e_step(i)
            for st in (s_in, s_cmp, s_out):
                torch.cuda.current_stream(dev).wait_stream(st)

        e2e_run(2)
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        torch.cuda.synchronize()
        ms = self.max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
        return {"ms_per_step": ms, "h2d_bytes_per_step": int(self.sum_over_ranks(h2d)),
                "d2h_bytes_per_step": int(self.sum_over_ranks(d2h)), "steps": e2e_steps}

    # ---- the other BASELINE configurations --------------------------------------------------
    def secondary(self, peaks):
        """Configs 2, 3 and (N > 1) 4 in the line the driver parses.  Each is timed like the headline: >= 3
        warm-up launches, two rotating operand sets larger than L2 together (config 3's are 2 x 67 MB),
        events on the launching stream, max over ranks."""
        import numpy as np

        torch, world = self.torch, self.world
        out = {}
        steps, warmup = max(3, self.args.secondary_steps), 5
        # config 2: decode shapes, W N-split over the ranks
        k, n = 8192, 28672
        c2 = {}
        for m in (16, 64, 128):
            lm, ln, lk = self.shard("c2", m, n, k)
            sets = self.make_sets("c2", lm, ln, lk)
            ms, _, launches = self.time_steps(self.make_step("c2", sets, None), steps, warmup)
            by = algorithmic_bytes("c2", m, n, k)
            sel = self.lib.select_kernel(lm, ln, lk)
            c2[f"m{m}"] = {"ms": ms, "value": by / ms / 1e6, "unit": "GB/s", "frac": by / world / ms / 1e6 / peaks["hbm_gbs"],
                           "frac_of_nominal_8000": by / world / ms / 1e6 / 8000.0,
                           "kernel": "skinny_gemm_kernel" if sel == 2 else "dense_gemm_kernel<fp8, single>",
                           "launches": int(self.sum_over_ranks(launches))}
            del sets
            torch.cuda.empty_cache()
        out["c2"] = {"workload": WORKLOAD_NAME["c2"], "n": n, "k": k, "n_gpus": world,
                     "parallelism": "single GPU" if world == 1 else f"N-split x{world}, no collective",
                     "peak": peaks["hbm_gbs"], "peak_source": f"MEASURED_PEAKS hbm_gbs ({peaks['source']})", **c2}
        # config 3: int8 + dequant (one GPU's worth of work per rank; reported for rank 0's device)
        m = n3 = k3 = 4096
        sets = self.make_sets("c3", m, n3, k3)
        ms, _, launches = self.time_steps(self.make_step("c3", sets, None), steps, warmup)
        check = self.make_sets("c3", m, n3, k3, emit_s32=True)
        call, ops, res = check[0]
        call.execute(self.stream, self.local_rank)
        torch.cuda.synchronize()
        from oracle import scaled_dot_oracle as o        # the checker: s32 block of rows against the CPU restatement
        rows = np.arange(0, m, 32)
        exp = o.dot_s8(ops[0][rows].cpu().numpy(), ops[1].cpu().numpy())
        got = res[1][rows].cpu().numpy()
        exp_bf16 = o.dequant_s32_to_bf16(exp, ops[2][rows].cpu().numpy(), ops[3].cpu().numpy())
        got_bf16 = res[0][rows].view(torch.int16).cpu().numpy().view(np.uint16)
        ops3 = 2.0 * m * n3 * k3
        out["c3"] = {"workload": WORKLOAD_NAME["c3"], "m": m, "n": n3, "k": k3, "ms": ms, "value": ops3 / ms / 1e9, "unit": "TOP/s",
                     "frac": ops3 / ms / 1e9 / (2.0 * peaks["bf16_tflops"]), "frac_of_nominal_4500": ops3 / ms / 1e9 / 4500.0,
                     "s32_mismatches": int((exp != got).sum()), "bf16_mismatches": int((exp_bf16 != got_bf16).sum()),
                     "checked": f"{len(rows)} rows x {n3} columns of the s32 accumulator and of the bf16 result against the CPU oracle",
                     "kernel": "dense_gemm_kernel<int8, pair>", "launches": int(launches), "n_gpus": 1}
        del sets, check
        torch.cuda.empty_cache()
        # MX block-scaled dot (one GPU's worth of work per rank; reported for rank 0's device)
        mm, mn, mk = DEFAULT_DIMS["mx"]
        sets = self.make_sets("mx", mm, mn, mk)
        ms, _, launches = self.time_steps(self.make_step("mx", sets, None), min(50, steps), 5)
        call, ops, res = sets[0]
        call.execute(self.stream, self.local_rank)
        torch.cuda.synchronize()
        rows = np.arange(5, mm, mm // 16)
        a_np, b_np = ops[0][rows].view(torch.uint8).cpu().numpy(), ops[1].view(torch.uint8).cpu().numpy()
        sa_np, sb_np = ops[2][rows].cpu().numpy(), ops[3].cpu().numpy()
        exp = o.bf16_bits_to_f32(o.block_scaled_dot(a_np, b_np, sa_np, sb_np, out_dtype=o.BF16))
        got = res[0][rows].float().cpu().numpy()
        # per element: f32 summation-order slack 2^-16 of sum |a_k b_k|, plus one bf16 step
        slack = np.matmul(np.abs(o.mx_dequantize(a_np, sa_np)), np.abs(o.mx_dequantize(b_np, sb_np)).T) * 2.0 ** -16 + np.abs(exp) * 2.0 ** -7
        flops = 2.0 * mm * mn * mk
        out["mx"] = {"workload": WORKLOAD_NAME["mx"], "m": mm, "n": mn, "k": mk, "ms": ms, "value": flops / ms / 1e9, "unit": "TFLOP/s",
                     "frac": flops / ms / 1e9 / (2.0 * peaks["bf16_tflops"]), "frac_of_nominal_4500": flops / ms / 1e9 / 4500.0,
                     "mismatches": int((np.abs(got - exp) > slack).sum()),
                     "checked": f"{len(rows)} rows x {mn} columns against the CPU oracle, |diff| <= 2^-16 sum|a b| + one bf16 step",
                     "kernel": "mx_gemm_kernel", "launches": int(launches), "n_gpus": 1}
        del sets
        torch.cuda.empty_cache()
        # config 4: K-split + sum across ranks
        if world > 1:
            m4, n4, k4 = DEFAULT_DIMS["c4"]
            lm, ln, lk = self.shard("c4", m4, n4, k4)
            sets = self.make_sets("c4", lm, ln, lk)
            runners, how = self.c4_runner(sets, lm, ln, self.args.overlap, self.args.multicast)
            ms, _, launches = self.time_steps(self.make_step("c4", sets, runners), min(50, steps), 5)
            flops = 2.0 * m4 * n4 * k4
            fp8_peak = 2.0 * peaks["bf16_tflops"]
            t_tensor = flops / world / (fp8_peak * 1e9)
            link_bytes = c4_link_bytes(world, m4, n4, "NVSwitch" in how and "fetched" in how)
            t_link = link_bytes / 770e9 * 1e3
            out["c4"] = {"workload": WORKLOAD_NAME["c4"], "m": m4, "n": n4, "k": k4, "n_gpus": world, "ms": ms,
                         "value": flops / ms / 1e9, "unit": "TFLOP/s", "sum": how,
                         "roofline": {"bound": "tensor" if t_tensor >= t_link else "nvlink", "tensor_ms": t_tensor, "nvlink_ms": t_link,
                                      "nvlink_bytes_per_rank": link_bytes, "target_ms": max(t_tensor, t_link),
                                      "frac": max(t_tensor, t_link) / ms,
                                      "peak_source": "2 x bf16_tflops burst; 770 GB/s measured peer copy per direction"},
                         "launches": int(self.sum_over_ranks(launches))}
            del sets, runners
            torch.cuda.empty_cache()
        return out

    def counters(self, grid_ctas):
        """The kernels' own wait counters of the last dense launch (tuning build only)."""
        import ctypes as C

        from xla_b200 import _native

        fn = getattr(_native.product, "b200sd_debug_read_timing", None)
        if fn is None:
            return {"unavailable": "the loaded library is the product build; load the tuning build through B200SD_LIBRARY"}
        slots = 24
        n = slots * grid_ctas
        buf = (C.c_ulonglong * n)()
        fn(buf, n)
        rows = [buf[slots * i:slots * i + slots] for i in range(grid_ctas)]
        rows = [r for r in rows if r[8] > 0]
        leaders = [r for r in rows if r[2] > 0]
        if not leaders:
            return {"unavailable": "no counters were written: set B200SD_TIMING=1"}
        mean = lambda j, src: sum(r[j] for r in src) / len(src)     # noqa: E731
        total = mean(2, leaders)
        t0 = min(r[8] for r in rows)
        rel = lambda j, src, f: (f(r[j] for r in src if r[j] > 0) - t0) / 1e3     # noqa: E731  (us after the first CTA's entry)
        return {"ctas": len(rows), "ctas_with_issuer": len(leaders), "issuer_cycles": total,
                "issuer_wait_operands_frac": mean(0, leaders) / total,
                "issuer_wait_accumulator_frac": mean(1, leaders) / total, "issuer_wait_preload_frac": mean(7, leaders) / total,
                "producer_wait_stage_frac": mean(3, rows) / total,
                "epilogue_wait_frac": mean(5, rows) / total, "epilogue_busy_frac": mean(6, rows) / total,
                "epilogue_busy_split": {"tmem_load_wait": mean(16, rows) / max(1.0, mean(6, rows)), "arithmetic": mean(17, rows) / max(1.0, mean(6, rows)),
                                        "stage_flush": mean(18, rows) / max(1.0, mean(6, rows))},
                "issuer_ns_min_mean_max": [min(r[4] for r in leaders), mean(4, leaders), max(r[4] for r in leaders)],
                "sm_mhz_in_kernel": 1e3 * total / mean(4, leaders),
                "timeline_us": {"last_cta_entry": rel(8, rows, max), "setup_done_max": rel(9, rows, max),
                                "first_operands_min": rel(10, leaders, min), "first_operands_max": rel(10, leaders, max),
                                "issuer_done_min": rel(11, leaders, min), "issuer_done_max": rel(11, leaders, max),
                                "last_accumulator_complete_max": rel(14, rows, max), "last_tile_stored_max": rel(15, rows, max),
                                "epilogue_done_max": rel(12, rows, max), "cta_exit_max": rel(13, rows, max)}}


def gpu_arm(args):
    B = Bench(args)
    torch, world, rank = B.torch, B.world, B.rank
    kind = args.workload
    m, n, k = workload_dims(args)
    steps, warmup = args.steps, max(3, args.warmup)
    lm, ln, lk = B.shard(kind, m, n, k)
    sets = B.make_sets(kind, lm, ln, lk, kernel=args.kernel)
    runners, c4_how = (B.c4_runner(sets, lm, ln, args.overlap, args.multicast) if (kind == "c4" and world > 1) else (None, ""))
    step = B.make_step(kind, sets, runners)
    ms, clocks, launches = B.time_steps(step, steps, warmup, sample_clocks=True)
    launches_total = int(B.sum_over_ranks(launches))
    counters = B.counters(2 * 74 if lm > 128 else 148) if args.counters else None

    e2e = None if args.no_e2e else B.e2e(kind, sets, runners, steps)

    flops = 2.0 * m * n * k
    peaks = measured_peaks()
    # The other configurations come BEFORE the seconds-long sustained run: that run drives the GPU into its power
    # cap (SM clock about 1.2 GHz), and a bandwidth-bound decode launch timed right behind it is 20 % slower than
    # on a GPU at its normal clocks.
    secondary = None if (args.no_secondary or kind != "c1" or (args.m or args.n or args.k)) else B.secondary(peaks)
    sustained = None
    if not args.no_sustained and kind in ("c1", "plain", "c3", "mx"):
        n_steps = max(steps, int(math.ceil(args.sustained_seconds * 1e3 / ms)))
        s_ms, s_clocks, _ = B.time_steps(step, n_steps, 3, sample_clocks=True)
        rate = flops / world / s_ms / 1e9
        sustained = {"steps": n_steps, "seconds": n_steps * s_ms / 1e3, "ms_per_step": s_ms, "value": flops / s_ms / 1e9,
                     "unit": "TFLOP/s" if kind != "c3" else "TOP/s", "clocks": s_clocks}
        if s_clocks and s_clocks.get("sm_mhz"):
            sustained["frac_of_tensor_rate_at_median_clock"] = rate * 1e12 / (148 * FLOP_PER_CLK_PER_SM * s_clocks["sm_mhz"] * 1e6)
        sustained["frac_of_2x_bf16_sustained"] = flops / world / sustained["ms_per_step"] / 1e9 / (2.0 * peaks["bf16_tflops_sustained"])
    del sets, runners, step
    torch.cuda.empty_cache()
    if rank != 0:
        if world > 1:
            B.dist.destroy_process_group()
        return

    # ---- report ------------------------------------------------------------------------------
    if kind == "c2":
        algo_bytes = algorithmic_bytes("c2", m, n, k)
        value, unit = algo_bytes / ms / 1e6, "GB/s"
        roof = {"bound": "hbm", "achieved": algo_bytes / world / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "peak_source": f"MEASURED_PEAKS hbm_gbs ({peaks['source']})"}
    else:
        value, unit = flops / ms / 1e9, "TFLOP/s"
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": flops / world / ms / 1e9, "peak": fp8_peak, "unit": "TFLOP/s",
                "peak_source": f"2 x MEASURED_PEAKS bf16_tflops burst ({peaks['source']}); 8-bit tensor rate is twice bf16",
                "frac_of_nominal_4500": flops / world / ms / 1e9 / 4500.0,
                "frac_of_sustained": flops / world / ms / 1e9 / (2.0 * peaks["bf16_tflops_sustained"]),
                "algorithmic_bytes": algorithmic_bytes(kind, m, n, k) / world}
        if clocks and clocks.get("sm_mhz"):
            roof["frac_of_tensor_rate_at_median_clock"] = flops / world / ms * 1e3 / (148 * FLOP_PER_CLK_PER_SM * clocks["sm_mhz"] * 1e6)
    roof["frac"] = roof["achieved"] / roof["peak"]
    if kind == "c4" and world > 1:
        # A dot followed by its sum across the ranks: the target time is the slower of the dot at the measured
        # tensor peak and the bytes every rank must send (reduce-scatter + all-gather of the bf16 [m, n] result)
        # at the measured peer-copy rate of this pool, 770 GB/s per direction.
        t_tensor_ms = flops / world / (fp8_peak * 1e9)
        link_bytes = c4_link_bytes(world, m, n, "NVSwitch" in c4_how and "fetched" in c4_how)
        t_link_ms = link_bytes / 770e9 * 1e3
        roof["fused"] = {"bound": "tensor" if t_tensor_ms >= t_link_ms else "nvlink", "tensor_ms": t_tensor_ms, "nvlink_ms": t_link_ms,
                         "nvlink_bytes_per_rank": link_bytes, "target_ms": max(t_tensor_ms, t_link_ms),
                         "frac": max(t_tensor_ms, t_link_ms) / ms}
    roof["traffic"] = NCU_DRAM_BYTES_PER_LAUNCH.get((kind, m, n, k)) if world == 1 else None
    c2_kernel = args.kernel or B.lib.select_kernel(lm, ln, lk)
    roof["kernel"] = {"c2": "skinny_gemm_kernel" if c2_kernel == 2 else "dense_gemm_kernel<fp8, single>",
                      "c3": "dense_gemm_kernel<int8, pair>", "mx": "mx_gemm_kernel"}.get(kind, "dense_gemm_kernel<fp8, pair>")
    parallelism = ("single GPU" if world == 1 else
                   (f"K-split x{world}, sum {c4_how}" if kind == "c4" else f"N-split x{world}, no collective"))
    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if kind == "c3" else "f8e4m3fn", "data": "synthetic",
        "config": config_block(kind, m, n, k, parallelism),
        "clocks": clocks, "gpu_launches": launches_total, "roofline": roof,
    }
    if e2e is not None:
        units = algorithmic_bytes("c2", m, n, k) / 1e6 if kind == "c2" else flops / 1e9
        line["e2e"] = {"value": units / e2e["ms_per_step"], "unit": unit, "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                       "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "ms_per_step": e2e["ms_per_step"],
                       "steps": e2e["steps"]}
    if sustained is not None:
        line["sustained"] = sustained
    if secondary is not None:
        line["secondary"] = secondary
    if counters is not None:
        line["counters"] = counters
    if world == 1 and not args.no_cpu_baseline and kind != "mx":
        line["cpu_baseline"] = cpu_arm((kind, (m, n, k)), budget_s=20.0, steps=3, warmup=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        B.dist.destroy_process_group()


def reference_arm(args):
    """The reference arithmetic on the host cores, same workload, same line.  Under torchrun only rank 0 works;
    the thread count is set here (torchrun exports OMP_NUM_THREADS=1, which would otherwise serialise BLAS)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind = args.workload
    m, n, k = workload_dims(args)
    steps, warmup = args.steps, max(3, args.warmup)
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    res = cpu_arm((kind, (m, n, k)), budget_s=120.0, steps=steps, warmup=warmup)
    parallelism = ("single GPU" if world == 1 else
                   (f"K-split x{world}" if kind == "c4" else f"N-split x{world}, no collective"))
    cfg = config_block(kind, m, n, k, parallelism)
    cfg["note"] = ("reference arm: XLA's CPU backend is not buildable offline; the oracle port of the same HLO runs on the "
                   "host cores of rank 0, each step over the bounded sample named in cpu_baseline.sample")
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": res["unit"],
        "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if kind == "c3" else "f8e4m3fn", "data": "synthetic",
        "config": cfg,
        "cpu_baseline": {"value": res["value"], "unit": res["unit"], "cores": res["cores"], "kind": "port",
                         "sample": res["sample"]},
        "e2e": {"value": res["value"], "unit": res["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cublaslt_arm(args):
    """The library the reference's GPU path calls (cuBLASLt, reached here through torch._scaled_mm /
    torch._int_mm), timed on one GPU on the same shapes for a side-by-side note.  It is not the
    product and not the reference arm: it has no GELU, no amax and no fused dequantisation, so
    config 1 runs as dot + bias -> bf16 and config 3 as the bare s8 dot -> s32."""
    import torch

    kind = args.workload
    m, n, k = workload_dims(args)
    dev = torch.device("cuda", 0)
    steps, warmup = args.steps, max(3, args.warmup)
    sets = []
    for i in range(2):
        g = torch.Generator(device=dev).manual_seed(1000 * i + 1)
        if kind == "c3":
            sets.append((torch.randint(-127, 128, (m, k), dtype=torch.int8, device=dev, generator=g),
                         torch.randint(-127, 128, (k, n), dtype=torch.int8, device=dev, generator=g), None))
        elif kind == "mx":
            # cuBLASLt wants each scale tensor as 128-row x 4-column blocks stored as 32 x 16 bytes.
            def blocked(s):
                r, c = s.shape
                t = s.view(r // 128, 128, c // 4, 4).permute(0, 2, 1, 3).reshape(-1, 4, 32, 4).transpose(1, 2)
                return t.reshape(-1).contiguous().view(torch.float8_e8m0fnu)
            a = torch.randn((m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
            bt = torch.randn((n, k), device=dev, generator=g).to(torch.float8_e4m3fn)
            sa = torch.randint(121, 132, (m, k // 32), dtype=torch.uint8, device=dev, generator=g)
            sb = torch.randint(121, 132, (n, k // 32), dtype=torch.uint8, device=dev, generator=g)
            sets.append((a, bt, (blocked(sa), blocked(sb))))
        else:
            a = torch.randn((m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
            bt = torch.randn((n, k), device=dev, generator=g).to(torch.float8_e4m3fn)     # column-major B, as cuBLASLt wants it
            sets.append((a, bt, (torch.randn(n, device=dev, generator=g) * 0.02).bfloat16() if kind == "c1" else None))
    one = torch.ones((), device=dev)

    def step(i):
        a, b, bias = sets[i & 1]
        if kind == "c3":
            torch._int_mm(a, b)
        elif kind == "mx":
            torch._scaled_mm(a, b.t(), scale_a=bias[0], scale_b=bias[1], out_dtype=torch.bfloat16)
        else:
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, bias=bias, out_dtype=torch.bfloat16, use_fast_accum=True)

    def timed(n_steps):
        for i in range(warmup):
            step(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n_steps):
            step(i)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n_steps

    ms = timed(steps)
    if kind == "c2":
        value, unit, per_ms = algorithmic_bytes("c2", m, n, k) / ms / 1e6, "GB/s", algorithmic_bytes("c2", m, n, k) / 1e6
    else:
        value, unit, per_ms = 2.0 * m * n * k / ms / 1e9, "TFLOP/s", 2.0 * m * n * k / 1e9
    line = {"impl": "cublaslt", "metric": METRIC, "value": value, "unit": unit, "n_gpus": 1, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "config": {"workload": kind, "m": m, "n": n, "k": k,
                       "note": "torch._scaled_mm / torch._int_mm (cuBLASLt); no GELU, amax or dequantisation fused"}}
    if not args.no_sustained and kind != "c2":
        n_steps = max(steps, int(math.ceil(args.sustained_seconds * 1e3 / ms)))
        s_ms = timed(n_steps)
        line["sustained"] = {"steps": n_steps, "ms_per_step": s_ms, "value": per_ms / s_ms, "unit": unit}
    print(json.dumps(line), flush=True)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        # All host threads, whatever the launcher exported: set before NumPy / BLAS are loaded.
        for var in ("OMP_NUM_THREADS", "OPENBLAS_NUM_THREADS", "MKL_NUM_THREADS"):
            os.environ[var] = str(host_threads())
    if a.impl == "cublaslt":
        cublaslt_arm(a)
    elif a.impl == "reference":
        reference_arm(a)
    else:
        gpu_arm(a)
