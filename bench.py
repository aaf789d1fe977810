#!/usr/bin/env python
"""Benchmark of the quantized scaled-dot hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference|cublaslt] [--workload c1|...]

A "step" is one pass of the hot path over one batch of synthetic input: one custom call through
the XLA FFI boundary of libb200_scaled_dot.so.  Default workload `c1` is BASELINE config 1:
M=N=K=8192 e4m3fn operands (values from N(0,1) scaled to amax 448), per-tensor f32 scales, bf16
bias ~N(0,0.02), GELU, scaled e4m3fn output (out_scale 1.0) and an f32 amax.  On N>1 GPUs B, bias
and D are N-split column-parallel (A replicated) with no collective: total work is fixed, so
scaling is "strong".  Other workloads (plain, c2 decode, c3 int8, c4 row-parallel + all-reduce)
exist for the profiles and the design notes; `--m/--n/--k` shrink a workload for ncu captures.

Timing: W (>=3) untimed warm-up steps, then exactly K steps between two CUDA events on the
launching stream, bracketed by barrier + synchronize; max over ranks.  Two operand/result sets
are used alternately and together exceed the 126 MB L2, so no step finds its inputs in cache.
The JSON line also carries: `e2e` (same call with HOST buffers: pinned host -> device copies of
every input and device -> host copies of every result inside the timed region, the upload, the
call and the download of consecutive steps overlapped on three streams), `roofline` for the
dominant kernel, `cpu_baseline` (the CPU oracle timed on a bounded sample), SM clocks sampled
through NVML during the timed region, and the number of kernels launched.

`--impl cublaslt` times the library the reference's GPU path calls on the same shapes (one GPU),
for the side-by-side note under profiles/.  `--impl reference` times the reference arithmetic on the host cores instead (XLA's own CPU
backend cannot be built offline, so this is the NumPy/BLAS port in oracle/), on a bounded sample of
the same workload, and prints the same line with "impl": "reference".
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FP8 scaled-dot TFLOP/s at 8192^3 per B200 and at 2/4/8 GPUs; % of FP8 dense peak"


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=100)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--impl", default="ours", choices=["ours", "reference", "cublaslt"])
    p.add_argument("--workload", default="c1", choices=["c1", "plain", "c2", "c3", "c4"])
    p.add_argument("--overlap", type=int, default=-1, help="c4, N>1: 2 = sum formed inside the dot's kernel over peer memory, 1 = NCCL all-reduce of finished row blocks "
                   "on a second stream, 0 = dot then one NCCL all-reduce; default: 2 up to 4 GPUs, 0 beyond (measured faster)")
    p.add_argument("--multicast", type=int, default=0, help="c4 fused: write finished rows through the NVSwitch multicast mapping")
    p.add_argument("--ar-rows", type=int, default=2048, help="c4 overlap: rows of D per all-reduce")
    p.add_argument("--gemm-ctas", type=int, default=132, help="c4 overlap: SMs the dot may occupy")
    p.add_argument("--nccl-ctas", type=int, default=16, help="c4 overlap: CTAs the collective may use (0 = NCCL's choice)")
    p.add_argument("--m", type=int, default=0)
    p.add_argument("--n", type=int, default=0)
    p.add_argument("--k", type=int, default=0)
    p.add_argument("--kernel", type=int, default=0, help="0 auto, 1 dense, 2 split-K, 3 dense single-CTA, 4 dense CTA pair, 5 CTA pair with a stream-K tail")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-cpu-baseline", action="store_true")
    return p.parse_args()


def workload_dims(args):
    dflt = {"c1": (8192, 8192, 8192), "plain": (8192, 8192, 8192), "c2": (64, 28672, 8192),
            "c3": (4096, 4096, 4096), "c4": (8192, 8192, 28672)}[args.workload]
    return (args.m or dflt[0], args.n or dflt[1], args.k or dflt[2])


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# --------------------------------------------------------------------------------------------- CPU arm
def cpu_sample_step(wl, m_rows, n_cols, seed=0):
    """One pass of the oracle over an [m_rows, K] x [K, n_cols] sample of the workload.  Returns
    (seconds, algorithmic units) where units are flops (c1/plain/c3/c4) or bytes (c2)."""
    import numpy as np
    from oracle import scaled_dot_oracle as o

    kind, (m, n, k) = wl
    rng = np.random.default_rng(seed)
    if kind == "c3":
        a = rng.integers(-127, 128, size=(m_rows, k), dtype=np.int8)
        b = rng.integers(-127, 128, size=(k, n_cols), dtype=np.int8)
        rs = rng.uniform(0.001, 0.02, size=m_rows).astype(np.float32)
        cs = rng.uniform(0.001, 0.02, size=n_cols).astype(np.float32)
        t0 = time.perf_counter()
        o.dequant_s32_to_bf16(o.dot_s8(a, b), rs, cs)
        return time.perf_counter() - t0, 2.0 * m_rows * n_cols * k
    a = rng.integers(0, 0x7F, size=(m_rows, k), dtype=np.uint8)       # finite e4m3 code points
    b = rng.integers(0, 0x7F, size=(k, n_cols), dtype=np.uint8)
    bias = rng.standard_normal(n_cols).astype(np.float32) * np.float32(0.02)
    t0 = time.perf_counter()
    if kind == "c1":
        o.scaled_dot_f8(a, b, 0.01, 0.01, bias=bias, epilogue=o.EPI_BIAS_GELU, d_scale=1.0, out_dtype=o.F8E4M3FN,
                        want_amax=True)
    else:
        o.scaled_dot_f8(a, b, 0.01, 0.01, out_dtype=o.BF16)
    dt = time.perf_counter() - t0
    units = (k * n_cols + m_rows * k + 2 * m_rows * n_cols) if kind == "c2" else 2.0 * m_rows * n_cols * k
    return dt, units


def cpu_arm(wl, budget_s, steps, warmup):
    """Times `steps` oracle passes on a sample sized so that everything fits in `budget_s`."""
    import torch

    kind, (m, n, k) = wl
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    m_rows, n_cols = min(m, 64), min(n, 1024)
    dt, _ = cpu_sample_step(wl, m_rows, n_cols)           # calibration (also warms the BLAS threads)
    per_step_budget = budget_s / max(1, steps + warmup)
    while dt * 3.0 < per_step_budget and (m_rows < m or n_cols < n):
        if n_cols < n:
            n_cols = min(n, n_cols * 2)
        else:
            m_rows = min(m, m_rows * 2)
        dt, _ = cpu_sample_step(wl, m_rows, n_cols)
    for _ in range(min(warmup, 2)):
        cpu_sample_step(wl, m_rows, n_cols)
    total_t, total_u = 0.0, 0.0
    for i in range(steps):
        t, u = cpu_sample_step(wl, m_rows, n_cols, seed=i)
        total_t += t
        total_u += u
    scale = 1e-9 if kind == "c2" else 1e-12
    return {"value": total_u / total_t * scale, "unit": "GB/s" if kind == "c2" else "TFLOP/s", "cores": cores,
            "kind": "port", "ms_per_step": 1e3 * total_t / steps,
            "sample": f"{steps} passes of the NumPy/BLAS oracle over A[{m_rows},{k}] x B[{k},{n_cols}] "
                      f"(a {m_rows}x{n_cols} block of the {m}x{n} output), dequantise + dot + epilogue"}


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
def gpu_arm(args):
    import torch
    import torch.distributed as dist

    import xla_b200
    from xla_b200 import sharding
    from xla_b200.scaled_dot import Epilogue, GemmBackendConfig, Int8DotCall, ScaledDotCall

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    kind = args.workload
    m, n, k = workload_dims(args)
    steps, warmup = args.steps, max(3, args.warmup)
    stream = torch.cuda.current_stream().cuda_stream

    # ---- this rank's shard of the problem ---------------------------------------------------
    if kind == "c4":
        ks = sharding.row_parallel_slices(k, world, rank)
        lm, ln, lk = m, n, ks.stop - ks.start
    else:
        cols = sharding.column_parallel_slices(n, world, rank)
        lm, ln, lk = m, cols.stop - cols.start, k

    def f8_operand(shape, seed):
        g = torch.Generator(device=dev).manual_seed(seed)
        v = torch.randn(shape, device=dev, generator=g)
        s = (v.abs().max() / 448.0).reshape(()).float()
        return (v / s).to(torch.float8_e4m3fn), s

    sets, host_sets = [], []
    for i in range(2):                                           # two rotating operand/result sets
        if kind == "c3":
            g = torch.Generator(device=dev).manual_seed(3000 + i)
            a = torch.randint(-127, 128, (lm, lk), dtype=torch.int8, device=dev, generator=g)
            b = torch.randint(-127, 128, (lk, ln), dtype=torch.int8, device=dev, generator=g)
            rs = torch.rand(lm, device=dev, generator=g) * 0.019 + 0.001
            cs = torch.rand(ln, device=dev, generator=g) * 0.019 + 0.001
            d = torch.empty((lm, ln), dtype=torch.bfloat16, device=dev)
            ws = torch.empty(32 << 20, dtype=torch.int8, device=dev)   # the s8[] scratch XLA appends to the call
            ops, res = [a, b, rs, cs], [d, ws]
            call = Int8DotCall(ops, res, selected_algorithm=args.kernel)
        else:
            a, sa = f8_operand((lm, lk), 1000 * i + 1)           # A replicated (same seed on every rank) unless K-split
            b, sb = f8_operand((lk, ln), 1000 * i + 2 + 17 * rank)
            ws = torch.empty(32 << 20, dtype=torch.int8, device=dev)
            if kind == "c1":
                bias = (torch.randn(ln, device=dev) * 0.02).bfloat16()
                d = torch.empty((lm, ln), dtype=torch.float8_e4m3fn, device=dev)
                amax = torch.zeros((), dtype=torch.float32, device=dev)
                ops, res = [a, b, sa, sb, bias, torch.ones((), device=dev)], [d, amax, ws]
                cfg = GemmBackendConfig(epilogue=Epilogue.BIAS_GELU, damax_output=True, selected_algorithm=args.kernel)
            else:
                d = torch.empty((lm, ln), dtype=torch.bfloat16, device=dev)
                ops, res = [a, b, sa, sb], [d, ws]
                cfg = GemmBackendConfig(selected_algorithm=args.kernel)
            call = ScaledDotCall(ops, res, cfg)
        call.run(stream, local_rank)                             # instantiate + initialize + first execute
        sets.append((call, ops, res))
    torch.cuda.synchronize()
    assert xla_b200.device_status() == 0

    overlapped = None
    if args.overlap < 0:
        args.overlap = 2 if world <= 4 else 0
    if kind == "c4" and world > 1 and args.overlap == 2:
        fused = [sharding.PeerReducedRowParallelScaledDot(lm, ln, device=dev, multicast=bool(args.multicast)) for _ in sets]
        overlapped = [(lambda f=f, ops=ops: f(ops[0], ops[1], ops[2], ops[3])) for f, (_, ops, _) in zip(fused, sets)]
        for i, f in enumerate(fused):                            # results now land in the symmetric buffers
            sets[i] = (sets[i][0], sets[i][1], [f.out] + list(sets[i][2][1:]))
    elif kind == "c4" and world > 1 and args.overlap == 1:
        group = None
        if args.nccl_ctas > 0:
            opts = dist.ProcessGroupNCCL.Options()
            opts.config.max_ctas = args.nccl_ctas
            opts.config.min_ctas = min(args.nccl_ctas, 4)
            group = dist.new_group(backend="nccl", pg_options=opts)
        overlapped = [sharding.OverlappedRowParallelScaledDot(ops[0], ops[1], ops[2], ops[3], res[0], rows_per_block=args.ar_rows,
                                                              gemm_ctas=args.gemm_ctas, group=group)
                      for _, ops, res in sets]

    def step(i):
        call, ops, res = sets[i & 1]
        if overlapped is not None:
            overlapped[i & 1]()                                  # dot + row-block all-reduces on a second stream
            return
        call.execute(stream, local_rank)
        if kind == "c4" and world > 1:
            dist.all_reduce(res[0], op=dist.ReduceOp.SUM)        # bf16 partials, one NCCL all-reduce

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches0 = xla_b200.launch_count()
    sampler = ClockSampler(local_rank)
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.finish()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    launches = xla_b200.launch_count() - launches0
    ms = e0.elapsed_time(e1) / steps
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    assert xla_b200.device_status() == 0

    # ---- end to end with host buffers ----------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        # Host buffers in pinned memory; every step copies ALL inputs to the device, runs the call through the
        # FFI boundary and copies ALL results back.  The three legs run on three streams and the two device
        # operand/result sets alternate, so step i+1's upload and step i-1's download overlap step i's kernel
        # (PCIe is full duplex); every byte still moves inside the timed region.
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
                if overlapped is not None:
                    overlapped[j]()
                else:
                    call.execute(s_cmp.cuda_stream, local_rank)
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
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
        hd = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(hd, op=dist.ReduceOp.SUM)
        e2e = {"ms_per_step": e2e_ms, "h2d_bytes_per_step": int(hd[0].item()), "d2h_bytes_per_step": int(hd[1].item()),
               "steps": e2e_steps}

    launches_t = torch.tensor([launches], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(launches_t, op=dist.ReduceOp.SUM)
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- report ------------------------------------------------------------------------------
    peaks = measured_peaks()
    flops = 2.0 * m * n * k
    if kind == "c2":
        algo_bytes = k * n + m * k + 2 * m * n
        value, unit = algo_bytes / ms / 1e6, "GB/s"
        per_launch = algo_bytes / world
        roof = {"bound": "hbm", "achieved": per_launch / ms / 1e6, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "peak_source": f"MEASURED_PEAKS hbm_gbs ({peaks['source']})"}
    else:
        value, unit = flops / ms / 1e9, "TFLOP/s"
        fp8_peak = 2.0 * peaks["bf16_tflops"]
        roof = {"bound": "tensor", "achieved": flops / world / ms / 1e9, "peak": fp8_peak, "unit": "TFLOP/s",
                "peak_source": f"2 x MEASURED_PEAKS bf16_tflops burst ({peaks['source']}); 8-bit tensor rate is twice bf16",
                "frac_of_nominal_4500": flops / world / ms / 1e9 / 4500.0,
                "frac_of_sustained": flops / world / ms / 1e9 / (2.0 * peaks["bf16_tflops_sustained"])}
    roof["frac"] = roof["achieved"] / roof["peak"]
    if kind == "c4" and world > 1:
        # A dot followed by its sum across the ranks: the target time is the slower of the dot at the measured
        # tensor peak and the bytes every rank must send (reduce-scatter + all-gather of the bf16 [m, n] result)
        # at the measured peer-copy rate of this pool, 770 GB/s per direction.
        t_tensor_ms = flops / world / (fp8_peak * 1e9)
        link_bytes = 2.0 * (world - 1) / world * m * n * 2
        t_link_ms = link_bytes / 770e9 * 1e3
        roof["fused"] = {"bound": "tensor" if t_tensor_ms >= t_link_ms else "nvlink", "tensor_ms": t_tensor_ms, "nvlink_ms": t_link_ms,
                         "nvlink_bytes_per_rank": link_bytes, "target_ms": max(t_tensor_ms, t_link_ms),
                         "frac": max(t_tensor_ms, t_link_ms) / ms}
    # dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
    # (single GPU, default sizes only; bytes).
    measured_traffic = {("c1", 8192, 8192, 8192): 396.0e6, ("c2", 64, 28672, 8192): 240.2e6,
                        ("c3", 4096, 4096, 4096): 33.8e6}
    roof["traffic"] = measured_traffic.get((kind, m, n, k)) if world == 1 else None
    c2_kernel = args.kernel or xla_b200.select_kernel(lm, ln, lk)
    roof["kernel"] = {"c2": "skinny_gemm_kernel" if c2_kernel == 2 else "dense_gemm_kernel<fp8, single>",
                      "c3": "dense_gemm_kernel<int8>"}.get(kind, "dense_gemm_kernel<fp8>")
    if kind == "c2" and c2_kernel != 2:   # the dense single-CTA kernel's capture (profiles/dense_gemm_single_fp8_c2_m64.md)
        roof["traffic"] = 240.06e6 if (world == 1 and (m, n, k) == (64, 28672, 8192)) else None
    line = {
        "metric": METRIC, "value": value, "unit": unit, "n_gpus": world, "steps": steps, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if kind == "c3" else "f8e4m3fn", "data": "synthetic",
        "config": {"workload": {"c1": "config 1: dense FP8 linear 8192^3, bias + GELU + scaled e4m3 output + amax",
                                "plain": "scaled dot, bf16 output, no epilogue",
                                "c2": "config 2: decode-shape FP8 dot, bf16 output",
                                "c3": "config 3: int8 dot + per-row x per-column dequant to bf16",
                                "c4": "config 4: row-parallel FP8 dot + one NCCL all-reduce of bf16 partials"}[kind],
                   "m": m, "n": n, "k": k,
                   "parallelism": ("single GPU" if world == 1 else
                                   (f"K-split x{world} + all-reduce" + ({2: " formed inside the dot's kernel over peer memory (no collective launch" +
                                        (", finished rows via NVSwitch multicast)" if args.multicast else ")"),
                                     1: f" of {args.ar_rows}-row blocks overlapped with the dot ({args.gemm_ctas} SMs dot, "
                                        f"{args.nccl_ctas} CTAs NCCL)"}.get(args.overlap, "") if overlapped is not None else "")
                                    if kind == "c4" else f"N-split x{world}, no collective")),
                   "l2": "two operand/result sets used alternately; together larger than the 126 MB L2"},
        "clocks": clocks, "gpu_launches": int(launches_t.item()), "roofline": roof,
    }
    if e2e is not None:
        units = (k * n + m * k + 2 * m * n) / 1e6 if kind == "c2" else flops / 1e9
        line["e2e"] = {"value": units / e2e["ms_per_step"], "unit": unit, "h2d_bytes_per_step": e2e["h2d_bytes_per_step"],
                       "d2h_bytes_per_step": e2e["d2h_bytes_per_step"], "ms_per_step": e2e["ms_per_step"],
                       "steps": e2e["steps"]}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_arm((kind, (m, n, k)), budget_s=20.0, steps=3, warmup=1)
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    kind = args.workload
    m, n, k = workload_dims(args)
    steps, warmup = args.steps, max(1, min(args.warmup, 3))
    res = cpu_arm((kind, (m, n, k)), budget_s=120.0, steps=steps, warmup=warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": res["value"], "unit": res["unit"],
        "n_gpus": int(os.environ.get("WORLD_SIZE", str(args.gpus))), "steps": steps, "warmup": warmup,
        "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "s8" if kind == "c3" else "f8e4m3fn", "data": "synthetic",
        "config": {"workload": kind, "m": m, "n": n, "k": k,
                   "note": "XLA's CPU backend is not buildable offline; this is the oracle port of the same HLO on host cores"},
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
        else:
            a = torch.randn((m, k), device=dev, generator=g).to(torch.float8_e4m3fn)
            bt = torch.randn((n, k), device=dev, generator=g).to(torch.float8_e4m3fn)     # column-major B, as cuBLASLt wants it
            sets.append((a, bt, (torch.randn(n, device=dev, generator=g) * 0.02).bfloat16() if kind == "c1" else None))
    one = torch.ones((), device=dev)

    def step(i):
        a, b, bias = sets[i & 1]
        if kind == "c3":
            torch._int_mm(a, b)
        else:
            torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, bias=bias, out_dtype=torch.bfloat16, use_fast_accum=True)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    if kind == "c2":
        value, unit = (k * n + m * k + 2 * m * n) / ms / 1e6, "GB/s"
    else:
        value, unit = 2.0 * m * n * k / ms / 1e9, "TFLOP/s"
    print(json.dumps({"impl": "cublaslt", "metric": METRIC, "value": value, "unit": unit, "n_gpus": 1, "steps": steps,
                      "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
                      "config": {"workload": kind, "m": m, "n": n, "k": k,
                                 "note": "torch._scaled_mm / torch._int_mm (cuBLASLt); no GELU, amax or dequantisation fused"}}),
          flush=True)


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "cublaslt":
        cublaslt_arm(a)
    elif a.impl == "reference":
        reference_arm(a)
    else:
        gpu_arm(a)
