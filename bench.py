#!/usr/bin/env python
"""Benchmark of the FP8 W8A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line.  A "step" is one pass of the hot path over one batch of seeded synthetic
input.  `value` is device-timed with the inputs resident in HBM; `e2e` repeats the measurement
through the public API with pinned HOST buffers (H2D of the step's inputs and D2H of its result
inside the timed region).  `roofline` is for the dominant kernel, timed with CUDA events on the
launching stream; `cpu_baseline` times the CPU oracle on a bounded sample of the same workload.
`--impl reference` times the reference's CPU path (the torch edition of the oracle: the reference is
Python and its CPU path is torch) on the host cores for the same workload and metric.

Workloads (BASELINE.json configs): ep_moe (configs[3]: DeepSeek-V3-shaped expert-parallel MoE layer,
128 tokens per rank, masked layout; the default, the one that shards over GPUs), moe_c3
(configs[2]), moe_c5 (configs[4]), silu_c2 (configs[1]), quant_c1 and gemm_c1 (configs[0]).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

FP8 = torch.float8_e4m3fn


# ------------------------------------------------------------------------------------------------
# helpers
# ------------------------------------------------------------------------------------------------

def measured_peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.005):
        self.index, self.period = index, period_s
        self.samples, self.active = [], False
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                if self.active:
                    self.samples.append((mhz, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()

    def stop(self) -> dict:
        self._stop.set()
        if self._thr is not None:
            self._thr.join(timeout=1.0)
        if self.nv is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        nv = self.nv
        mhz = sorted(s[0] for s in self.samples)
        bits = 0
        for _, r in self.samples:
            bits |= r
        names = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake": 0x80, "sync_boost": 0x10, "display_clock": 0x100, "applications_clocks": 0x2}
        try:
            mx = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            mx = None
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": mx, "reasons": [k for k, v in names.items() if bits & v],
                "samples": len(mhz)}


def dist_info():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


class Timed:
    """K steps, each bracketed by CUDA events on the current stream; an optional L2 flush (a read of a
    buffer larger than L2) runs between steps outside the events.  Whole region bracketed by barrier +
    synchronize; max over ranks."""

    def __init__(self, world: int, flush_bytes: int = 0, device=None):
        self.world = world
        self.flush = torch.zeros(flush_bytes // 8, dtype=torch.int64, device=device) if flush_bytes else None

    def barrier(self):
        if self.world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    def run(self, step, steps: int, warmup: int, sampler: ClockSampler | None = None) -> float:
        for i in range(warmup):
            step(i)
        self.barrier()
        if sampler is not None:
            sampler.active = True
        evs = []
        for i in range(steps):
            if self.flush is not None:
                # Reading a buffer twice the size of L2 evicts it with CLEAN lines (a written buffer would leave
                # dirty lines whose write-back lands inside the next timed kernel) and keeps the GPU busy while
                # the host queues the step, so the events bracket device time rather than launch cadence.
                self._sink = self.flush.sum()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step(warmup + i)
            b.record()
            evs.append((a, b))
        self.barrier()
        if sampler is not None:
            sampler.active = False
        total_ms = sum(a.elapsed_time(b) for a, b in evs)
        if self.world > 1:
            t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
            torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
            total_ms = float(t.item())
        return total_ms / steps


def run_graph(world: int, step, steps: int, warmup: int, sampler: ClockSampler | None = None, many=None) -> float:
    """For kernels of a few microseconds to a few tens of microseconds: the K steps are captured in ONE CUDA
    graph (so the launches are back to back on the device and the host's launch cadence is not what is timed)
    and that graph is timed with one pair of CUDA events.  The caller's step(i) must rotate through inputs and
    outputs whose total size exceeds L2, so that no step finds its data cached.  Warm-up: `warmup` eager steps,
    one untimed replay and a quarter of a second of further untimed replays (watched by the clock sampler, as is the
    timed one)."""
    if many is not None:          # many(n): n steps that overlap each other (forked streams inside), as one call
        many(warmup)
    else:
        for i in range(warmup):
            step(i)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        if many is not None:
            many(steps)
        else:
            for i in range(steps):
                step(warmup + i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    # about a quarter of a second of untimed replays: clocks and caches as in a running loop.  Their number is agreed
    # between the ranks (a step of the expert-parallel layer needs every rank to take it)
    n_pre = max(1, min(1000, int(250.0 / max(a.elapsed_time(b), 0.05))))
    if world > 1:
        t = torch.tensor([n_pre], dtype=torch.int64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        n_pre = int(t.item())
    if sampler is not None:
        sampler.active = True
    for _ in range(n_pre):
        graph.replay()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    if sampler is not None:
        sampler.active = False
    total_ms = a.elapsed_time(b)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        total_ms = float(t.item())
    return total_ms / steps


def measured_traffic(kernel: str, scale: float):
    """dram read + write bytes per launch of `kernel` from the profiler summary kept with the repository (one line per
    kernel: name, workload, bytes), times `scale`; None when there is no such line."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    try:
        for line in open(path):
            f = line.split()
            if len(f) >= 3 and not line.startswith("#") and f[0] == kernel:
                return float(f[2]) * scale
    except OSError:
        pass
    return None


def triton_ref(name: str):
    """kb-nano's own Triton kernel file `name` from oracle/_ref (the reference's GPU implementation of the operation,
    timed beside this library's as the competitor; never on the product path), or None when it is not there."""
    if not os.path.isfile(os.path.join(ROOT, "oracle", "_ref", name + ".py")):
        return None
    try:
        import importlib
        return importlib.import_module("oracle._ref." + name)
    except Exception:
        return None


def time_competitor(world, step, steps, warmup):
    """run_graph on the reference's kernel; None when it does not launch on this machine."""
    try:
        step(0)
        torch.cuda.synchronize()
        return run_graph(world, step, steps, warmup)
    except Exception:
        return None


def cpu_threads() -> int:
    n = os.cpu_count() or 1
    try:
        n = min(n, len(os.sched_getaffinity(0)))
    except Exception:
        pass
    return n


# ------------------------------------------------------------------------------------------------
# CPU side (oracle port): used by cpu_baseline and by --impl reference
# ------------------------------------------------------------------------------------------------

def cpu_silu_c2(rows: int, reps: int):
    from kb_nano_b200 import inputs
    from oracle import torch_oracle as to
    x = inputs.activations(rows, 4096, seed=0, outlier_frac=1e-3)
    to.silu_mul_quant_1x128(x)
    t0 = time.perf_counter()
    for _ in range(reps):
        to.silu_mul_quant_1x128(x)
    dt = (time.perf_counter() - t0) / reps
    byts = rows * (4096 * 2 + 2048 + 64)
    return byts / dt / 1e9, dt, f"{rows} of 16384 rows, {reps} passes, torch CPU port"


def cpu_quant(m: int, k: int, reps: int):
    from kb_nano_b200 import inputs
    from oracle import torch_oracle as to
    x = inputs.activations(m, k, seed=0)
    to.quant_1x128(x)
    t0 = time.perf_counter()
    for _ in range(reps):
        to.quant_1x128(x)
    dt = (time.perf_counter() - t0) / reps
    return (3 * m * k + 4 * m * (k // 128)) / dt / 1e9, dt, f"[{m},{k}] full size, {reps} passes, torch CPU port"


def cpu_gemm_c1(n_cols: int, reps: int):
    from kb_nano_b200 import inputs
    from oracle import torch_oracle as to
    x = inputs.activations(512, 7168, seed=0)
    w_q, w_s = inputs.weight(n_cols, 7168, seed=1)
    a_q, a_s = to.quant_1x128(x)
    to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    t0 = time.perf_counter()
    for _ in range(reps):
        to.gemm_nt_dequant(a_q, a_s, w_q, w_s)
    dt = (time.perf_counter() - t0) / reps
    return 2.0 * 512 * n_cols * 7168 / dt / 1e12, dt, f"N={n_cols} of 4096 output columns (time is linear in N), {reps} passes, torch CPU port"


def cpu_moe(t: int, h: int, i: int, e: int, topk: int, routing: str, n_experts_sample: int, reps: int):
    """Times the oracle's MoE layer restricted to the first `n_experts_sample` experts that have tokens and
    scales to the whole layer by the share of (token, slot) pairs those experts hold."""
    from kb_nano_b200 import inputs
    from oracle import torch_oracle as to
    x = inputs.activations(t, h, seed=0)
    logits = inputs.router_logits(t, e, seed=0)
    tw, ti = (inputs.route_sigmoid_topk if routing == "sigmoid" else inputs.route_softmax_topk)(logits, topk)
    counts = torch.bincount(ti.reshape(-1).long(), minlength=e)
    chosen = [int(x_) for x_ in torch.nonzero(counts).flatten()[:n_experts_sample]]
    w13_q = torch.zeros(e, 1, 1, dtype=torch.uint8).view(FP8)   # placeholders, indexed per expert below
    store13, store2 = {}, {}
    for ex in chosen:
        store13[ex] = inputs.weight(2 * i, h, seed=1 * 1000003 + ex)
        store2[ex] = inputs.weight(h, i, seed=2 * 1000003 + ex)

    class _Pick:
        def __init__(self, d, j):
            self.d, self.j = d, j

        def __getitem__(self, ex):
            return self.d[ex][self.j]

    def one():
        return to.moe_layer(x, _Pick(store13, 0), _Pick(store13, 1), _Pick(store2, 0), _Pick(store2, 1), tw, ti, experts=chosen)

    one()                                   # warm-up pass
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        one()
        times.append(time.perf_counter() - t0)
    dt = sorted(times)[len(times) // 2]     # median pass
    share = float(counts[chosen].sum()) / float(counts.sum())
    # dequantising an expert's weights costs the same however few rows it has: scale by experts, not pairs,
    # when rows per expert are few
    active = int((counts > 0).sum())
    factor = max(active / len(chosen), 1.0) if t * topk / e < 64 else 1.0 / share
    est_full = dt * factor
    del w13_q
    return t / est_full, dt, (f"{len(chosen)} of {active} active experts with their routed rows ({share * 100:.1f}% of pairs), median of "
                              f"{reps} passes after one warm-up pass ({dt * 1e3:.0f} ms), torch CPU port; whole layer = sample x {factor:.2f}")


# ------------------------------------------------------------------------------------------------
# GPU workloads
# ------------------------------------------------------------------------------------------------

def wl_silu_c2(args, rank, world, dev, sampler):
    from kb_nano_b200 import _lib, inputs, ops
    m, n = 16384, 4096
    nbuf = 4
    xs = [inputs.activations(m, n, seed=b, device=dev, outlier_frac=1e-3) for b in range(nbuf)]
    qs = [torch.empty(m, n // 2, dtype=FP8, device=dev) for _ in range(nbuf)]
    ss = [torch.empty(n // 256, m, device=dev).t() for _ in range(nbuf)]
    q, s = qs[0], ss[0]
    byts = m * n * 2 + m * n // 2 + 4 * m * (n // 256)
    l0 = _lib.launch_count()
    ms = run_graph(world, lambda i: ops.silu_mul_quant_fp8(xs[i % nbuf], qs[i % nbuf], ss[i % nbuf]), args.steps, args.warmup, sampler)
    launches = _lib.launch_count() - l0
    # e2e: pinned host input, device result copied back
    host_in = [x.cpu().pin_memory() for x in xs[:2]]
    d_in = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    h_q = torch.empty(m, n // 2, dtype=torch.uint8).pin_memory()
    h_s = torch.empty(n // 256, m, dtype=torch.float32).pin_memory()

    def e2e_step(i):
        d_in.copy_(host_in[i % 2], non_blocking=True)
        ops.silu_mul_quant_fp8(d_in, q, s)
        h_q.copy_(q.view(torch.uint8), non_blocking=True)
        h_s.copy_(s.t(), non_blocking=True)

    ms_e2e = Timed(world, 0, dev).run(e2e_step, max(3, args.steps // 4), 2)
    peaks = measured_peaks()
    gbs = byts / (ms * 1e-3) / 1e9
    # the same operation by kb-nano's Triton kernel (tasks/baseline/L1/silu_mul_quant_fp8.py), same inputs, same timing
    vs_triton = None
    mod = triton_ref("silu_mul_quant_fp8")
    if mod is not None:
        smq = mod.SiluMulQuantFp8()
        ms_t = time_competitor(world, lambda i: smq(xs[i % nbuf], qs[i % nbuf]), args.steps, args.warmup)
        vs_triton = ms_t / ms if ms_t else None
    return {
        "vs_triton": vs_triton,
        "metric": "fused SiLU*Mul+FP8 quant throughput", "value": gbs * world, "unit": "GB/s", "ms_per_step": ms,
        "dtype": "bf16->e4m3 (fp32 math)", "scaling": "weak",
        "config": {"workload": "silu_c2: BASELINE configs[1], bf16 [16384, 2x2048] -> e4m3 [16384,2048] + UE8M0 scales [16384,16]",
                   "l2": "inputs larger than L2: 4 rotating input buffers (537 MB) and 4 rotating output buffers (142 MB)",
                   "timing": "the K steps are captured in one CUDA graph and timed with one CUDA-event pair", "replicas": world},
        "e2e": {"value": byts / (ms_e2e * 1e-3) / 1e9 * world, "unit": "GB/s", "h2d_bytes_per_step": m * n * 2,
                "d2h_bytes_per_step": m * n // 2 + 4 * m * (n // 256)},
        "gpu_launches": launches // (args.steps + args.warmup) * args.steps,
        "roofline": {"bound": "hbm", "kernel": "silu_mul_quant_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": measured_traffic("silu_mul_quant", 1.0), "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": byts},
        "_cpu": lambda: cpu_silu_c2(2048, 3),
    }


def wl_quant_c1(args, rank, world, dev, sampler, m=512, k=7168):
    from kb_nano_b200 import _lib, inputs, ops
    # enough rotating input copies that a step never finds its input in the 126 MB L2
    nbuf = max(4, -(-(320 << 20) // (m * k * 2)))
    x = inputs.activations(m, k, seed=0, device=dev)
    xs = [x] + [x.clone() for _ in range(nbuf - 1)]
    nout = max(4, -(-(192 << 20) // (m * k)))
    qs = [torch.empty(m, k, dtype=FP8, device=dev) for _ in range(nout)]
    ss = [torch.empty(k // 128, m, device=dev).t() for _ in range(nout)]
    q, s = qs[0], ss[0]
    byts = 3 * m * k + 4 * m * (k // 128)
    l0 = _lib.launch_count()
    ms = run_graph(world, lambda i: ops.per_token_group_quant_fp8(xs[i % nbuf], qs[i % nout], ss[i % nout]), args.steps, args.warmup, sampler)
    launches = _lib.launch_count() - l0
    hx = x.cpu().pin_memory()
    dx = torch.empty_like(x)
    hq = torch.empty(m, k, dtype=torch.uint8).pin_memory()

    def e2e_step(i):
        dx.copy_(hx, non_blocking=True)
        ops.per_token_group_quant_fp8(dx, q, s)
        hq.copy_(q.view(torch.uint8), non_blocking=True)

    ms_e2e = Timed(world, 256 << 20, dev).run(e2e_step, args.steps, 2)
    peaks = measured_peaks()
    gbs = byts / (ms * 1e-3) / 1e9
    # the same operation by kb-nano's Triton kernel (tasks/baseline/L1/fp8_linear.py:181-215, launched as :269-279 does)
    vs_triton = None
    mod = triton_ref("fp8_group_quant")
    if mod is not None:
        def tq(i):
            xi, qi, si = xs[i % nbuf], qs[i % nout], ss[i % nout]
            mod._fp8_group_quant_kernel[(m * (k // 128),)](xi, qi, si, xi.stride(0), qi.stride(0), si.stride(0), si.stride(1), k,
                                                          fp8_max=448.0, GROUP_SIZE=128, USE_UE8M0=True)
        ms_t = time_competitor(world, tq, args.steps, args.warmup)
        vs_triton = ms_t / ms if ms_t else None
    return {
        "vs_triton": vs_triton,
        "metric": "1x128 FP8 activation quant throughput", "value": gbs * world, "unit": "GB/s", "ms_per_step": ms,
        "dtype": "bf16->e4m3", "scaling": "weak",
        "config": {"workload": f"quant_{'c1' if m == 512 else 'c3'}: activation of BASELINE configs[{0 if m == 512 else 2}], bf16 [{m},{k}], column-major UE8M0 scales",
                   "l2": f"inputs larger than L2: {nbuf} rotating input buffers ({nbuf * m * k * 2 >> 20} MB) and {nout} rotating output buffers ({nout * m * k >> 20} MB)",
                   "timing": "the K steps are captured in one CUDA graph and timed with one CUDA-event pair", "replicas": world},
        "e2e": {"value": byts / (ms_e2e * 1e-3) / 1e9 * world, "unit": "GB/s", "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * k},
        "gpu_launches": launches // (args.steps + args.warmup) * args.steps,
        "roofline": {"bound": "hbm", "kernel": "quant_1x128_kernel", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"], "traffic": measured_traffic("quant_1x128", 1.0) if m == 4096 else None,
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": byts},
        "_cpu": lambda: cpu_quant(m, k, 20 if m == 512 else 3),
    }


def wl_gemm_c1(args, rank, world, dev, sampler):
    from kb_nano_b200 import _lib, inputs, ops
    m, n, k = 512, 4096, 7168
    x = inputs.activations(m, k, seed=0, device=dev)
    w_q, w_s = inputs.weight(n, k, seed=1, device=dev)
    a_q = torch.empty(m, k, dtype=FP8, device=dev)
    a_s = torch.empty(k // 128, m, device=dev).t()
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    ops.per_token_group_quant_fp8(x, a_q, a_s)
    sfb = ops.packed_weight_scales(w_s, n, k)     # weight scales are powers of two: block-scaled tensor-core path
    sfa = ops.pack_sf_rows(a_s, k)
    flop = 2.0 * m * n * k
    nbuf = 8                                      # 8 copies of the 29 MB weight: 235 MB, no step finds its weight in L2
    ws = [w_q] + [w_q.clone() for _ in range(nbuf - 1)]
    outs = [out] + [torch.empty_like(out) for _ in range(nbuf - 1)]
    l0 = _lib.launch_count()
    ms = run_graph(world, lambda i: ops.fp8_gemm_nt_ue8m0(a_q, sfa, ws[i % nbuf], sfb, outs[i % nbuf]), args.steps, args.warmup, sampler)
    launches = _lib.launch_count() - l0
    hx = x.cpu().pin_memory()
    dx = torch.empty_like(x)
    hout = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()

    def e2e_step(i):   # the Fp8Linear call: quant + GEMM on a host activation, result back on the host
        dx.copy_(hx, non_blocking=True)
        ops.fp8_linear(dx, a_q, a_s, w_q, w_s, out)
        hout.copy_(out, non_blocking=True)

    ms_e2e = Timed(world, 256 << 20, dev).run(e2e_step, args.steps, 2)
    peaks = measured_peaks()
    tf = flop / (ms * 1e-3) / 1e12
    fp8_peak = 2.0 * peaks["bf16_tflops"]
    assert ops.gemm_status(dev) == 0
    return {
        "metric": "block-scaled FP8 GEMM throughput", "value": tf * world, "unit": "TFLOP/s", "ms_per_step": ms,
        "dtype": "e4m3 x e4m3 -> fp32 -> bf16", "scaling": "weak",
        "config": {"workload": "gemm_c1: BASELINE configs[0], M=512 K=7168 N=4096, 1x128 / 128x128 UE8M0 scales",
                   "l2": "inputs larger than L2: 8 rotating copies of the weight (235 MB) and of the output (34 MB)",
                   "timing": "the K steps are captured in one CUDA graph and timed with one CUDA-event pair", "replicas": world},
        "e2e": {"value": flop / (ms_e2e * 1e-3) / 1e12 * world, "unit": "TFLOP/s", "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2},
        "gpu_launches": launches // (args.steps + args.warmup) * args.steps,
        "roofline": {"bound": "tensor", "kernel": "fp8_gemm_mx_pair_kernel", "achieved": tf, "peak": fp8_peak, "unit": "TFLOP/s", "frac": tf / fp8_peak,
                     "traffic": measured_traffic("fp8_gemm_mx_pair", 1.0), "peak_source": peaks["source"] + " bf16 burst x2 (no FP8 entry in MEASURED_PEAKS.json)",
                     "frac_of_nominal_4500": tf / 4500.0, "algorithmic_flop_per_launch": flop},
        "_cpu": lambda: cpu_gemm_c1(512, 3),
    }


def build_moe_inputs(t, h, i, e, topk, routing, dev, seed=0):
    from kb_nano_b200 import inputs
    x = inputs.activations(t, h, seed=seed, device=dev)
    logits = inputs.router_logits(t, e, seed=seed, device=dev)
    tw, ti = (inputs.route_sigmoid_topk if routing == "sigmoid" else inputs.route_softmax_topk)(logits, topk)
    w13_q, w13_s = inputs.expert_weights(e, 2 * i, h, seed=1, device=dev)
    w2_q, w2_s = inputs.expert_weights(e, h, i, seed=2, device=dev)
    return x, tw.contiguous(), ti.contiguous(), w13_q, w13_s, w2_q, w2_s


def wl_moe_single(args, rank, world, dev, sampler, name):
    """One-GPU MoE layer in the contiguous grouped layout (configs[2] / configs[4])."""
    from kb_nano_b200 import _lib, moe, ops
    if name == "moe_c3":
        t, h, i, e, topk, routing = 4096, 7168, 2048, 256, 8, "sigmoid"
        desc = "moe_c3: BASELINE configs[2], DeepSeek-V3-shaped FP8 MoE layer, 4096 tokens, 256 experts, top-8, contiguous layout"
        if args.experts != 256:          # same rows per expert with fewer experts and tokens: small enough for a profiler capture
            e, t = args.experts, 16 * args.experts
            desc += f" [REDUCED to {e} experts and {t} tokens: profiling case, not the benchmark configuration]"
    else:
        t, h, i, e, topk, routing = 16384, 4096, 14336, 8, 2, "softmax"
        desc = "moe_c5: BASELINE configs[4], Mixtral-8x7B-shaped FP8 MoE layer, 16384 tokens, 8 experts, top-2, contiguous layout"
    x, tw, ti, w13_q, w13_s, w2_q, w2_s = build_moe_inputs(t, h, i, e, topk, routing, dev)
    sc = moe.get_scratch(t, topk, e, h, i, dev)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)

    def step(_):
        moe.fused_experts_fp8(x, w13_q, w2_q, tw, ti, e, w13_s, w2_s, scratch=sc, out=out)

    l0 = _lib.launch_count()
    ms = Timed(world, 0, dev).run(step, args.steps, args.warmup, sampler)
    launches = _lib.launch_count() - l0
    # dominant kernel: the two grouped GEMM launches, timed alone with events on the same inputs
    evs = []
    p13, p2 = ops.packed_weight_scales(w13_s, 2 * i, h), ops.packed_weight_scales(w2_s, h, i)
    sf1 = ops.pack_sf_rows(sc.a_s_perm, h)
    for _ in range(max(3, min(args.steps, 10))):
        a, b = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        a.record()
        ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(sc.a_perm, sf1, w13_q, p13, sc.mm1(i), sc.row_expert)
        b.record()
        ops.silu_mul_quant_fp8_rows(sc.mm1(i), sc.a2_q, sc.a2_s, sc.row_expert)
        sf2 = ops.pack_sf_rows(sc.a2_s, i)
        d, f = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        d.record()
        ops.m_grouped_fp8_gemm_nt_contiguous_ue8m0(sc.a2_q, sf2, w2_q, p2, sc.mm2(h), sc.row_expert)
        f.record()
        evs.append((a, b, d, f))
    torch.cuda.synchronize()
    gemm_ms = sum(a.elapsed_time(b) + d.elapsed_time(f) for a, b, d, f in evs) / len(evs) / 2.0   # per launch
    pairs = t * topk
    active = int((torch.bincount(ti.reshape(-1).long(), minlength=e) > 0).sum())
    g1 = active * 2 * i * h + pairs * h + pairs * 2 * i * 2 + 4 * pairs * (h // 128)
    g2 = active * h * i + pairs * i + pairs * h * 2 + 4 * pairs * (i // 128)
    flop = 2.0 * pairs * (2 * i * h + h * i)
    peaks = measured_peaks()
    assert ops.gemm_status(dev) == 0
    # e2e through the public layer call with pinned host activations / routing and the result copied back
    hx, htw, hti = x.cpu().pin_memory(), tw.cpu().pin_memory(), ti.cpu().pin_memory()
    dx, dtw, dti = torch.empty_like(x), torch.empty_like(tw), torch.empty_like(ti)
    hout = torch.empty(t, h, dtype=torch.bfloat16).pin_memory()

    def e2e_step(_):
        dx.copy_(hx, non_blocking=True)
        dtw.copy_(htw, non_blocking=True)
        dti.copy_(hti, non_blocking=True)
        moe.fused_experts_fp8(dx, w13_q, w2_q, dtw, dti, e, w13_s, w2_s, scratch=sc, out=out)
        hout.copy_(out, non_blocking=True)

    ms_e2e = Timed(world, 0, dev).run(e2e_step, max(3, args.steps // 2), 2)
    # the two grouped GEMMs by kb-nano's Triton kernel (tasks/baseline/L1/moe_grouped_gemm.py:86-189 through its
    # MoeGroupedGemm module, sorted-token layout, the module's own default configuration), same operands
    vs_triton = None
    mod = triton_ref("moe_grouped_gemm")
    if mod is not None:
        try:
            gg = mod.MoeGroupedGemm()
            cfg = gg.get_config(t, 2 * i, e, use_fp8=True, block_shape=[128, 128])
            bm = cfg["BLOCK_SIZE_M"]
            flat = ti.reshape(-1).long()
            order = torch.argsort(flat, stable=True)
            cnt = torch.bincount(flat, minlength=e)
            padded = (cnt + bm - 1) // bm * bm
            starts = torch.cumsum(padded, 0) - padded
            sorted_ids = torch.full((int(padded.sum()),), pairs, dtype=torch.int32, device=dev)
            rank_in_e = torch.arange(pairs, device=dev) - (torch.cumsum(cnt, 0) - cnt)[flat[order]]
            sorted_ids[(starts[flat[order]] + rank_in_e)] = order.to(torch.int32)
            blk_e = torch.repeat_interleave(torch.arange(e, device=dev, dtype=torch.int32), (padded // bm))
            ntpp = torch.tensor([sorted_ids.numel()], dtype=torch.int32, device=dev)
            a_s_rm = sc.a_s.contiguous()
            c1 = sc.mm1(i)[:pairs]
            a2_s_rm = sc.a2_s[:pairs].contiguous()
            c2 = sc.mm2(h)[:pairs]
            twf = tw.float().contiguous()

            def tri(_):
                gg(sc.a_q, w13_q, c1, twf, sorted_ids, blk_e, ntpp, False, topk, config=cfg, a_scale=a_s_rm, b_scale=w13_s,
                   use_fp8_w8a8=True, block_shape=[128, 128])
                gg(sc.a2_q[:pairs], w2_q, c2, twf, sorted_ids, blk_e, ntpp, True, 1, config=cfg, a_scale=a2_s_rm, b_scale=w2_s,
                   use_fp8_w8a8=True, block_shape=[128, 128])

            tri(0)
            torch.cuda.synchronize()
            tev = []
            for _ in range(5):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                tri(0)
                b.record()
                tev.append((a, b))
            torch.cuda.synchronize()
            tri_ms = sorted(a.elapsed_time(b) for a, b in tev)[len(tev) // 2]
            vs_triton = tri_ms / (2.0 * gemm_ms)
        except Exception:
            vs_triton = None
    hbm_bound = (pairs / e) < 562      # rows per expert below the machine balance: weights dominate
    if hbm_bound:
        ach = (g1 + g2) / 2.0 / (gemm_ms * 1e-3) / 1e9
        roof = {"bound": "hbm", "kernel": "fp8_gemm_mx_kernel (grouped, 2 launches per layer)", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": ach / peaks["hbm_gbs"], "traffic": measured_traffic("fp8_gemm_mx_contig", (e * 3.0 * i * h) / (32 * 3.0 * 2048 * 7168)),
                "peak_source": peaks["source"], "algorithmic_bytes_per_launch": (g1 + g2) / 2.0,
                "tflops": flop / 2.0 / (gemm_ms * 1e-3) / 1e12}
    else:
        ach = flop / 2.0 / (gemm_ms * 1e-3) / 1e12
        roof = {"bound": "tensor", "kernel": "fp8_gemm_mx_kernel (grouped, 2 launches per layer)", "achieved": ach, "peak": 2.0 * peaks["bf16_tflops_sustained"],
                "unit": "TFLOP/s", "frac": ach / (2.0 * peaks["bf16_tflops_sustained"]), "traffic": None,
                "peak_source": peaks["source"] + " bf16 sustained x2 (no FP8 entry in MEASURED_PEAKS.json)",
                "frac_of_nominal_4500": ach / 4500.0, "algorithmic_flop_per_launch": flop / 2.0}
    n_cpu = 4 if name == "moe_c3" else 1
    return {
        "vs_triton": vs_triton,
        "metric": "FP8 MoE layer throughput", "value": t / (ms * 1e-3) * world, "unit": "tokens/s", "ms_per_step": ms,
        "dtype": "e4m3 x e4m3 -> fp32 -> bf16", "scaling": "weak",
        "config": {"workload": desc, "l2": "expert weights (>= 1.4 GB) exceed the 126 MB L2", "replicas": world,
                   "layer_hbm_gbs": (g1 + g2 + 3 * t * h + pairs * (h + 2 * 2 * i + i) + (topk + 1) * t * h * 2) / (ms * 1e-3) / 1e9,
                   "layer_tflops": flop / (ms * 1e-3) / 1e12},
        "e2e": {"value": t / (ms_e2e * 1e-3) * world, "unit": "tokens/s", "h2d_bytes_per_step": t * h * 2 + t * topk * 8, "d2h_bytes_per_step": t * h * 2},
        "gpu_launches": launches // (args.steps + args.warmup) * args.steps,
        "roofline": roof,
        "_cpu": lambda: cpu_moe(t, h, i, e, topk, routing, n_cpu, 3),
    }


def ep_parity(out, x, tw, ti, h, i, dev, world, n_tokens=2):
    """A few of this rank's tokens of the expert-parallel result against the CPU oracle's single-process layer: the
    experts those tokens route to are generated again from their seeds (on this rank's GPU, whose generator gives the
    bits the owning rank's gave) and brought to the host.  Tolerance: |d| <= 1e-2 + 1e-2 |ref| element-wise,
    max|d| / max|ref| <= 1e-2, cosine > 0.9999.  Returns the worst figures over all ranks."""
    from kb_nano_b200 import inputs
    from oracle import torch_oracle as to
    torch.set_num_threads(max(1, cpu_threads() // world))
    t = x.shape[0]
    sel = torch.linspace(0, t - 1, steps=min(n_tokens, t)).long().unique()
    xs, tws, tis = x[sel].cpu(), tw[sel].cpu(), ti[sel].cpu()
    need = sorted(set(int(v) for v in tis.flatten()))
    w13, w2 = {}, {}
    for ex in need:
        q, s_ = inputs.weight(2 * i, h, seed=1 * 1000003 + ex, device=dev)
        w13[ex] = (q.cpu(), s_.cpu())
        q, s_ = inputs.weight(h, i, seed=2 * 1000003 + ex, device=dev)
        w2[ex] = (q.cpu(), s_.cpu())

    class _Pick:
        def __init__(self, d, j):
            self.d, self.j = d, j

        def __getitem__(self, ex):
            return self.d[ex][self.j]

    ref = to.moe_layer(xs, _Pick(w13, 0), _Pick(w13, 1), _Pick(w2, 0), _Pick(w2, 1), tws, tis, experts=need).float().flatten()
    got = out[sel].float().cpu().flatten()
    d = (got - ref).abs()
    ratio = float((d / (1e-2 + 1e-2 * ref.abs())).max())
    rel_inf = float(d.max() / ref.abs().max().clamp_min(1e-30))
    cos = float(torch.nn.functional.cosine_similarity(got.double(), ref.double(), dim=0))
    finite = bool(torch.isfinite(got).all())
    worst = torch.tensor([ratio, rel_inf, -cos, 0.0 if finite else 1.0], dtype=torch.float64, device=dev)
    if world > 1:
        torch.distributed.all_reduce(worst, op=torch.distributed.ReduceOp.MAX)
    ratio, rel_inf, cos, bad = float(worst[0]), float(worst[1]), -float(worst[2]), float(worst[3])
    ok = bad == 0.0 and ratio <= 1.0 and rel_inf <= 1e-2 and cos > 0.9999
    return {"against": "CPU oracle, single-process layer on the same seeded inputs", "tokens_per_rank": int(sel.numel()), "ranks": world,
            "experts_regenerated_per_rank": len(need), "ratio": ratio, "rel_inf": rel_inf, "cos": cos, "ok": ok}


EP_SHAPES = {
    # name: (hidden, inter, experts, topk, routing, tokens(world) per rank, max_m, scaling, description)
    "ep_moe": (7168, 2048, None, 8, "sigmoid", lambda w: 128, 256, "weak",
               "ep_moe: BASELINE configs[3], DeepSeek-V3-shaped FP8 MoE layer (hidden 7168, intermediate 2048, 256 experts, "
               "top-8 sigmoid routing), expert-parallel, 128 tokens per rank, masked layout, <=256 rows per expert"),
    "ep_moe_1024": (7168, 2048, None, 8, "sigmoid", lambda w: 1024 // w, 256, "strong",
                    "ep_moe_1024: BASELINE configs[3] at a FIXED global batch of 1024 tokens (1024/N per rank), masked layout, "
                    "<=256 rows per expert"),
    "ep_c5": (4096, 14336, 8, 2, "softmax", lambda w: 16384 // w, 5120, "strong",
              "ep_c5: BASELINE configs[4] expert-parallel, Mixtral-8x7B-shaped FP8 MoE layer (hidden 4096, intermediate 14336, "
              "8 experts, top-2 softmax routing), 16384 tokens in total (16384/N per rank), masked layout, <=5120 rows per expert"),
}


def wl_ep_moe(args, rank, world, dev, sampler, name="ep_moe"):
    """Expert-parallel MoE layer: experts split over the ranks, masked layout, dispatch/combine by peer stores
    over NVLink.  `name` picks the shape (BASELINE configs[3], its fixed-global-batch form, or configs[4])."""
    from kb_nano_b200 import _lib, ep, inputs, ops
    h, i, e_fixed, topk, routing, t_of, max_m, scaling, desc = EP_SHAPES[name]
    e = e_fixed if e_fixed is not None else args.experts
    t = t_of(world)
    route = inputs.route_sigmoid_topk if routing == "sigmoid" else inputs.route_softmax_topk
    lo, hi = ep.expert_range(rank, world, e)
    e_l = hi - lo
    x = inputs.activations(t, h, seed=rank, device=dev)
    tw, ti = route(inputs.router_logits(t, e, seed=rank, device=dev), topk)
    tw, ti = tw.contiguous(), ti.contiguous()
    w13_q, w13_s = inputs.expert_weights(e_l, 2 * i, h, seed=1, device=dev, first=lo)
    w2_q, w2_s = inputs.expert_weights(e_l, h, i, seed=2, device=dev, first=lo)
    layer = ep.EpMoe(rank, world, e, h, i, max_tokens=t, topk=topk, max_m=max_m, device=dev)
    out = torch.empty(t, h, dtype=torch.bfloat16, device=dev)

    def step(_):
        layer.forward(x, ti, tw, w13_q, w13_s, w2_q, w2_s, out=out)

    # the K steps are captured in one CUDA graph and that graph is timed with one event pair, the way kb-nano replays
    # a decode step (infra/engine.py:2410-2427): launches counted here are the warm-up's and the capture's, replays
    # launch the same kernels again
    l0 = _lib.launch_count()
    ms = run_graph(world, step, args.steps, args.warmup, sampler)
    launches = _lib.launch_count() - l0
    layer.check()
    # rows every local expert receives (routing of all ranks is reproducible from the seeds)
    counts = torch.zeros(e, dtype=torch.long)
    for r in range(world):
        _, ti_r = route(inputs.router_logits(t, e, seed=r), topk)
        counts += torch.bincount(ti_r.reshape(-1).long(), minlength=e)
    local = counts[lo:hi]
    assert int(local.max()) <= max_m
    # dominant kernels: the two masked grouped GEMM launches (GEMM1 with the activation epilogue, GEMM2 with the combine
    # epilogue, the second started while the first still runs) as the layer launches them, on the rows the last step left
    # in the receive buffers; the pair is timed with CUDA events on the launching stream
    masked = local.to(torch.int32).to(dev)
    expected_m = max(1, -(-t * world * topk // e))
    evs = []
    for k_ in range(3 + max(5, min(args.steps, 20))):
        a, b = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        a.record()
        layer.expert_phase(w13_q, w13_s, w2_q, w2_s, masked, expected_m)
        b.record()
        if k_ >= 3:
            evs.append((a, b))
    if world > 1:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    gemm_ms = sum(a.elapsed_time(b) for a, b in evs) / len(evs) / 2.0         # per launch
    if world > 1:
        tmax = torch.tensor([gemm_ms], dtype=torch.float64, device=dev)
        torch.distributed.all_reduce(tmax, op=torch.distributed.ReduceOp.MAX)
        gemm_ms = float(tmax.item())
    active, rows = int((local > 0).sum()), int(local.sum())
    g1 = active * 2 * i * h + rows * h + rows * i + 4 * rows * (i // 128) + 4 * rows * (h // 128)
    g2 = active * h * i + rows * i + rows * h * 2 + 4 * rows * (i // 128)
    peaks = measured_peaks()
    ach = (g1 + g2) / 2.0 / (gemm_ms * 1e-3) / 1e9
    gemm_tflops = 2.0 * rows * 3 * i * h / 2.0 / (gemm_ms * 1e-3) / 1e12
    # e2e: pinned host activations and routing in, result back to the host, through the package's host pipeline: the
    # three inputs travel as one staged buffer (one H2D copy per step), the copies of neighbouring steps overlap the
    # layer of the current one over two or three rotating device buffers
    # one copy stream; three device buffers for small steps (the decode layer: 1.8 MB each way), two for large ones
    # (configs[4]: tens of MB each way) -- measured on 2 GPUs, ms per step of configs[4]: 3.98 with two buffers, 4.13 with
    # three, 4.20-4.23 with a copy stream per direction
    big = t * h * 2 >= (8 << 20)
    pipe = ep.EpMoeHostPipeline(layer, depth=args.e2e_depth or (2 if big else 3), copy_streams=args.e2e_streams or 1)
    hblob, hout = pipe.new_host_buffers()
    pipe.pack(hblob, x.cpu(), tw.cpu(), ti.cpu())

    def e2e_steps(n):
        pipe.begin()
        for _ in range(n):
            pipe.submit(hblob, hout, w13_q, w13_s, w2_q, w2_s)
        pipe.join()

    # the K steps (copy in, layer, copy out) are captured in one CUDA graph, the way a serving loop replays a decode
    # step: the layer keeps its step counter on the device, so a captured step can be replayed
    ms_e2e = run_graph(world, None, args.steps, 3, many=e2e_steps)
    assert_close_to_device = (hout.to(dev).view(torch.int16) == out.view(torch.int16)).all()
    assert bool(assert_close_to_device), "host pipeline result differs from the device-resident run"
    layer.check()
    assert ops.gemm_status(dev) == 0
    # the outputs of the timed configuration against the oracle, on every rank (outside every timed region)
    parity = ep_parity(out, x, tw, ti, h, i, dev, world) if args.parity else None
    layer.close()
    if parity is not None and not parity["ok"]:
        raise SystemExit(f"expert-parallel output differs from the oracle beyond the tolerance: {parity}")
    flop = 2.0 * t * topk * world * 3 * i * h
    # rows per streamed expert decide the bound: below ~560 rows per weight pass the weights' HBM traffic dominates
    tensor_bound = rows / max(active, 1) >= 560
    if tensor_bound:
        fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
        roof = {"bound": "tensor", "kernel": "fp8_gemm_mx_kernel (masked grouped; GEMM1 with the activation epilogue and GEMM2 with the combine epilogue, 2 overlapping launches per layer; max over ranks)", "achieved": gemm_tflops,
                "peak": fp8_peak, "unit": "TFLOP/s", "frac": gemm_tflops / fp8_peak, "traffic": None,
                "peak_source": peaks["source"] + " (2 x sustained bf16 cuBLAS figure; no FP8 figure is measured)",
                "algorithmic_flop_per_launch": 2.0 * rows * 3 * i * h / 2.0, "gemm_ms_per_launch": gemm_ms}
    else:
        roof = {"bound": "hbm", "kernel": "fp8_gemm_mx_kernel (masked grouped; GEMM1 with the activation epilogue and GEMM2 with the combine epilogue, 2 overlapping launches per layer; rank 0's bytes over the slowest rank's time)", "achieved": ach,
                "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": ach / peaks["hbm_gbs"],
                # DRAM bytes per launch as a profiler capture of the 32-expert case counted them, scaled by the bytes of the
                # experts whose weights are streamed (the traffic is proportional to them)
                "traffic": measured_traffic("fp8_gemm_mx_masked", active * (3.0 * i * h) / (32 * 3.0 * 2048 * 7168)), "peak_source": peaks["source"],
                "algorithmic_bytes_per_launch": (g1 + g2) / 2.0, "gemm_ms_per_launch": gemm_ms}
    return {
        "metric": "EP FP8 MoE layer throughput", "value": t * world / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
        "dtype": "e4m3 x e4m3 -> fp32 -> bf16", "scaling": scaling,
        "config": {"workload": desc + ("" if e_fixed is not None or e == 256 else
                                       f" [REDUCED to {e} experts: profiling case, not the benchmark configuration]"),
                   "parallelism": f"ep{world}", "experts_per_rank": e_l, "tokens_per_rank": t, "global_tokens": t * world,
                   "l2": f"local expert weights ({e_l * 3 * i * h / 1e9:.2f} GB) exceed the 126 MB L2",
                   "exchange": "peer stores over NVLink (dispatch fp8 rows + scales, combine bf16 rows), release/acquire flags",
                   "timing": "K layer steps captured in one CUDA graph (the layer's step counter lives on the device), untimed replays "
                             "for a quarter of a second, then one replay between two CUDA events; max over ranks",
                   "e2e": "EpMoeHostPipeline: per step one pinned-host -> device copy of the inputs, the layer, one device -> host copy "
                          "of the result; the copies run on a stream of their own over two or three rotating device buffers and overlap the "
                          "neighbouring steps' layer; the K steps are captured in one CUDA graph and timed with one CUDA-event pair",
                   "layer_tflops": flop / world / (ms * 1e-3) / 1e12},
        "e2e": {"value": t * world / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": t * h * 2 + t * topk * 8, "d2h_bytes_per_step": t * h * 2},
        "gpu_launches": launches // (args.steps + args.warmup) * args.steps,
        "roofline": roof,
        "parity": parity,
        "_cpu": lambda: cpu_moe(t, h, i, e, topk, routing, 8 if routing == "sigmoid" else 1, 5 if routing == "sigmoid" else 3),
    }


WORKLOADS = {
    "ep_moe": wl_ep_moe,
    "silu_c2": wl_silu_c2,
    "quant_c1": wl_quant_c1,
    "gemm_c1": wl_gemm_c1,
    "quant_c3": lambda *a: wl_quant_c1(*a, m=4096, k=7168),
    "moe_c3": lambda *a: wl_moe_single(*a, "moe_c3"),
    "moe_c5": lambda *a: wl_moe_single(*a, "moe_c5"),
    "ep_moe_1024": lambda *a: wl_ep_moe(*a, name="ep_moe_1024"),
    "ep_c5": lambda *a: wl_ep_moe(*a, name="ep_c5"),
}
DEFAULT_WORKLOAD = "ep_moe"


def reference_arm(args, rank, world):
    """The reference's CPU path for the workload (torch on the host cores), rank 0 only."""
    if rank != 0:
        return
    torch.set_num_threads(cpu_threads())
    wl = args.workload
    reps = max(1, min(args.steps, 3))
    if wl == "silu_c2":
        v, dt, sample = cpu_silu_c2(4096, reps)
        metric, unit = "fused SiLU*Mul+FP8 quant throughput", "GB/s"
    elif wl in ("quant_c1", "quant_c3"):
        v, dt, sample = cpu_quant(512 if wl == "quant_c1" else 4096, 7168, max(reps, 10) if wl == "quant_c1" else reps)
        metric, unit = "1x128 FP8 activation quant throughput", "GB/s"
    elif wl == "gemm_c1":
        v, dt, sample = cpu_gemm_c1(1024, reps)
        metric, unit = "block-scaled FP8 GEMM throughput", "TFLOP/s"
    elif wl == "moe_c5":
        v, dt, sample = cpu_moe(16384, 4096, 14336, 8, 2, "softmax", 1, 1)
        metric, unit = "FP8 MoE layer throughput", "tokens/s"
    elif wl == "moe_c3":
        v, dt, sample = cpu_moe(4096, 7168, 2048, 256, 8, "sigmoid", 8, 1)
        metric, unit = "FP8 MoE layer throughput", "tokens/s"
    else:
        h, i, e_fixed, topk, routing, t_of, _, _, desc = EP_SHAPES[wl]
        e = e_fixed if e_fixed is not None else args.experts
        v, dt, sample = cpu_moe(t_of(world) * world, h, i, e, topk, routing, 8 if routing == "sigmoid" else 1, 1)
        metric, unit = "EP FP8 MoE layer throughput", "tokens/s"
        wl = desc
    line = {"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32 (torch CPU)", "data": "synthetic",
            "config": {"workload": wl, "parallelism": "host cores of rank 0"},
            "cpu_baseline": {"value": v, "unit": unit, "cores": cpu_threads(), "kind": "port", "sample": sample},
            "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-depth", type=int, default=0, help="device buffers of the host pipeline in the end-to-end leg (0: by step size)")
    ap.add_argument("--e2e-streams", type=int, default=0, help="copy streams of the host pipeline (0: by step size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-components", action="store_true",
                    help="default workload only: skip the other configurations' figures reported beside the headline number")
    ap.add_argument("--no-parity", dest="parity", action="store_false",
                    help="expert-parallel workloads: skip the comparison of the timed configuration's output with the CPU oracle")
    ap.add_argument("--experts", type=int, default=256,
                    help="ep_moe and moe_c3: total experts (256 = the benchmark configuration; 32 on one GPU reproduces the "
                         "per-rank load of the 8-GPU run with 1.4 GB of weights, small enough for a profiler capture; moe_c3 "
                         "scales its tokens along, 16 per expert)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank, local, world = dist_info()
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        torch.distributed.init_process_group("nccl", device_id=dev)
    from kb_nano_b200 import _lib
    _lib.load()
    sampler = ClockSampler(local)
    sampler.start()
    res = WORKLOADS[args.workload](args, rank, world, dev, sampler)
    clocks = sampler.stop()
    cpu_fn = res.pop("_cpu", None)
    line = {"metric": res["metric"], "value": res["value"], "unit": res["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": res["ms_per_step"], "higher_is_better": True, "scaling": res["scaling"], "vs_baseline": None, "dtype": res["dtype"],
            "data": "synthetic", "config": res["config"], "e2e": res["e2e"], "gpu_launches": res["gpu_launches"], "roofline": res["roofline"],
            "clocks": clocks}
    if "parity" in res:
        line["parity"] = res["parity"]
    if res.get("vs_triton") is not None:
        line["vs_triton"] = res["vs_triton"]
    if args.workload == DEFAULT_WORKLOAD and args.experts == 256 and not args.no_components:
        # The other parts of the composite metric, each measured by its own workload function exactly as
        # `--workload <name>` would and under a clock-sampling window of its own, reported beside the headline number:
        # at N=1 the GEMM TFLOP/s, the quantiser GB/s and the one-GPU MoE layers of configs[2] and configs[4]; at N>1 the
        # expert-parallel layer at a fixed global batch and the expert-parallel configs[4] (both strong scaling).
        comp = {}
        sub = argparse.Namespace(**vars(args))
        sub.steps, sub.warmup = 20, 3
        names = ("gemm_c1", "silu_c2", "quant_c3", "quant_c1", "moe_c3", "moe_c5") if world == 1 else ("ep_moe_1024", "ep_c5")
        for name in names:
            torch.cuda.empty_cache()
            cs = ClockSampler(local)
            cs.start()
            r = WORKLOADS[name](sub, rank, world, dev, cs)
            entry = {"value": r["value"], "unit": r["unit"], "us_per_step": r["ms_per_step"] * 1e3, "bound": r["roofline"]["bound"],
                     "achieved": r["roofline"]["achieved"], "peak": r["roofline"]["peak"], "frac": r["roofline"]["frac"],
                     "e2e": r["e2e"]["value"], "scaling": r["scaling"], "clocks": cs.stop()}
            if r.get("parity") is not None:
                entry["parity_ok"] = r["parity"]["ok"]
            if r.get("vs_triton") is not None:
                # time of kb-nano's own Triton kernel(s) for the same operation on this GPU / time of this library's
                entry["vs_triton"] = r["vs_triton"]
            comp[name] = entry
        line["components"] = comp
    if rank == 0 and world == 1 and cpu_fn is not None and not args.no_cpu_baseline:
        torch.set_num_threads(cpu_threads())
        v, dt, sample = cpu_fn()
        line["cpu_baseline"] = {"value": v, "unit": res["unit"], "cores": cpu_threads(), "kind": "port", "sample": sample}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
