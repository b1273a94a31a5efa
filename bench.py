#!/usr/bin/env python
"""Benchmark of the low-precision linear hot path on B200.

Workload: NVFP4 linear forward + dgrad + wgrad at the Llama-3-8B
MLP-up shape -- X[8192,4096] ~ N(0,1), W[14336,4096] ~ N(0,0.02), dY[8192,14336] ~ N(0,1e-3),
bf16; E4M3 block-16 scales + FP32 tensorwise outer scale; W in 16x16 blocks; 16-point
randomised Hadamard on the wgrad operands; stochastic rounding of the gradients.  Data are
seeded synthetic tensors of those shapes and distributions.

One "step" = one forward + backward through the public autograd entry point
(``alto_b200.nvfp4._to_nvfp4_then_scaled_mm``): 5 amax/quantize passes and 3 block-scaled
GEMMs.  FLOPs counted: 3 * 2*M*N*K (quantizer work is in the time, not in the FLOPs).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Under torchrun (N > 1) every rank runs the same per-GPU workload on its own batch (data
parallel replicas, no collective on the path); the timed region is bracketed by a barrier and
``torch.cuda.synchronize()``, timed with CUDA events, and the maximum over ranks is used.
``--impl reference`` times the CPU restatement of the reference's PyTorch emulation path
(``oracle/``) on the host cores on a bounded row-sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch

M, K, N = 8192, 4096, 14336
FLOPS_PER_STEP = 3 * 2 * M * N * K
METRIC = "nvfp4_linear_fwd_dgrad_wgrad_tflops"
UNIT = "TFLOP/s"
CONFIG = {
    "workload": "NVFP4 linear fwd+dgrad+wgrad, Llama-3-8B MLP-up: X[8192,4096] W[14336,4096] dY[8192,14336] bf16; "
                "1D-16 activations/grads, 2D 16x16 weights, E4M3 inner + FP32 tensorwise outer scale, "
                "RHT-16 on wgrad operands, SR on gradients",
    "shape": {"M": M, "K": K, "N": N},
    "l2_policy": "per-step inputs (400 MB) exceed the 126 MB L2; no explicit flush",
    "parallelism": "data-parallel replicas, one process per GPU, no data-path collective",
    "overlap": "the 13 kernels of a step run back to back on one stream, each launched with programmatic stream "
               "serialisation (its launch overlaps the tail of its predecessor; ALTOB200_PDL=0 turns that off)",
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# DRAM bytes (read + write) per GEMM launch at the default shape: ncu dram__bytes_read.sum +
# dram__bytes_write.sum from a one-pass capture of this command, mean of the step's three launches
# (fprop 113.3 + 192.4, dgrad 127.5 + 47.2, wgrad 85.2 + 80.5 MB read + written).  Part of each output is
# still in the write-back L2 when the kernel ends; part of each input is found there.
GEMM_DRAM_BYTES_PER_LAUNCH = (113.3e6 + 192.4e6 + 127.5e6 + 47.2e6 + 85.2e6 + 80.5e6) / 3
# algorithmic bytes per launch: codes + packed scales of both operands + bf16 output, mean of the three
GEMM_ALGORITHMIC_BYTES_PER_LAUNCH = (52.0e6 + 234.9e6 + 84.9e6 + 117.4e6 + 99.1e6 + 67.1e6) / 3
NOMINAL_FP4_TFLOPS = 9000.0  # dense FP4 tensor peak of the part (datasheet)
SUSTAINED_SECONDS = 3.0      # length of the sustained leg
CPU_SAMPLE_ROWS = 2048     # token rows of the CPU sample
CPU_SAMPLE_FEATS = 2048    # output features (rows of W) of the CPU sample
CPU_BASELINE_REPS = 10     # steps of the sample timed for `cpu_baseline` (10-20 s of host work in all)


def load_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ------------------------------------------------------------------------------------------
# clocks sampler (nvidia-smi, read only)
# ------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and clock-event reasons through NVML (read-only queries) every
    few milliseconds from a thread, for the duration of the timed region."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            # CUDA_VISIBLE_DEVICES remaps indices: resolve through the PCI bus id of the torch device
            bus = torch.cuda.get_device_properties(self.index).pci_bus_id \
                if hasattr(torch.cuda.get_device_properties(self.index), "pci_bus_id") else None
            self._h = None
            if bus is not None:
                for i in range(pynvml.nvmlDeviceGetCount()):
                    h = pynvml.nvmlDeviceGetHandleByIndex(i)
                    if pynvml.nvmlDeviceGetPciInfo(h).bus == bus:
                        self._h = h
                        break
            if self._h is None:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self._max = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                clk = nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._h)
                pw = nv.nvmlDeviceGetPowerUsage(self._h) / 1000.0
                self.samples.append((clk, rs, pw))
            except Exception:
                pass
            time.sleep(0.005)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = sorted(c for c, _, _ in self.samples)
        reasons = sorted(n for n, bit in self.REASONS.items() if any(r & bit for _, r, _ in self.samples))
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self._max, "reasons": reasons, "samples": len(sm),
                "power_w_max": max(p for _, _, p in self.samples)}


# ------------------------------------------------------------------------------------------
# CPU arm: the oracle (port of the reference's PyTorch emulation path) on a row sample
# ------------------------------------------------------------------------------------------
def cpu_sample_inputs(rows: int):
    g = torch.Generator().manual_seed(0)
    x = torch.randn(rows, K, generator=g).bfloat16()
    nf = CPU_SAMPLE_FEATS
    w = (torch.randn(nf, K, generator=g) * 0.02).bfloat16()
    dy = (torch.randn(rows, nf, generator=g) * 1e-3).bfloat16()
    rn = torch.randint(0, 2 ** 32, (2, rows, nf // 2), generator=g, dtype=torch.int64)
    rm = torch.randint(0, 2 ** 32, (2, nf, rows // 2), generator=g, dtype=torch.int64)
    return x, w, dy, rn, rm


def cpu_step(inputs, W_had):
    from oracle import alto_oracle as O
    x, w, dy, rn, rm = inputs
    return O.nvfp4_linear(x, w, dy, use_2dblock_w=True, use_outer=True, W_had=W_had, rand_dy_n=rn, rand_dy_m=rm)


def cpu_baseline(rows: int, reps: int = 1):
    from oracle import alto_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    W_had, _, _ = O.random_hadamard(16, torch.Generator().manual_seed(0))
    inputs = cpu_sample_inputs(rows)
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_step(inputs, W_had)
    dt = (time.perf_counter() - t0) / reps
    flops = 3 * 2 * rows * CPU_SAMPLE_FEATS * K
    return {"value": flops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"{rows} of {M} token rows x {CPU_SAMPLE_FEATS} of {N} output features (K={K} full): quantize + "
                      f"Hadamard + dequantize + fp32 matmuls of one fwd+dgrad+wgrad step, {dt:.2f} s per step, {reps} steps timed"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import alto_oracle as O
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    W_had, _, _ = O.random_hadamard(16, torch.Generator().manual_seed(0))
    rows = CPU_SAMPLE_ROWS
    inputs = cpu_sample_inputs(rows)
    for _ in range(args.warmup):
        cpu_step(inputs, W_had)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(inputs, W_had)
    dt = time.perf_counter() - t0
    flops = 3 * 2 * rows * CPU_SAMPLE_FEATS * K * args.steps
    val = flops / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "nvfp4 (e2m1 codes, e4m3 scales, fp32 accumulate)", "data": "synthetic",
        "config": CONFIG,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"each step = {rows} of {M} token rows x {CPU_SAMPLE_FEATS} of {N} output features, CPU "
                                   "restatement of the reference's PyTorch emulation path (quantize, Hadamard, "
                                   "dequantize, fp32 matmul)"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
class KernelTimer:
    """Wraps the C-ABI launch wrappers with CUDA events on the launching (current) stream."""

    def __init__(self):
        self.records = []
        self.enabled = False
        self.launches = 0

    def wrap(self, mod, name, family, work):
        orig = getattr(mod, name)
        timer = self

        def wrapped(*a, **kw):
            timer.launches += 1
            if not timer.enabled:
                return orig(*a, **kw)
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record()
            r = orig(*a, **kw)
            e1.record()
            timer.records.append((family, work(*a, **kw), e0, e1))
            return r

        setattr(mod, name, wrapped)

    def count(self, mod, name):
        """Counts launches of a wrapper whose kernel is too small to be worth timing."""
        orig = getattr(mod, name)
        timer = self

        def wrapped(*a, **kw):
            timer.launches += 1
            return orig(*a, **kw)

        setattr(mod, name, wrapped)

    def summary(self):
        out = {}
        for fam, work, e0, e1 in self.records:
            d = out.setdefault(fam, {"launches": 0, "ms": 0.0, "work": 0.0})
            d["launches"] += 1
            d["ms"] += e0.elapsed_time(e1)
            d["work"] += work
        return out


def run_ours(args):
    from alto_b200 import _lib as L
    from alto_b200 import nvfp4 as NV

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    peaks, peak_src = load_peaks()
    NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)

    timer = KernelTimer()
    fp4_bytes = lambda r, c: r * c * (2 + 0.5 + 1.0 / 16)  # noqa: E731  bf16 in, codes + scales out
    timer.wrap(L, "amax", "amax", lambda x, *a, **k: x.numel() * 2.0)
    timer.wrap(L, "quantize_rowwise", "quantize_rowwise", lambda x, *a, **k: fp4_bytes(*x.shape))
    timer.wrap(L, "quantize_colwise", "quantize_colwise", lambda x, *a, **k: fp4_bytes(*x.shape))
    timer.wrap(L, "quantize_2d", "quantize_2d",
               lambda x, *a, **k: x.numel() * (2 + 2 * (0.5 + 1.0 / 16)))
    timer.wrap(L, "gemm_blockscaled", "gemm", lambda fa, fb, m, n, k, *a, **kw: 2.0 * m * n * k)
    timer.wrap(L, "gemm_mxfp4_two_level", "gemm", lambda m, n, k, *a, **kw: 2.0 * m * n * k)
    timer.count(L, "philox_tile")   # the two 16 KB random-word tables of a step's stochastic-rounding quantizers

    g = torch.Generator(device=dev).manual_seed(rank)
    gw = torch.Generator(device=dev).manual_seed(12345)  # identical weights on every rank
    x = torch.randn(M, K, generator=g, device=dev, dtype=torch.float32).bfloat16().requires_grad_(True)
    w = (torch.randn(N, K, generator=gw, device=dev, dtype=torch.float32) * 0.02).bfloat16().requires_grad_(True)
    dy = (torch.randn(M, N, generator=g, device=dev, dtype=torch.float32) * 1e-3).bfloat16()

    def step():
        x.grad = None
        w.grad = None
        if args.recipe == "nvfp4":
            y = NV._to_nvfp4_then_scaled_mm(x, w, False, True, True, use_outer_scale=True, use_hadamard=True)
        else:   # profiling captures of the other recipes on a small case; never the headline
            from alto_b200 import mxfp4 as MXR
            y = MXR._to_mxfp4_then_scaled_mm(x, w, False, True, True, False, "none", True,
                                             args.recipe == "mxfp4_two_level")
        y.backward(dy)
        return y

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    n0 = timer.launches
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    launches = timer.launches - n0
    st, detail = L.status_read()
    if st != 0:
        raise RuntimeError(f"device-side wait timed out: {detail}")
    t = torch.tensor([ms], device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    value = world * FLOPS_PER_STEP * args.steps / (ms * 1e-3) / 1e12

    # ---- per-kernel timing pass (events around every launch; not part of the headline) ----
    # The quantizer/GEMM stream overlap is switched off here so that every kernel is timed alone.
    from alto_b200 import _linear as E
    overlap = E.OVERLAP
    E.OVERLAP = False
    timer.enabled = True
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    timer.enabled = False
    E.OVERLAP = overlap
    fam = timer.summary()
    kernels = {}
    for name, d in fam.items():
        avg_ms = d["ms"] / d["launches"]
        if name == "gemm":
            kernels[name] = {"launches_per_step": d["launches"] // args.steps, "avg_ms": avg_ms,
                             "tflops": d["work"] / d["launches"] / (avg_ms * 1e-3) / 1e12}
        else:
            kernels[name] = {"launches_per_step": d["launches"] // args.steps, "avg_ms": avg_ms,
                             "gbs": d["work"] / d["launches"] / (avg_ms * 1e-3) / 1e9,
                             "frac_of_hbm_peak": d["work"] / d["launches"] / (avg_ms * 1e-3) / 1e9 / peaks["hbm_gbs"]}
    # Denominator of the tensor roofline: the dense FP4 proxy 4 x measured cuBLAS bf16 throughput.  The
    # measured file holds a burst figure (a kernel timed alone at full clocks) and a sustained one (seconds
    # under the power cap); which of them applies is decided by the clocks this run actually saw.
    burst_peak, sustained_peak = 4.0 * peaks["bf16_tflops"], 4.0 * peaks["bf16_tflops_sustained"]
    at_max_clock = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz")
                        and clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"])
    fp4_peak = burst_peak if (at_max_clock or clocks is None or not clocks.get("sm_mhz")) else sustained_peak
    default_shape = (M, K, N) == (8192, 4096, 14336)
    gemm_tf = kernels["gemm"]["tflops"]
    roofline = {"bound": "tensor", "achieved": gemm_tf, "peak": fp4_peak, "unit": "TFLOP/s",
                "frac": gemm_tf / fp4_peak, "traffic": GEMM_DRAM_BYTES_PER_LAUNCH if default_shape else None,
                "frac_of_burst_proxy": gemm_tf / burst_peak, "frac_of_sustained_proxy": gemm_tf / sustained_peak,
                "frac_of_nominal": gemm_tf / NOMINAL_FP4_TFLOPS,
                "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one-pass capture of this "
                                  "command, mean of the step's three GEMM launches; algorithmic operand + output "
                                  f"bytes per launch {GEMM_ALGORITHMIC_BYTES_PER_LAUNCH:.4g}",
                "kernel": "gemm_blockscaled_pair_kernel<NVF4,bf16> (tcgen05 cta_group::2; 3 launches per step, 962 GFLOP each)",
                "peak_source": f"4 x {peak_src} cuBLAS bf16 throughput (dense FP4 proxy), "
                               f"{'burst' if fp4_peak == burst_peak else 'sustained'} figure because the median SM "
                               f"clock of the timed region was {'at' if fp4_peak == burst_peak else 'below'} the maximum; "
                               f"nominal dense FP4 {NOMINAL_FP4_TFLOPS:.0f}"}

    # ---- the other recipes the target names, same shape, device-timed (not the headline); before the
    # seconds-long leg below, which leaves the GPU power-capped for a while ----
    extra = {}
    if default_shape and not args.no_extra:
        from alto_b200 import mxfp4 as MX

        def time_fn(fn, reps=10):
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(reps):
                fn()
            b.record()
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps

        def mx_step(macro):
            x.grad = None
            w.grad = None
            MX._to_mxfp4_then_scaled_mm(x, w, False, True, True, False, "none", True, macro).backward(dy)

        for name, macro in (("mxfp4_linear", False), ("mxfp4_two_level_linear", True)):
            t_ms = time_fn(lambda: mx_step(macro))
            extra[name] = {"ms_per_step": t_ms, "tflops": FLOPS_PER_STEP / (t_ms * 1e-3) / 1e12,
                           "recipe": "MXFP4 1D-32 activations/grads, 2D 32x32 weights, RHT-16 on wgrad operands, SR on "
                                     "gradients" + (", 128 macro-block two-level scale (folded in the GEMM)" if macro else "")}
        NV.HadamardFactory.configure(block_size=16, randomized=True, dtype=torch.float32, seed=0)

    # ---- sustained leg: the same step back to back for seconds, clocks sampled throughout ----
    sustained = None
    if not args.no_sustained:
        barrier()
        samp2 = ClockSampler(local)
        if rank == 0:
            samp2.start()
        n_sus = 0
        es, ee = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        chunk = max(50, int(0.25 / max(ms / args.steps * 1e-3, 1e-6)))   # ~0.25 s of steps between host checks
        t_wall = time.perf_counter()
        es.record()
        while True:
            for _ in range(chunk):
                step()
            n_sus += chunk
            torch.cuda.synchronize()
            if time.perf_counter() - t_wall >= SUSTAINED_SECONDS:
                break
        ee.record()
        torch.cuda.synchronize()
        sus_ms = es.elapsed_time(ee)
        c2 = samp2.stop() if rank == 0 else None
        ts = torch.tensor([sus_ms / n_sus], device=dev)
        if dist is not None:
            dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        per_step = float(ts.item())
        sustained = {"seconds": sus_ms * 1e-3, "steps": n_sus, "ms_per_step": per_step,
                     "value": world * FLOPS_PER_STEP / (per_step * 1e-3) / 1e12, "unit": UNIT, "clocks": c2,
                     "ms_x_median_mhz": (per_step * c2["sm_mhz"]) if (c2 and c2.get("sm_mhz")) else None,
                     "frac_of_sustained_proxy_whole_step": FLOPS_PER_STEP / (per_step * 1e-3) / 1e12 / sustained_peak}

    # ---- end to end through the public API with host buffers ----
    # one pinned buffer per direction (x | W | dY in, y | dX | dW out); the per-tensor views serve the serial leg
    n_x, n_w, n_dy = x.numel(), w.numel(), dy.numel()
    hin = torch.empty(n_x + n_w + n_dy, dtype=torch.bfloat16).pin_memory()
    hout = torch.empty(n_dy + n_x + n_w, dtype=torch.bfloat16).pin_memory()
    xh, wh, dyh = hin[:n_x].view(M, K), hin[n_x:n_x + n_w].view(N, K), hin[n_x + n_w:].view(M, N)
    yh, dxh, dwh = hout[:n_dy].view(M, N), hout[n_dy:n_dy + n_x].view(M, K), hout[n_dy + n_x:].view(N, K)
    xh.copy_(x.detach())
    wh.copy_(w.detach())
    dyh.copy_(dy)

    def e2e_step():
        with torch.no_grad():
            x.copy_(xh, non_blocking=True)
            w.copy_(wh, non_blocking=True)
            dy.copy_(dyh, non_blocking=True)
        y = step()
        yh.copy_(y.detach(), non_blocking=True)
        dxh.copy_(x.grad, non_blocking=True)
        dwh.copy_(w.grad, non_blocking=True)

    def timed(loop):
        barrier()
        e0.record()
        loop(args.steps)
        e1.record()
        barrier()
        tt = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    e2e_step()
    serial_ms = timed(lambda n: [e2e_step() for _ in range(n)])

    # The same work with the copies of neighbouring steps overlapped, as a caller feeding batches from
    # host memory would run it: three streams and two sets of device buffers; step i computes while the
    # inputs of step i+1 arrive and the results of step i-1 leave.  Every step still copies its own
    # inputs from pinned host memory and its own three results back.  Each direction moves one
    # contiguous buffer per step (x | W | dY in, y | dX | dW out); --e2e-copies 3 moves the three
    # tensors separately (no measurable difference on one box: the leg is bound by the PCIe link).
    comp = torch.cuda.current_stream(dev)
    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    din = [torch.empty(n_x + n_w + n_dy, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dout = [torch.empty(n_dy + n_x + n_w, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    sets = [(d[:n_x].view(M, K).requires_grad_(True), d[n_x:n_x + n_w].view(N, K).requires_grad_(True),
             d[n_x + n_w:].view(M, N)) for d in din]
    consumed = [None, None]
    left = [None, None]

    def pipelined(n):
        for i in range(n):
            b = i & 1
            xs, ws, dys = sets[b]
            with torch.cuda.stream(s_in):
                if consumed[b] is not None:
                    s_in.wait_event(consumed[b])
                if args.e2e_copies == 1:
                    din[b].copy_(hin, non_blocking=True)
                else:   # one copy per tensor, for comparison on the same box
                    for lo, hi in ((0, n_x), (n_x, n_x + n_w), (n_x + n_w, n_x + n_w + n_dy)):
                        din[b][lo:hi].copy_(hin[lo:hi], non_blocking=True)
                arrived = torch.cuda.Event()
                arrived.record(s_in)
            comp.wait_event(arrived)
            if left[b] is not None:
                comp.wait_event(left[b])     # the results of step i-2 have left this output buffer
            xs.grad = None
            ws.grad = None
            y = NV._to_nvfp4_then_scaled_mm(xs, ws, False, True, True, use_outer_scale=True, use_hadamard=True)
            y.backward(dys)
            o = dout[b]
            with torch.no_grad():
                o[:n_dy].view(M, N).copy_(y)
                o[n_dy:n_dy + n_x].view(M, K).copy_(xs.grad)
                o[n_dy + n_x:].view(N, K).copy_(ws.grad)
            done = torch.cuda.Event()
            done.record(comp)
            consumed[b] = done
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                if args.e2e_copies == 1:
                    hout.copy_(o, non_blocking=True)
                else:
                    for lo, hi in ((0, n_dy), (n_dy, n_dy + n_x), (n_dy + n_x, n_dy + n_x + n_w)):
                        hout[lo:hi].copy_(o[lo:hi], non_blocking=True)
                gone = torch.cuda.Event()
                gone.record(s_out)
                left[b] = gone
        comp.wait_stream(s_in)
        comp.wait_stream(s_out)

    pipelined(2)
    e2e_ms = timed(pipelined)
    h2d = hin.numel() * 2
    d2h = hout.numel() * 2
    e2e = {"value": world * FLOPS_PER_STEP * args.steps / (e2e_ms * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms / args.steps,
           "how": "public autograd entry point; per step H2D of x, W, dY from pinned host memory and D2H of y, dX, dW; "
                  "copies of neighbouring steps overlap the compute (3 streams, 2 sets of device buffers, one contiguous "
                  "copy per direction and step)",
           "serial_ms_per_step": serial_ms / args.steps,
           "serial_value": world * FLOPS_PER_STEP * args.steps / (serial_ms * 1e-3) / 1e12}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "nvfp4 (e2m1 codes, e4m3 scales, fp32 accumulate)", "data": "synthetic", "config": CONFIG,
        "frac_of_fp4_peak": value / world / fp4_peak, "roofline": roofline, "kernels": kernels, "e2e": e2e,
        "gpu_launches": launches, "clocks": clocks, "sustained": sustained, "extra": extra,
    }
    if world > 1 and not args.no_sharded:
        line["sharded"] = run_sharded(dist, dev, rank, world)
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(CPU_SAMPLE_ROWS, CPU_BASELINE_REPS)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------
# N > 1: the two configurations with a real exchange step (expert-parallel MoE, column-sharded linear)
# ------------------------------------------------------------------------------------------
def run_sharded(dist, dev, rank, world):
    """After the replica headline: (a) the MXFP4 MoE layer at the GPT-OSS-20B shape (32 experts, top-4, hidden
    = intermediate = 2880, 16384 tokens in all; 2-D weight blocks with the 128 macro-block two-level scale,
    RHT-32 on the token-axis operands, SR on gradients), experts and tokens split over the ranks, dispatch
    and combine by NCCL all-to-all; (b) the MXFP8 linear 8192 x 4096 x 4096 with W split by output features and
    dX all-reduced.  Total work is fixed (strong scaling).  Times are CUDA events, slowest rank; parity is each
    rank's forward against the same rows computed on that GPU alone with all experts / its weight shard."""
    from alto_b200 import distributed as D
    from alto_b200 import mxfp8 as M8
    from alto_b200.grouped import _quantize_then_mxfp_scaled_grouped_mm as mx4
    from alto_b200.hadamard import HadamardFactory
    from alto_b200.swiglu import swiglu

    def gmm(A, B, offs):
        HadamardFactory.configure(block_size=32, randomized=True, dtype=torch.float32, seed=0)
        return mx4(A, B, offs, False, True, True, False, True, "none", True)

    def moe(x, ids, scores, W13, W2, dispatcher):
        xl, offs, st = dispatcher.dispatch(x, ids)
        h = gmm(xl, W13.transpose(-2, -1), offs)
        y = gmm(swiglu(h), W2.transpose(-2, -1), offs)
        return dispatcher.combine(y, st, scores)

    def step_time(fn, reps=5):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def all_ok(flag):
        t = torch.tensor([1 if flag else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    T, Dm, E, k = 16384, 2880, 32, 4
    g = torch.Generator(device=dev).manual_seed(0)
    logits = torch.randn(T, E, generator=g, device=dev)
    x_all = torch.randn(T, Dm, generator=g, device=dev).bfloat16()
    W13 = (torch.randn(E, 2 * Dm, Dm, generator=g, device=dev) * 0.02).bfloat16()
    W2 = (torch.randn(E, Dm, Dm, generator=g, device=dev) * 0.02).bfloat16()
    scores_all, ids_all = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    n, El = T // world, E // world
    x = x_all[rank * n:(rank + 1) * n].clone().requires_grad_(True)
    ids, scores = ids_all[rank * n:(rank + 1) * n], scores_all[rank * n:(rank + 1) * n].bfloat16()
    w13 = W13[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    w2 = W2[rank * El:(rank + 1) * El].clone().requires_grad_(True)
    ep = D.ExpertParallelDispatcher(E)
    out = moe(x, ids, scores, w13, w2, ep)
    one = D.ExpertParallelDispatcher.__new__(D.ExpertParallelDispatcher)
    one.group, one.world, one.rank, one.num_experts, one.local_experts, one.align = None, 1, 0, E, E, 128
    with torch.no_grad():
        ep_ok = all_ok(torch.equal(out, moe(x.detach(), ids, scores, W13, W2, one)))
    del W13, W2, x_all
    g_out = torch.ones_like(out) * 1e-3

    def moe_step():
        x.grad = w13.grad = w2.grad = None
        moe(x, ids, scores, w13, w2, ep).backward(g_out)

    t_moe = step_time(moe_step)
    ep_ok = ep_ok and all_ok(bool(torch.isfinite(x.grad).all() and torch.isfinite(w13.grad).all()))
    flop_moe = 3 * 2 * T * k * (2 * Dm * Dm + Dm * Dm)
    # rows that leave a rank: every routed row whose expert lives elsewhere, both ways, forward and backward
    a2a_bytes = int(T * k * Dm * 2 * (world - 1) / world) * 4

    fn = lambda a, b: M8._to_mxfp8_then_scaled_mm(a, b, "e4m3", False, False, True)  # noqa: E731
    g = torch.Generator(device=dev).manual_seed(1)
    xs = torch.randn(8192, 4096, generator=g, device=dev).bfloat16().requires_grad_(True)
    W = (torch.randn(4096, 4096, generator=g, device=dev) * 0.02).bfloat16()
    dy = (torch.randn(8192, 4096, generator=g, device=dev) * 1e-3).bfloat16()
    nw = 4096 // world
    ws = D.shard_rows(W).clone().requires_grad_(True)
    dys = dy[:, rank * nw:(rank + 1) * nw].contiguous()
    ys = D.column_sharded_linear(xs, ws, fn)
    with torch.no_grad():
        col_ok = all_ok(torch.equal(ys, fn(xs.detach(), W[rank * nw:(rank + 1) * nw])))

    def lin_step(overlap=False):
        xs.grad = ws.grad = None
        D.column_sharded_linear(xs, ws, fn, overlap_dx_reduction=overlap).backward(dys)

    t_lin = step_time(lin_step)
    # the same step with the dX all-reduce started right after the dgrad GEMM, beside the wgrad side
    t_lin_overlap = step_time(lambda: lin_step(True))
    col_ok = col_ok and all_ok(bool(torch.isfinite(xs.grad).all() and torch.isfinite(ws.grad).all()))
    return {"scaling": "strong (total work fixed)",
            "ep_moe_ms": t_moe, "ep_moe_tflops": flop_moe / (t_moe * 1e-3) / 1e12, "ep_parity_ok": ep_ok,
            "ep_recipe": "MXFP4, 2D weight blocks + 128 macro-block two-level scale, RHT-32, SR; W13 + SwiGLU + W2, "
                         "fwd + dgrad + wgrad with dispatch and combine",
            "a2a_bytes": a2a_bytes,
            "col_ms": t_lin, "col_tflops": 3 * 2 * 8192 * 4096 * 4096 / (t_lin * 1e-3) / 1e12, "col_parity_ok": col_ok,
            "col_ms_allreduce_beside_wgrad": t_lin_overlap,
            "allreduce_bytes": 8192 * 4096 * 2}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sustained", action="store_true", help="skip the seconds-long sustained leg")
    ap.add_argument("--no-extra", action="store_true", help="skip the MXFP4 recipes at the same shape")
    ap.add_argument("--no-sharded", action="store_true", help="N > 1: skip the expert-parallel and column-sharded runs")
    ap.add_argument("--e2e-copies", type=int, default=1, choices=[1, 3],
                    help="host<->device copies per direction and step in the end-to-end leg (1: one contiguous buffer)")
    ap.add_argument("--recipe", default="nvfp4", choices=["nvfp4", "mxfp4", "mxfp4_two_level"],
                    help="nvfp4 is the headline; the others exist for profiling captures of their kernels")
    ap.add_argument("--shape", default=None, metavar="M,K,N",
                    help="run the same step at another shape (profiling captures on a small case); the "
                         "headline workload is the default")
    args = ap.parse_args()
    if args.shape:
        global M, K, N, FLOPS_PER_STEP
        M, K, N = (int(v) for v in args.shape.split(","))
        FLOPS_PER_STEP = 3 * 2 * M * N * K
        CONFIG["shape"] = {"M": M, "K": K, "N": N}
        CONFIG["workload"] = f"NOT the headline workload: same NVFP4 step at M={M} K={K} N={N}"
    if args.recipe != "nvfp4":
        CONFIG["workload"] = f"NOT the headline workload: {args.recipe} step at M={M} K={K} N={N}"
        args.no_extra = True
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
