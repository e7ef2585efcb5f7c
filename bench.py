#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path through libluxgpu_backend_cuda.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

N = 1   workload "int4_g128_gemv_14336x4096" (benchmark configuration 2, the one the
        headline metric "qmatmul GEMV weight GB/s" is quoted on): one step = one decode
        GEMV y[1,14336] = x[1,4096] . dequant(W)^T.  The weights rotate through a pool
        of device copies larger than L2, so every step streams from HBM.
N > 1   workload "llama70b_mlp_tp" (configuration 5): one step = the tensor-parallel
        FFN (column-parallel gate_up + SwiGLU, row-parallel down, all-reduce of the f16
        partials) at batch 1; total work is fixed as N grows (strong scaling).  `value` at
        N = 1 and at N > 1 therefore belong to DIFFERENT workloads and must not be divided
        by one another: every N > 1 line carries its own one-GPU time of the same FFN,
        measured on rank 0 of the same box in the same harness (`tp1_us_same_box`), and the
        strong-scaling efficiency against it; the N = 1 line carries the same block as the
        extra key `ffn70b_cfg5_tp1`.  Every line also carries `parity_rel_l2` of a step that
        included the collective against the CPU oracle's sharded computation, and
        `ranks_identical`.

`value` is the whole-job weight bandwidth with inputs resident in HBM, timed with CUDA
events on the launching stream (max over ranks).  `e2e` is the same metric through the
host-pointer C-ABI call (x copied host->device and y device->host inside the timed
region; weights are model state and stay on the device).  `roofline` describes the
dominant kernel; `cpu_baseline` is the reference's shader arithmetic restated for host
cores (oracle/cpu_baseline.c; the WGSL itself needs a WebGPU runtime) timed on this
machine's cores, all of them and one.
Extra keys report the int8 GEMV (configuration 1) and the M=512 tcgen05 GEMM
(configuration 3, TFLOP/s against the measured bf16 peak).
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
# the CPU baseline's OpenMP workers sleep between parallel regions instead of spinning on the cores
# the GPU arm's host thread needs (read by the OpenMP runtime when the oracle libraries load)
os.environ.setdefault("OMP_WAIT_POLICY", "passive")

import numpy as np  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read.sum + dram__bytes_write.sum of ONE config-2 launch in the ncu capture summarised
# in profiles/qgemv_i4_g128_units_fx_config2.md.  Reported as `traffic` only while the kernel the
# library launches is the one that was captured; otherwise `traffic` is null.
NCU_TRAFFIC_CONFIG2 = {"kernel": "lux_qgemv_i4_g128_units_fx", "bytes": 30554795,
                       "source": "profiles/qgemv_i4_g128_units_fx_config2.md"}
NOMINAL_HBM_GBS = 8000.0          # the benchmark specification's "~8 TB/s"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_HBM_GBS = 6650.0         # used only when MEASURED_PEAKS.json is absent
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return dict(hbm=float(p["hbm_gbs"]), bf16=float(p["bf16_tflops"]),
                    bf16_sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), source="measured")
    except Exception:
        return dict(hbm=FALLBACK_HBM_GBS, bf16=FALLBACK_BF16_TFLOPS, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the GPU is under load."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread:
            self._stop.set()
            self._thread.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ----------------------------------------------------------------------------------------
# device-side helpers
# ----------------------------------------------------------------------------------------

class Rig:
    """Plugin context bound to a torch stream, so CUDA events see the kernels."""

    eager = False       # time_graph: enqueue the timed launches one by one instead of replaying a graph

    def __init__(self, local_rank: int, tunes=()):
        import torch
        from webgpu_b200 import backend as B

        self.torch, self.B = torch, B
        torch.cuda.set_device(local_rank)
        self.backend = B.load()
        for kv in tunes:
            key, _, val = kv.partition("=")
            self.backend.tune(key, int(val))
        self.ctx = self.backend.create_context(local_rank)
        self.stream = torch.cuda.Stream()
        self.ctx.set_stream(self.stream.cuda_stream)

    def pool(self, layer, min_bytes):
        """Device copies of one layer, enough of them to exceed `min_bytes`."""
        first = self.ctx.upload_layer(layer)
        n = max(2, -(-min_bytes // first.weight_bytes))
        return [first] + [self.ctx.upload_layer(layer) for _ in range(n - 1)]

    def time_graph(self, launch, n_variants, steps, warmup, graph_len=None, align=None):
        """Times exactly `steps` launches (launch(i) enqueues one on self.stream) as CUDA-graph
        replays: one graph of all of them up to 240 steps, else graphs of a whole number of
        rotations.  The timed region opens behind a short spin kernel, so that the host's
        submission latency of the first replay is not counted as device time; a synchronize
        stands on both sides.  `align` (multi-GPU) is enqueued behind the spin kernel and before the
        first event: one more untimed step whose collective brings the ranks' streams to the same
        point, so that the timed region does not open with one rank waiting for another that is
        still capturing its graph.  Returns (seconds per step, graph)."""
        torch = self.torch
        if graph_len:
            glen = max(1, min(graph_len, steps))
        elif steps <= 240:
            glen = steps
        else:
            glen = max(n_variants, 240 // n_variants * n_variants)
        with torch.cuda.stream(self.stream):
            for i in range(max(warmup, 3)):
                launch(i)
            self.stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=self.stream, capture_error_mode="relaxed"):
                for i in range(glen):
                    launch(i)
            rem = steps % glen
            g2 = None
            if rem:
                g2 = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g2, stream=self.stream, capture_error_mode="relaxed"):
                    for i in range(rem):
                        launch(i)
            g.replay()
            self.stream.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            torch.cuda._sleep(400_000 if align else 200_000)   # 0.1-0.2 ms of spinning: what follows queues up behind it
            if align is not None:
                align()
            e0.record(self.stream)
            if self.eager:
                for i in range(steps):
                    launch(i)
            else:
                for _ in range(steps // glen):
                    g.replay()
                if g2 is not None:
                    g2.replay()
            e1.record(self.stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / steps, g


def algorithmic_bytes(layer, M, x_item, y_item, swiglu=False):
    n_out = layer.N // 2 if swiglu else layer.N
    return layer.weight_bytes + M * layer.K * x_item + M * n_out * y_item


# ----------------------------------------------------------------------------------------
# N = 1: configuration 2 (headline), plus configurations 1 and 3 as extra keys
# ----------------------------------------------------------------------------------------

def bench_single(args, peaks):
    from oracle import oracle as orc      # parity spot checks after the timed regions
    from webgpu_b200 import synth

    rig = Rig(0, args.tune)
    B, ctx, torch = rig.B, rig.ctx, rig.torch
    sampler = ClockSampler(0)

    # ---- configuration 2: int4 g128 GEMV 14336 x 4096, f16 ------------------------------
    x, layer = synth.config2()
    pool = rig.pool(layer, int(2.9 * L2_BYTES))
    xb = ctx.upload(x)
    yb = ctx.alloc(layer.N * 2)
    d_x, d_y = B.F16, B.F16

    def launch(i):
        ctx.qmatmul(xb, pool[i % len(pool)], yb, 1, d_x, d_y, flags=B.FLAG_NO_SYNC)

    sampler.start()
    l0 = rig.backend.launch_count()
    sec, graph = rig.time_graph(launch, len(pool), args.steps, args.warmup)
    kernel = rig.backend.last_kernel_name()          # the library picks a kernel per shape
    captured = rig.backend.launch_count() - l0
    # the same GEMV as a long chain (2400 launches): with programmatic dependent launch every kernel's
    # start overlaps its predecessor's drain, and the two ends of the chain weigh nothing.  Reported
    # beside the headline so that the launch-overlap effect can be told from the kernel itself.
    sec_chain = sec
    if args.steps < 2400:
        sec_chain, _ = rig.time_graph(launch, len(pool), 2400, 5)
    # keep the same load running a little longer so that the clock sampler sees it
    t_end = time.time() + 0.4
    with torch.cuda.stream(rig.stream):
        while time.time() < t_end:
            graph.replay()
            rig.stream.synchronize()
    clocks = sampler.stop()
    clocks["window"] = "timed region plus 0.4 s of the identical load"

    wbytes = layer.weight_bytes
    abytes = algorithmic_bytes(layer, 1, 2, 2)
    value = wbytes / sec / 1e9
    achieved = abytes / sec / 1e9

    y = yb.to_host(np.float16, (1, layer.N))          # what was just timed; checked after the e2e loop

    # ---- e2e: host x -> device, kernel, y -> host, through the host-pointer C-ABI call ---
    out = np.empty((1, layer.N), np.float16)
    ctx.set_stream(None)
    # a decode loop marshals the call's arguments once per layer (fixed host buffers): qmatmul_host_bound
    calls = [ctx.qmatmul_host_bound(x, L, out) for L in pool]
    for i in range(50):                                # the first calls after the graph replays run cold
        calls[i % len(calls)]()
    n_e2e = min(max(args.steps, 500), 2000)
    t0 = time.perf_counter()
    for i in range(n_e2e):
        calls[i % len(calls)]()
    e2e_sec = (time.perf_counter() - t0) / n_e2e
    ctx.set_stream(rig.stream.cuda_stream)

    # parity spot check of the timed GEMV and of the last e2e result.  The oracle runs only now:
    # its OpenMP workers keep spinning for a while after a parallel region, which would sit on the
    # host cores during the host-latency-bound e2e loop above.
    ref = orc.qmatmul(x, *layer.triple, bits=4, group=128)
    parity = orc.rel_l2(y, ref)
    parity_e2e = orc.rel_l2(out, ref)

    # ---- CPU baseline: the reference's arithmetic on the host cores, bounded sample --------------
    from oracle import cpu_baseline as cb
    cores = cb.num_procs()

    def cpu_time(threads, budget_s):
        cb.qmatmul_i4(x, *layer.triple, threads=threads)
        n, t0 = 0, time.perf_counter()
        while n < 400 and time.perf_counter() - t0 < budget_s:
            cb.qmatmul_i4(x, *layer.triple, threads=threads)
            n += 1
        return (time.perf_counter() - t0) / n, n

    cpu_sec, reps = cpu_time(0, 8.0)
    cpu_sec1, reps1 = cpu_time(1, 4.0)

    extra = {}
    # ---- configuration 1: int8 g32 GEMV 4096 x 4096, f32 ----------------------------------
    try:
        x1, l1 = synth.config1()
        pool1 = rig.pool(l1, int(2.9 * L2_BYTES))
        xb1, yb1 = ctx.upload(x1), ctx.alloc(l1.N * 4)
        sec1, _ = rig.time_graph(lambda i: ctx.qmatmul(xb1, pool1[i % len(pool1)], yb1, 1, B.F32, B.F32,
                                                       flags=B.FLAG_NO_SYNC), len(pool1), args.steps, args.warmup)
        ab1 = algorithmic_bytes(l1, 1, 4, 4)
        err1 = orc.rel_l2(yb1.to_host(np.float32, (1, l1.N)), orc.qmatmul(x1, *l1.triple, bits=8, group=32))
        extra["gemv_int8_cfg1"] = {
            "kernel": rig.backend.last_kernel_name(),
            "weight_gbs": l1.weight_bytes / sec1 / 1e9, "total_gbs": ab1 / sec1 / 1e9, "us": sec1 * 1e6,
            "frac_of_measured_hbm": ab1 / sec1 / 1e9 / peaks["hbm"], "frac_of_nominal_8tbs": ab1 / sec1 / 1e9 / NOMINAL_HBM_GBS,
            "rel_l2_vs_oracle": err1}
        del pool1
    except Exception as e:  # keep the headline line even if an extra fails
        extra["gemv_int8_cfg1"] = {"error": repr(e)}
    # ---- configuration 3: int4 g128 GEMM M=512, bf16, tcgen05 -----------------------------
    try:
        x3, l3 = synth.config3()
        pool3 = rig.pool(l3, int(2.9 * L2_BYTES))
        xb3, yb3 = ctx.upload(x3), ctx.alloc(512 * l3.N * 2)
        steps3 = min(args.steps, 400)
        sec3, _ = rig.time_graph(lambda i: ctx.qmatmul(xb3, pool3[i % len(pool3)], yb3, 512, B.BF16, B.BF16,
                                                       flags=B.FLAG_NO_SYNC), len(pool3), steps3, min(args.warmup, 20))
        flops = 2.0 * 512 * l3.N * l3.K
        rows = np.arange(0, 512, 64)
        y3 = yb3.to_host(np.uint16, (512, l3.N))
        err3 = orc.rel_l2(y3[rows], orc.qmatmul(x3[rows], *l3.triple, bits=4, group=128, w_round=orc.BF16))
        tf = flops / sec3 / 1e12
        extra["gemm_m512_cfg3"] = {
            "kernel": rig.backend.last_kernel_name(),
            "tflops": tf, "us": sec3 * 1e6, "frac_of_measured_bf16_burst": tf / peaks["bf16"],
            "frac_of_measured_bf16_sustained": tf / peaks["bf16_sustained"],
            "frac_of_nominal_2250": tf / NOMINAL_BF16_TFLOPS, "rel_l2_vs_oracle": err3,
            "device_status": ctx.last_device_status()}
    except Exception as e:
        extra["gemm_m512_cfg3"] = {"error": repr(e)}

    # ---- configuration 5 on one GPU: the anchor the N > 1 lines of this program scale against ----
    if not args.skip_ffn:
        try:
            del pool3
        except NameError:
            pass
        try:
            d5 = synth.MLP70B
            gu5, dn5 = synth.mlp_layers(d5["K"], d5["I"], d5["H"], 0, "cfg5")
            x5 = synth.activations(1, d5["K"], "f16", 0, "cfg5.x")
            extra["ffn70b_cfg5_tp1"] = ffn_tp1_block(rig, args, peaks, 1, x5, gu5, dn5)
        except Exception as e:
            extra["ffn70b_cfg5_tp1"] = {"error": repr(e)}

    line = {
        "metric": "qmatmul GEMV weight GB/s", "value": value, "unit": "GB/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int4 weights, f16 x, f32 accumulate",
        "data": "synthetic",
        "config": {"workload": "int4_g128_gemv_14336x4096 (config 2, Llama-3-8B MLP up, batch 1)",
                   "l2": f"inputs larger than L2: {len(pool)} weight copies x {wbytes / 1e6:.1f} MB rotated per step",
                   "timing": "CUDA graph replays of the launch sequence, CUDA events on the launching stream",
                   "note": "the N > 1 lines of this program run a different workload (config 5, tensor-parallel FFN); "
                           "their one-GPU anchor is the key ffn70b_cfg5_tp1, not this value"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm"], "traffic": NCU_TRAFFIC_CONFIG2["bytes"] if kernel == NCU_TRAFFIC_CONFIG2["kernel"] else None,
                     "traffic_source": NCU_TRAFFIC_CONFIG2["source"] + " (one ncu capture of this kernel on this workload, per launch)",
                     "peak_source": peaks["source"],
                     "frac_of_nominal_8tbs": achieved / NOMINAL_HBM_GBS, "algorithmic_bytes": abytes,
                     "kernel": kernel,
                     "chain_of_2400": {"us": sec_chain * 1e6, "frac": abytes / sec_chain / 1e9 / peaks["hbm"]}},
        "cpu_baseline": {"value": wbytes / cpu_sec / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{reps} full config-2 GEMVs (oracle/cpu_baseline.c: -O3, scale and zero-point "
                                   f"hoisted per group, OpenMP over rows)",
                         "one_thread": {"value": wbytes / cpu_sec1 / 1e9, "unit": "GB/s", "cores": 1,
                                        "sample": f"{reps1} full config-2 GEMVs"}},
        "e2e": {"value": wbytes / e2e_sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(x.nbytes),
                "d2h_bytes_per_step": int(out.nbytes), "us_per_step": e2e_sec * 1e6, "parity_rel_l2": parity_e2e,
                "path": "lux_cuda_qmatmul_host: host x in, host y out, weights resident (model state)"},
        "gpu_launches": args.steps, "launches_captured": captured,
        "clocks": clocks, "parity_rel_l2": parity,
    }
    line.update(extra)
    return line


# ----------------------------------------------------------------------------------------
# --workload sweep: configuration 4 (Llama-3-8B decode linears at batch 1, 4, 16, 64) and the
# kernels either side of the linear layers.  Not the headline: the supporting figures.
# ----------------------------------------------------------------------------------------

def bench_sweep(args, peaks):
    from webgpu_b200 import synth

    rig = Rig(0, args.tune)
    B, ctx, torch = rig.B, rig.ctx, rig.torch
    steps = min(args.steps, 120)
    out = {"metric": "qmatmul GEMV weight GB/s", "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
           "config": {"workload": "int4_g128 decode sweep (config 4): qkv / o / gate_up / down at batch 1, 4, 16, 64",
                      "l2": "weight copies rotated per step so that every launch streams from HBM",
                      "timing": "CUDA graph replays, CUDA events on the launching stream"},
           "data": "synthetic", "layers": {}}
    attention_only = args.workload == "attention"       # the decode-attention block alone (small enough to profile)
    for name in ([] if attention_only else synth.SWEEP_LAYERS):
        _, layer = synth.config4(name, 1)
        pool = rig.pool(layer, int(2.9 * L2_BYTES))
        for M in synth.SWEEP_M:
            x, _ = synth.config4(name, M)
            xb, yb = ctx.upload(x), ctx.alloc(M * layer.N * 2)
            sec, _ = rig.time_graph(lambda i: ctx.qmatmul(xb, pool[i % len(pool)], yb, M, B.F16, flags=B.FLAG_NO_SYNC),
                                    len(pool), steps, args.warmup)
            ab = algorithmic_bytes(layer, M, 2, 2)
            out["layers"][f"{name}_m{M}"] = {
                "us": sec * 1e6, "kernel": rig.backend.last_kernel_name(), "weight_gbs": layer.weight_bytes / sec / 1e9,
                "frac_of_measured_hbm": ab / sec / 1e9 / peaks["hbm"], "tflops": 2.0 * M * layer.N * layer.K / sec / 1e12}
        del pool
    # the quantize kernel: f32 [14336, 4096] -> int4 g128 (reads 4 bytes, writes ~0.53 per element)
    if not attention_only:
        wf = torch.randn(14336, 4096, device="cuda", dtype=torch.float32)
        wb = ctx.wrap(wf.data_ptr(), wf.numel() * 4)
        qw, qs, qz = ctx.alloc(14336 * 2048), ctx.alloc(14336 * 32 * 2), ctx.alloc(14336 * 16)
        import ctypes as C
        d = B.make_desc(0, 14336, 4096, 4, 128, B.F32, B.F16, B.F32, B.FLAG_NO_SYNC)
        lib = rig.backend.lib
        sec, _ = rig.time_graph(lambda i: lib.lux_cuda_qquantize(ctx.handle, C.byref(d), wb.handle, qw.handle, qs.handle, qz.handle),
                                1, steps, args.warmup)
        qbytes = 14336 * 4096 * 4 + 14336 * 2048 + 14336 * 32 * 2 + 14336 * 16
        out["quantize_int4_14336x4096"] = {"us": sec * 1e6, "gbs": qbytes / sec / 1e9, "frac_of_measured_hbm": qbytes / sec / 1e9 / peaks["hbm"],
                                           "note": "235 MB read + 31 MB written per launch: larger than L2"}
        del wf
    if not attention_only:
        # the f32 slots either side of a linear layer and the integer path: blocking calls (the vtable's
        # convention), timed with events around each call on 268 MB tensors (larger than L2)
        def timed(call, reps=5):
            for _ in range(2):
                call()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            total = 0.0
            for _ in range(reps):
                e0.record(rig.stream)
                call()
                e1.record(rig.stream)
                torch.cuda.synchronize()
                total += e0.elapsed_time(e1) * 1e-3
            return total / reps
        rows, dim = 8192, 8192
        xt = torch.randn(rows, dim, device="cuda")
        ot = torch.empty_like(xt)
        gt = torch.randn(dim, device="cuda")
        xb_, ob_, gb_ = (ctx.wrap(t.data_ptr(), t.numel() * 4) for t in (xt, ot, gt))
        nbytes = 2 * rows * dim * 4
        ops = {"rms_norm": lambda: ctx.rms_norm_f32(xb_, gb_, ob_, rows, dim, 1e-5),
               "layer_norm": lambda: ctx.layer_norm_f32(xb_, gb_, gb_, ob_, rows, dim, 1e-5),
               "softmax": lambda: ctx.softmax_f32(xb_, ob_, rows, dim),
               "silu": lambda: ctx.unary_f32("silu", xb_, ob_, rows * dim),
               "gelu": lambda: ctx.unary_f32("gelu", xb_, ob_, rows * dim),
               "transpose": lambda: ctx.transpose_f32(xb_, ob_, rows, dim)}
        out["tensor_slots_8192x8192_f32"] = {}
        with torch.cuda.stream(rig.stream):
            for name, call in ops.items():
                sec = timed(call)
                out["tensor_slots_8192x8192_f32"][name] = {"us": sec * 1e6, "gbs": nbytes / sec / 1e9,
                                                           "frac_of_measured_hbm": nbytes / sec / 1e9 / peaks["hbm"]}
            del xt, ot
            # W8A8: C[M, N] (i32) = A[M, K] (i8) . B[K, N] (i8) on mma.sync.m16n8k32.s8; and the quantize step before it
            Mi = Ni = Ki = 4096
            at = torch.randint(-127, 128, (Mi, Ki), device="cuda", dtype=torch.int8)
            bt = torch.randint(-127, 128, (Ki, Ni), device="cuda", dtype=torch.int8)
            ct = torch.empty(Mi, Ni, device="cuda", dtype=torch.int32)
            ab_, bb_, cb_ = ctx.wrap(at.data_ptr(), at.numel()), ctx.wrap(bt.data_ptr(), bt.numel()), ctx.wrap(ct.data_ptr(), ct.numel() * 4)
            sec = timed(lambda: ctx.matmul_int8(ab_, bb_, cb_, Mi, Ni, Ki))
            out["matmul_int8_4096"] = {"us": sec * 1e6, "tops": 2.0 * Mi * Ni * Ki / sec / 1e12, "kernel": rig.backend.last_kernel_name()}
            ft = torch.randn(64 << 20, device="cuda")
            qt = torch.empty(64 << 20, device="cuda", dtype=torch.int8)
            st = torch.empty(4, device="cuda")
            fb_, qb_, sb_ = ctx.wrap(ft.data_ptr(), ft.numel() * 4), ctx.wrap(qt.data_ptr(), qt.numel()), ctx.wrap(st.data_ptr(), 16)
            sec = timed(lambda: ctx.dynamic_quantize(fb_, qb_, sb_, ft.numel()))
            dq_bytes = ft.numel() * (4 + 4 + 1)            # read for the maximum, read again, write int8
            out["dynamic_quantize_64m"] = {"us": sec * 1e6, "gbs": dq_bytes / sec / 1e9, "frac_of_measured_hbm": dq_bytes / sec / 1e9 / peaks["hbm"],
                                           "note": "two passes over 268 MB (tensor-wide maximum, then quantize) + 67 MB written"}
            del at, bt, ct, ft, qt
    # decode attention over an f32 KV cache with Llama-3-8B's heads (32 query, 8 key/value, 128 wide):
    # contiguous cache (sdpa_kv_cache) and 16-token pages (paged_attention), bytes = K and V read once
    H, HKV, D = 32, 8, 128
    out["attention_decode"] = {}
    shapes = ((1, 4096), (1, 32768), (8, 4096), (32, 4096))
    if args.attention_shape:
        shapes = (tuple(int(v) for v in args.attention_shape.split("x")),)
    for batch, ctx_len in shapes:
        kv_bytes = 2 * batch * HKV * ctx_len * D * 4
        copies = max(1, -(-int(2.9 * L2_BYTES) // kv_bytes))
        caches = [(torch.randn(batch, HKV, ctx_len, D, device="cuda"), torch.randn(batch, HKV, ctx_len, D, device="cuda")) for _ in range(copies)]
        wrapped = [(ctx.wrap(k.data_ptr(), k.numel() * 4), ctx.wrap(v.data_ptr(), v.numel() * 4)) for k, v in caches]
        q = torch.randn(batch, H, 1, D, device="cuda")
        o = torch.empty_like(q)
        qb, ob = ctx.wrap(q.data_ptr(), q.numel() * 4), ctx.wrap(o.data_ptr(), o.numel() * 4)
        scale = 1.0 / math.sqrt(D)
        sec, _ = rig.time_graph(lambda i: ctx.sdpa_kv_cache(qb, wrapped[i % copies][0], wrapped[i % copies][1], ob, batch, H, HKV, 1,
                                                            ctx_len - 1, ctx_len, D, scale, flags=B.FLAG_NO_SYNC), copies, steps, args.warmup)
        entry = {"contiguous_us": sec * 1e6, "contiguous_gbs": kv_bytes / sec / 1e9, "contiguous_frac_of_measured_hbm": kv_bytes / sec / 1e9 / peaks["hbm"]}
        # the same bytes seen as 16-token pages in a shuffled order
        bs = 16
        nblk = ctx_len // bs
        table = torch.stack([torch.randperm(nblk, device="cuda") + s * nblk for s in range(batch)]).to(torch.int32).contiguous()
        lens = torch.full((batch,), ctx_len, device="cuda", dtype=torch.int32)
        tb, lb = ctx.wrap(table.data_ptr(), table.numel() * 4), ctx.wrap(lens.data_ptr(), lens.numel() * 4)
        q3, o3 = ctx.wrap(q.data_ptr(), q.numel() * 4), ctx.wrap(o.data_ptr(), o.numel() * 4)
        # [batch, kv_heads, ctx, D] read as [batch * ctx / 16 blocks][...]: the bytes of a block are then not one
        # (block, head) tile, which changes what is computed, not what is read; timing only
        sec, _ = rig.time_graph(lambda i: ctx.paged_attention(q3, wrapped[i % copies][0], wrapped[i % copies][1], tb, lb, o3, batch, H, HKV, D,
                                                              bs, nblk, scale, flags=B.FLAG_NO_SYNC), copies, steps, args.warmup)
        entry.update({"paged16_us": sec * 1e6, "paged16_gbs": kv_bytes / sec / 1e9, "paged16_frac_of_measured_hbm": kv_bytes / sec / 1e9 / peaks["hbm"],
                      "kv_mb": kv_bytes / 1e6})
        out["attention_decode"][f"b{batch}_ctx{ctx_len}"] = entry
        del caches, wrapped
    if not args.attention_shape:
        # causal prefill of one 2048-token sequence with the same heads (f32 FMA arithmetic, no tensor cores)
        S = 2048
        qp, kp, vp = (torch.randn(1, h, S, D, device="cuda") for h in (H, HKV, HKV))
        op = torch.empty_like(qp)
        bufs = [ctx.wrap(t.data_ptr(), t.numel() * 4) for t in (qp, kp, vp, op)]
        sec, _ = rig.time_graph(lambda i: ctx.sdpa(bufs[0], bufs[1], bufs[2], bufs[3], 1, H, HKV, S, S, D, 1.0 / math.sqrt(D),
                                                   flags=B.FLAG_NO_SYNC | B.FLAG_ATTN_CAUSAL), 1, min(steps, 10), 2)
        out["attention_prefill_s2048_causal"] = {"us": sec * 1e6, "tflops": 4.0 * S * S * D * H / 2 / sec / 1e12,
                                                 "note": "f32 inputs, f32 FMA on the CUDA cores; keys stream through shared memory once per block of 16 query rows"}
    ctx.sync()
    return out


# ----------------------------------------------------------------------------------------
# configuration 5: the 70B-shaped FFN, on one GPU (anchor of the scaling curve) and tensor-parallel
# ----------------------------------------------------------------------------------------

def ffn_flops(M, d, world=1):
    return 2.0 * M * (2 * (d["I"] // world) * d["K"] + d["H"] * (d["I"] // world))


def ffn_parity(x, gate_up, down, y, world, M):
    """rel-L2 of the GPU result y[M, H] against the oracle's sharded FFN (partials narrowed to f16
    per rank and summed in rank order); for batches above four rows on a subset of the rows (rows
    are independent).  From 5 rows on the kernels multiply weights rounded to f16."""
    from oracle import oracle as orc      # checker only, outside every timed region
    from webgpu_b200 import tp
    rows = np.arange(M) if M <= 4 else np.unique(np.linspace(0, M - 1, 4).astype(int))
    shards = [tuple(l.triple for l in tp.shard_mlp(gate_up, down, r, world)) for r in range(world)]
    ref = orc.tp_mlp(np.ascontiguousarray(x[rows]), shards, fused=True, w_round=orc.F16 if M >= 5 else orc.F32)
    return orc.rel_l2(np.ascontiguousarray(y[rows]), ref), [int(r) for r in rows]


def ffn_tp1_block(rig, args, peaks, M, x, gate_up, down):
    """The unsharded configuration-5 FFN on this rig's GPU: kernels-only time in the same graph-replay
    harness as every other number here, and its parity against the oracle."""
    from webgpu_b200 import synth, tp
    torch, B, ctx = rig.torch, rig.B, rig.ctx
    d = synth.MLP70B
    total_wbytes = gate_up.weight_bytes + down.weight_bytes
    copies = max(2, -(-int(2.9 * L2_BYTES) // total_wbytes))
    mlps = [tp.TPMlp(ctx, gate_up, down, 0, 1, M, "f16", presharded=True) for _ in range(copies)]
    xt = torch.from_numpy(x).cuda()
    for m in mlps:
        m.x[:M].copy_(xt)
    torch.cuda.synchronize()
    steps = min(args.steps, 240)
    sec, _ = rig.time_graph(lambda i: mlps[i % copies].forward(M), copies, steps, args.warmup)
    kernel = rig.backend.last_kernel_name()
    y = mlps[(steps - 1) % copies].y[:M].cpu().numpy()
    ctx.sync()
    parity, rows = ffn_parity(x, gate_up, down, y, 1, M)
    alg = total_wbytes + M * d["K"] * 2 + 2 * M * d["I"] * 2 + M * d["H"] * 2
    out = {"us": sec * 1e6, "batch": M, "kernel": kernel, "weights_gbs": total_wbytes / sec / 1e9,
           "total_gbs": alg / sec / 1e9, "frac_of_measured_hbm": alg / sec / 1e9 / peaks["hbm"],
           "tflops": ffn_flops(M, d) / sec / 1e12, "steps": steps, "parity_rel_l2": parity, "parity_rows": rows,
           "l2": f"{copies} weight copies x {total_wbytes / 1e6:.1f} MB rotated per step"}
    del mlps
    torch.cuda.empty_cache()
    return out


def bench_tp(args, peaks):
    import torch
    import torch.distributed as dist
    from webgpu_b200 import synth, tp

    rank, local_rank, world = dist_env()
    d = synth.MLP70B
    M = args.batch
    workload = f"llama70b_mlp_tp (config 5): gate_up 8192->57344 + SwiGLU, down 28672->8192, batch {M}"
    if world > 1 and args.collective == "nccl" and M >= 32:
        # An NCCL all-reduce captured into the timing graphs at batch 32 and 256 did not finish on two
        # GPUs in two runs and no cause was found by reading; that combination is not run again.
        if rank == 0:
            print(json.dumps({"metric": "qmatmul GEMV weight GB/s", "n_gpus": world, "config": {"workload": workload},
                              "unavailable": "graph-captured NCCL all-reduce at batch >= 32 did not terminate on two GPUs "
                                             "(cause not found); use --collective push"}))
        return None
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    rig = Rig(local_rank, args.tune)
    B, ctx = rig.B, rig.ctx
    gate_up, down = synth.mlp_layers(d["K"], d["I"], d["H"], 0, "cfg5")
    x = synth.activations(M, d["K"], "f16", 0, "cfg5.x")
    total_wbytes = gate_up.weight_bytes + down.weight_bytes

    # ---- the one-GPU anchor of the scaling curve: the same FFN, unsharded, on rank 0 of this box ----
    tp1 = None
    if rank == 0 and not args.skip_tp1:
        tp1 = ffn_tp1_block(rig, args, peaks, M, x, gate_up, down)
    if world > 1:
        dist.barrier()

    shard_bytes = total_wbytes // world
    copies = max(2, -(-int(2.9 * L2_BYTES) // shard_bytes))
    g_sh, d_sh = tp.shard_mlp(gate_up, down, rank, world)
    peer, collective = None, "none"
    if world > 1:
        if args.collective == "push":
            # no silent fallback: if any rank cannot map its peers' windows, every rank stops
            ok, why = 1, ""
            try:
                if (M * d["H"]) % 8:
                    raise ValueError("the push all-reduce takes whole 16-byte pieces")
                peer = tp.PeerAllReduce(ctx, rank, world, M * d["H"] * 2)
            except Exception as exc:   # noqa: BLE001 - e.g. CUDA IPC refused in this environment
                ok, why = 0, repr(exc)
            flag = torch.tensor([ok], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) != 1:
                raise RuntimeError(f"rank {rank}: --collective push was asked for but the peer windows could not be "
                                   f"connected on every rank ({why or 'another rank failed'})")
            collective = ("push all-reduce over peer memory: the down kernel's epilogue stores into the peers' windows "
                          "(batch <= 2) and lux_peer_allreduce_push waits and sums; larger batches push from that kernel; "
                          "f16 partials, f32 sum in rank order")
        else:
            collective = "NCCL all-reduce of f16 partials (torch.distributed)"
    note = f"[bench] rank {rank}/{world}: batch {M}, collective = {collective}"
    print(note, file=sys.stderr, flush=True)
    mlps = [tp.TPMlp(ctx, g_sh, d_sh, rank, world, M, "f16", presharded=True, peer=peer) for _ in range(copies)]
    xt = torch.from_numpy(x).cuda()
    for m in mlps:
        m.x[:M].copy_(xt)
    sampler = ClockSampler(local_rank)
    torch.cuda.synchronize()

    def step(i):
        return mlps[i % copies].forward(M)

    def agree(ok):
        # the capture-or-eager choice is collective: ranks replaying graphs next to ranks launching
        # eagerly would issue different sequences of collectives and barriers
        return tp.all_ranks_agree(ok, device="cuda")

    def eager_time(fn):
        with torch.cuda.stream(rig.stream):
            for i in range(max(args.warmup, 3)):
                fn(i)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda._sleep(200_000)
            fn(copies - 1)                      # untimed: its collective aligns the ranks
            e0.record(rig.stream)
            for i in range(args.steps):
                fn(i)
            e1.record(rig.stream)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e-3 / args.steps

    # Timed as CUDA-graph replays of the step sequence (FFN kernels + collective captured together):
    # with tens of microseconds of GPU work per step, eager launches would measure the host.
    timing = "CUDA graph replays of the step sequence (kernels + all-reduce), CUDA events on the launching stream"
    if world > 1:
        dist.barrier()
    sampler.start()
    sec = sec_compute = None
    try:
        sec, _ = rig.time_graph(step, copies, args.steps, args.warmup, align=(lambda: step(copies - 1)) if world > 1 else None)
        captured = True
    except Exception as exc:   # noqa: BLE001
        captured = False
        print(f"[bench] rank {rank}: graph capture failed ({exc!r})", file=sys.stderr, flush=True)
    if not agree(captured):
        timing = "eager launches (graph capture failed on at least one rank)"
        sec = eager_time(step)
    if world > 1:
        dist.barrier()
    # compute-only time (no collective) to separate kernel bandwidth from all-reduce cost
    compute_only = lambda i: mlps[i % copies].forward(M, all_reduce=False)   # noqa: E731
    try:
        sec_compute, _ = rig.time_graph(compute_only, copies, args.steps, args.warmup)
        captured = True
    except Exception:   # noqa: BLE001
        captured = False
    if not agree(captured):
        sec_compute = eager_time(compute_only)
    if world > 1:
        dist.barrier()
    clocks = sampler.stop()
    t = torch.tensor([sec, sec_compute], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec, sec_compute = float(t[0]), float(t[1])

    # ---- parity of a step that INCLUDED the collective, and identical bits on every rank ----
    with torch.cuda.stream(rig.stream):
        out = step(0)
        rig.stream.synchronize()
    ctx.sync()                       # raises if a bounded device-side wait gave up
    y = out.cpu().numpy()
    ranks_identical = True
    if world > 1:
        import zlib
        h = torch.tensor([zlib.crc32(y.tobytes())], device="cuda", dtype=torch.int64)
        hs = [torch.zeros_like(h) for _ in range(world)]
        dist.all_gather(hs, h)
        ranks_identical = all(int(v.item()) == int(hs[0].item()) for v in hs)
    parity, parity_rows = (None, None)
    if rank == 0:
        parity, parity_rows = ffn_parity(x, gate_up, down, y, world, M)
    if world > 1:
        dist.barrier()

    # e2e: x from pinned host memory each step, y back to the host
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty((M, d["H"]), dtype=torch.float16).pin_memory()
    n_e2e = min(args.steps, 200)
    torch.cuda.synchronize()
    # One CUDA graph per weight copy holding the whole step a caller makes: x from pinned host
    # memory, the FFN with its collective, y back to pinned host memory; each timed step is one
    # replay plus one stream wait (the host reads y after every step).
    def e2e_step(m):
        m.x[:M].copy_(xh, non_blocking=True)
        o = m.forward(M)
        yh.copy_(o, non_blocking=True)

    e2e_path = "CUDA graph per step: pinned H2D copy of x, FFN + collective, D2H copy of y; one stream wait per step"
    graphs = None
    try:
        with torch.cuda.stream(rig.stream):
            for m in mlps:
                e2e_step(m)
            rig.stream.synchronize()
            graphs = []
            for m in mlps:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=rig.stream, capture_error_mode="relaxed"):
                    e2e_step(m)
                graphs.append(g)
            for g in graphs:
                g.replay()
            rig.stream.synchronize()
        captured = True
    except Exception:   # noqa: BLE001
        captured = False
    if not agree(captured):
        graphs = None
        e2e_path = "eager launches per step (graph capture failed on at least one rank)"
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    with torch.cuda.stream(rig.stream):
        for i in range(n_e2e):
            if graphs is not None:
                graphs[i % copies].replay()
            else:
                e2e_step(mlps[i % copies])
            rig.stream.synchronize()
    e2e_sec = (time.perf_counter() - t0) / n_e2e
    t = torch.tensor([e2e_sec], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_sec = float(t[0])

    per_gpu_alg = shard_bytes + M * d["K"] * 2 + 2 * M * (d["I"] // world) * 2 + M * d["H"] * 2
    line = None
    if rank == 0:
        line = {
            "metric": "qmatmul GEMV weight GB/s", "value": total_wbytes / sec / 1e9, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int4 weights, f16 activations, f32 accumulate", "data": "synthetic",
            "config": {"workload": workload,
                       "parallelism": f"tp{world}", "collective": collective,
                       "l2": f"inputs larger than L2: {copies} shard copies x {shard_bytes / 1e6:.1f} MB rotated per step",
                       "timing": timing,
                       "note": "a different workload from the N = 1 line of this program (config 2): compare this value "
                               "with tp1_us_same_box, not with the N = 1 value"},
            "roofline": {"bound": "hbm", "achieved": per_gpu_alg / sec_compute / 1e9, "peak": peaks["hbm"],
                         "unit": "GB/s", "frac": per_gpu_alg / sec_compute / 1e9 / peaks["hbm"], "traffic": None,
                         "peak_source": peaks["source"], "note": "per GPU, both FFN kernels, without the all-reduce",
                         "us_compute_only": sec_compute * 1e6, "us_with_allreduce": sec * 1e6},
            "e2e": {"value": total_wbytes / e2e_sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": int(x.nbytes),
                    "d2h_bytes_per_step": int(M * d["H"] * 2), "us_per_step": e2e_sec * 1e6, "path": e2e_path},
            "gpu_launches": (2 if world == 1 else 3) * args.steps, "clocks": clocks,
            "parity_rel_l2": parity, "parity_rows": parity_rows, "ranks_identical": ranks_identical,
            "tp1_us_same_box": tp1["us"] if tp1 else None, "ffn70b_cfg5_tp1": tp1,
            "strong_scaling_efficiency": tp1["us"] / (world * sec * 1e6) if tp1 else None,
        }
    if line is not None and M >= 5:
        # From 5 batch rows on both FFN kernels run on the tensor cores: the roofline that bounds
        # them is the dense 16-bit tensor peak, not HBM (the weights are read once either way).
        tf = ffn_flops(M, d, world) / sec_compute / 1e12
        line["roofline"] = {"bound": "tensor", "achieved": tf, "peak": peaks["bf16"], "unit": "TFLOP/s",
                            "frac": tf / peaks["bf16"], "frac_of_sustained": tf / peaks["bf16_sustained"], "traffic": None,
                            "peak_source": peaks["source"], "note": "per GPU, both FFN kernels, without the all-reduce",
                            "us_compute_only": sec_compute * 1e6, "us_with_allreduce": sec * 1e6,
                            "weights_gbs": per_gpu_alg / sec_compute / 1e9}
    ctx.sync()                       # raises if a bounded device-side wait gave up during the run
    if peer is not None:
        peer.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return line


# ----------------------------------------------------------------------------------------
# reference arm: the CPU oracle on this machine's cores (the WGSL cannot run here)
# ----------------------------------------------------------------------------------------

def bench_reference(args):
    """The reference arm: the reference's own arithmetic for this path on the host cores (its WGSL
    needs a WebGPU runtime, so what runs is the CPU restatement in oracle/cpu_baseline.c), all host
    threads, exactly --steps timed steps after --warmup untimed ones.  A step is the whole workload
    unless that would take minutes: then it is one tensor-parallel shard of it, and says so."""
    rank, _, world = dist_env()
    if rank != 0:
        return None
    from oracle import cpu_baseline as cb
    from webgpu_b200 import synth, tp

    cores = cb.num_procs()
    if args.gpus <= 1:
        x, layer = synth.config2()
        workload = "int4_g128_gemv_14336x4096 (config 2, Llama-3-8B MLP up, batch 1)"
        scaling = "weak"

        def make(frac):
            rows = layer.N // frac
            sub = (layer.w[:rows], layer.scales[:rows], None if layer.zeros is None else layer.zeros[:rows])
            nbytes = sum(t.nbytes for t in sub if t is not None)
            return (lambda: cb.qmatmul_i4(x, *sub)), nbytes, ("one full config-2 GEMV" if frac == 1 else
                                                              f"the first 1/{frac} of the rows of the config-2 GEMV")
    else:
        d = synth.MLP70B
        gate_up, down = synth.mlp_layers(d["K"], d["I"], d["H"], 0, "cfg5")
        x = synth.activations(args.batch, d["K"], "f16", 0, "cfg5.x")
        workload = f"llama70b_mlp_tp (config 5): gate_up 8192->57344 + SwiGLU, down 28672->8192, batch {args.batch}"
        scaling = "strong"

        def make(frac):
            g, dn = (gate_up, down) if frac == 1 else tp.shard_mlp(gate_up, down, 0, frac)
            nbytes = g.weight_bytes + dn.weight_bytes
            return (lambda: cb.mlp_i4(x, g.triple, dn.triple)), nbytes, (
                "the whole FFN on the host (no sharding: one host)" if frac == 1 else
                f"shard 0 of {frac} of the FFN (1/{frac} of the weights)")

    frac = 1
    fn, nbytes, sample = make(1)
    fn()
    t0 = time.perf_counter()
    fn()
    one = time.perf_counter() - t0
    total = (args.steps + args.warmup) * one
    while total / frac > 150.0 and frac < 64:
        frac *= 2
    if frac > 1:
        fn, nbytes, sample = make(frac)
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    sec = (time.perf_counter() - t0) / args.steps
    v = nbytes / sec / 1e9
    return {
        "impl": "reference", "metric": "qmatmul GEMV weight GB/s", "value": v, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": scaling, "vs_baseline": None, "dtype": "int4 weights, f16 x, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload},
        "cpu_baseline": {"value": v, "unit": "GB/s", "cores": cores, "kind": "port", "sample": "each step = " + sample,
                         "note": "CPU restatement of the reference's WGSL arithmetic (oracle/cpu_baseline.c, -O3, OpenMP); "
                                 "the shaders need a WebGPU runtime, which is unavailable on this box"},
        "e2e": {"value": v, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2400)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1, help="batch M of the tensor-parallel FFN workload")
    ap.add_argument("--workload", default="auto", choices=["auto", "gemv", "tp_mlp", "sweep", "attention"])
    ap.add_argument("--attention-shape", default="", help="attention workload: one BATCHxCONTEXT shape instead of the built-in four")
    ap.add_argument("--collective", default="push", choices=["push", "nccl"],
                    help="all-reduce of the tensor-parallel FFN: the plugin's push all-reduce over peer memory "
                         "(falls back to NCCL if the peer mapping is refused) or NCCL")
    ap.add_argument("--skip-tp1", action="store_true", help="N > 1: leave out the one-GPU anchor run on rank 0")
    ap.add_argument("--skip-ffn", action="store_true", help="N = 1: leave out the configuration-5 one-GPU block")
    ap.add_argument("--eager", action="store_true", help="time plain launches queued behind the spin kernel instead of CUDA-graph replays")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=VALUE",
                    help="override a launch heuristic (lux_cuda_tune_set), e.g. gemv_i4_kernel=2")
    args = ap.parse_args()
    Rig.eager = args.eager
    peaks = measured_peaks()
    if args.impl == "reference":
        line = bench_reference(args)
    else:
        _, _, world = dist_env()
        use_tp = args.workload == "tp_mlp" or (args.workload == "auto" and (args.gpus > 1 or world > 1))
        if args.workload in ("sweep", "attention"):
            line = bench_sweep(args, peaks)
        else:
            line = bench_tp(args, peaks) if use_tp else bench_single(args, peaks)
    if line is not None:
        print(json.dumps(line))


if __name__ == "__main__":
    main()
