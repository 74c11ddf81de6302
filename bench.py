#!/usr/bin/env python
"""Benchmark of the int8 quantized-linear hot path.

    python bench.py --gpus N --steps K --warmup W          # this backend (one process per GPU under torchrun for N > 1)
    python bench.py --impl reference ...                   # the CPU restatement of the reference on the host cores

A step is one pass of the hot path over one batch of synthetic input: f32 activations
[M,K] -> per-token int8 -> int8 x int8 -> int32 contraction on the tensor cores -> scale,
bias and activation fused in the epilogue -> f32 [M,N].  The default workload is the large
GEMM configuration (M 8192, K 4096, N 4096, GELU(tanh)); every rank processes its own M
rows against replicated weights (no collective on the data path), so the scaling is weak.

One JSON line is printed by rank 0.  `value` is tokens/s with inputs resident in HBM,
`e2e` is the same metric through the host-buffer entry point (pinned host memory in, host
memory out, copies inside the timed region), `roofline` describes the dominant kernel,
`cpu_baseline` the CPU port timed on this machine.  The same line carries, at every N, three
fixed-size (strong-scaling) records, each checked against the unsharded result on the same
GPUs: the large GEMM with its 8192 rows split over the ranks (`c3_strong`), and the stack of
four wide linears split by rows (`c5_mshard`) and by output channels with NCCL collectives
inside the library (`c5_nshard`).
"""
from __future__ import annotations

import argparse
import functools
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (M per GPU, K, N, activation)
    "c3_gemm_8192x4096x4096_gelu_tanh": (8192, 4096, 4096, "gelu_tanh"),
    "c3_gemm_8192x4096x4096_gelu_sigmoid": (8192, 4096, 4096, "gelu_sigmoid"),
    "small_2048x4096x4096_gelu_tanh": (2048, 4096, 4096, "gelu_tanh"),       # profiler-sized case
    "small_2048x4096x4096_gelu_sigmoid": (2048, 4096, 4096, "gelu_sigmoid"),
    "small_2048x4096x4096_none": (2048, 4096, 4096, "none"),
    # the short-K linears of the transformer block (config 4), as single-linear steps
    "c4_qkv_16384x768x2304_none": (16384, 768, 2304, "none"),
    "c4_fc1_16384x768x3072_gelu_sigmoid": (16384, 768, 3072, "gelu_sigmoid"),
    "c4_fc2_16384x3072x768_none": (16384, 3072, 768, "none"),
}
DEFAULT_WORKLOAD = "c3_gemm_8192x4096x4096_gelu_tanh"
C4_WORKLOAD = "c4_gpt_block_d768_h12_ff3072_32x512"
C5_WORKLOAD = "c5_stack_4096x8192x28672_silu"       # 4 linears 8192 -> 28672 -> 8192 -> 28672 -> 8192, M 4096 in total
C2_SHAPE = (16384, 4096)          # standalone quantize -> dequantize round trip
CPU_SAMPLE_ROWS = 64              # rows of M the CPU arm processes per step (rows are independent)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); smax.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                "power_w_max": max(power), "samples": len(sm)}


def gpu_numa_info(gpu_index: int) -> dict:
    """NUMA node of a GPU and the CPUs of that node, from sysfs (read only)."""
    info = {"gpu": gpu_index, "node": None, "cpus": None}
    try:
        bus = subprocess.check_output(["nvidia-smi", f"--id={gpu_index}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                                      text=True, stderr=subprocess.DEVNULL).strip().lower()
        if bus.count(":") == 2 and len(bus.split(":")[0]) == 8:
            bus = bus[4:]                                    # nvidia-smi prints an 8-digit domain, sysfs a 4-digit one
        info["pci"] = bus
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read().strip())
        info["node"] = node
        if node >= 0:
            info["cpus"] = open(f"/sys/devices/system/node/node{node}/cpulist").read().strip()
    except Exception as exc:                                  # no sysfs entry, no nvidia-smi: nothing to bind to
        info["error"] = f"{type(exc).__name__}: {exc}"
    return info


def _parse_cpulist(text: str):
    cpus = set()
    for part in text.split(","):
        if "-" in part:
            a, b = part.split("-")
            cpus.update(range(int(a), int(b) + 1))
        elif part:
            cpus.add(int(part))
    return cpus


def bind_to_numa_node(info: dict) -> dict:
    """Pins this process's threads to the CPUs of the GPU's NUMA node and prefers that node's memory for what it
    allocates from now on (set_mempolicy MPOL_PREFERRED).  Returns what was done."""
    out = {"node": info.get("node"), "bound": False}
    if info.get("node") is None or info["node"] < 0 or not info.get("cpus"):
        out["why"] = "the platform reports no NUMA node for this GPU" if not info.get("error") else info["error"]
        return out
    try:
        allowed = os.sched_getaffinity(0)
        want = _parse_cpulist(info["cpus"]) & allowed
        if want and want != allowed:
            os.sched_setaffinity(0, want)
            out["cpus"] = len(want)
        else:
            out["cpus"] = len(allowed)
        import ctypes
        libc = ctypes.CDLL(None, use_errno=True)
        mask = ctypes.c_ulong(1 << info["node"])
        rc = libc.syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(64))      # set_mempolicy(MPOL_PREFERRED, mask, 64)
        out["mempolicy"] = "preferred" if rc == 0 else f"set_mempolicy failed (errno {ctypes.get_errno()})"
        out["bound"] = bool(want and want != allowed) or rc == 0
        out["same_as_before"] = not (want and want != allowed)
    except Exception as exc:
        out["why"] = f"{type(exc).__name__}: {exc}"
    return out


def make_case(workload: str, rank: int):
    from mlfw_b200 import synth
    M, K, N, act = WORKLOADS[workload]
    seed = 0
    xs = [synth.normal(synth.tensor_seed(seed, 100 + 10 * rank + i), (M, K)) for i in range(2)]
    W = synth.randint_i8(synth.tensor_seed(seed, 1), (N, K))
    ws = synth.uniform(synth.tensor_seed(seed, 2), (N,), 1e-3, 1e-2)
    bias = synth.normal(synth.tensor_seed(seed, 3), (N,), 0.0, 0.01)
    return M, K, N, act, xs, W, ws, bias


@functools.lru_cache(maxsize=1)
def c2_input():
    from mlfw_b200 import synth
    M2, K2 = C2_SHAPE
    return synth.with_outliers(synth.normal(synth.tensor_seed(0, 20), (M2, K2)), synth.tensor_seed(0, 21), synth.tensor_seed(0, 22))


def run_quant_sweep(ctx, pk, iters=40):
    """Per-token quantize over row lengths and row counts, launched back to back (one event pair around `iters` launches,
    inputs rotating through more than L2's worth of buffers): the default kernel choice against the earlier
    shared-memory-staged kernel (b200q_set_quant_variant 4)."""
    rng = np.random.default_rng(0)
    out = {}
    for M in (8192, 16384):
        for K in (768, 1024, 2048, 3072, 4096, 8192):
            xs = [ctx.to_device(rng.standard_normal((M, K)).astype(np.float32)) for _ in range(max(2, int(300e6 / (M * K * 4)) + 1))]
            q, s = ctx.empty((M, K), np.int8), ctx.empty((M,), np.float32)
            rec = {}
            for variant, name in ((4, "staged"), (0, "default")):
                ctx.set_quant_variant(variant)
                for i in range(5):
                    ctx.quantize_per_token(xs[i % len(xs)], M, K, q, s)
                ctx.sync()
                ctx.timer_start()
                for i in range(iters):
                    ctx.quantize_per_token(xs[i % len(xs)], M, K, q, s)
                ms = ctx.timer_stop() / iters
                gbs = (5.0 * M * K + 4.0 * M) / (ms * 1e-3) / 1e9
                rec[name] = {"us": ms * 1e3, "GBps": gbs, "frac": gbs / pk["hbm_gbs"]}
            ctx.set_quant_variant(0)
            out[f"{M}x{K}"] = rec
            for b in xs + [q, s]:
                b.free()
    ctx.check_status()
    return out


def run_conv_bench(ctx, pk, iters=20):
    """quantized_conv2d (gather + tensor-core contraction) on ResNet-sized 3x3 and 1x1 layers, channel-last and
    channel-first, 32 images: time per call back to back, TOP/s over 2 * outputs * taps, and the split between the
    gather / re-lay kernels and the contraction from the per-family event timing of a second pass."""
    rng = np.random.default_rng(0)
    out = {}
    for (C, HW, O, KK, pad) in ((64, 56, 64, 3, 1), (128, 28, 128, 3, 1), (256, 14, 256, 3, 1), (256, 56, 64, 1, 0)):
        N = 32
        for layout in ("NHWC", "NCHW"):
            xs = (N, HW, HW, C) if layout == "NHWC" else (N, C, HW, HW)
            ks = (O, KK, KK, C) if layout == "NHWC" else (O, C, KK, KK)
            dx = ctx.to_device(rng.integers(-127, 128, xs, dtype=np.int8))
            dk = ctx.to_device(rng.integers(-127, 128, ks, dtype=np.int8))
            do = ctx.empty((N * HW * HW * O,), np.int32)
            call = lambda: ctx.quantized_conv2d(dx, dk, (N, C, HW, HW), (O, KK, KK), do, (1, 1), ((pad, pad), (pad, pad)), (1, 1), 1, 0, 0, layout)
            for _ in range(3):
                call()
            ctx.sync()
            ctx.timer_start()
            for _ in range(iters):
                call()
            ms = ctx.timer_stop() / iters
            ctx.profile_enable(True); ctx.profile_reset()
            for _ in range(iters):
                call()
            fam = ctx.profile_read()
            ctx.profile_enable(False)
            ops = 2.0 * N * HW * HW * O * C * KK * KK
            out[f"c{C}_{HW}x{HW}_o{O}_k{KK}_{layout}"] = {
                "us": ms * 1e3, "TOPs": ops / (ms * 1e-3) / 1e12, "frac_of_int8_proxy": ops / (ms * 1e-3) / 1e12 / (2 * pk["bf16_tflops"]),
                "gather_and_relay_us": fam.get("weights", (0.0, 1))[0] / iters * 1e3, "contraction_us": fam.get("gemm_tensor_core", (0.0, 1))[0] / iters * 1e3,
                "gathered_bytes": N * HW * HW * ((C * KK * KK + 15) // 16 * 16)}
            for b in (dx, dk, do):
                b.free()
    # per-group INT4 codes of a weight the size of config 5's (8192 x 28672 f32 = 940 MB read, 235 MB of codes written)
    n, G = 8192 * 28672, 128
    dw = ctx.to_device(rng.standard_normal(n).astype(np.float32))
    dq, ds = ctx.empty((n,), np.int8), ctx.empty((n // G,), np.float64)
    ctx.quantize_per_group(dw, n, G, 4, dq, ds, None)
    ctx.sync()
    ctx.timer_start()
    for _ in range(3):
        ctx.quantize_per_group(dw, n, G, 4, dq, ds, None)
    ms = ctx.timer_stop() / 3
    out["per_group_int4_8192x28672_g128"] = {"ms": ms, "GBps": (5.0 * n + 8.0 * n / G) / (ms * 1e-3) / 1e9,
                                             "frac": (5.0 * n + 8.0 * n / G) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"]}
    for b in (dw, dq, ds):
        b.free()
    ctx.check_status()
    return out


def run_tail_sweep(ctx, iters=4):
    """Config 5's up-projection shape (M 4096, K 8192, N 28672) through b200q_int8_linear with every tail: what the
    fused activation costs on top of the contraction."""
    rng = np.random.default_rng(0)
    M, N, K = 4096, 28672, 8192
    A = ctx.to_device(rng.integers(-127, 128, (M, K), dtype=np.int8))
    s = ctx.to_device(rng.uniform(0.01, 0.02, M).astype(np.float32))
    W = ctx.to_device(rng.integers(-127, 128, (N, K), dtype=np.int8))
    ws = ctx.to_device(rng.uniform(1e-4, 2e-4, N).astype(np.float32))
    out = ctx.empty((M, N), np.float32)
    res = {}
    for act, mode in (("none", 0), ("relu", 0), ("gelu_tanh", 0), ("silu", 1), ("silu", 0), ("gelu_sigmoid", 0)):
        ctx.set_tail_mode(mode)
        for _ in range(2):
            ctx.int8_linear(A, s, W, ws, None, act, M, N, K, out)
        ctx.sync()
        time.sleep(0.3)
        ctx.timer_start()
        for _ in range(iters):
            ctx.int8_linear(A, s, W, ws, None, act, M, N, K, out)
        ms = ctx.timer_stop() / iters
        res[act + ("_hardware_exp" if mode else "")] = {"us": ms * 1e3, "TOPs": 2.0 * M * N * K / (ms * 1e-3) / 1e12}
    ctx.set_tail_mode(0)
    ctx.check_status()
    return res


def run_c1(ctx, iters=200):
    """Config 1, the two-layer MLP (256 tokens, 512 -> 1024 -> 256, ReLU, per-token activation scales): weights prepared
    on the device, then the forward pass as plain launches and as one recorded graph per pass."""
    from mlfw_b200 import synth
    M, D0, D1, D2 = 256, 512, 1024, 256
    x = ctx.to_device(synth.normal(synth.tensor_seed(0, 0), (M, D0)))
    layers = []
    for (n, k, sw, sb) in ((D1, D0, 1, 2), (D2, D1, 3, 4)):
        w = ctx.to_device(synth.normal(synth.tensor_seed(0, sw), (n, k), 0.0, 0.02))
        qw, ws = ctx.empty((n, k), np.int8), ctx.empty((n,), np.float32)
        ctx.quantize_weights_per_channel(w, n, k, 0, qw, ws)
        layers.append((qw, ws, ctx.to_device(synth.uniform(synth.tensor_seed(0, sb), (n,), -0.1, 0.1))))
    q0, s0 = ctx.empty((M, D0), np.int8), ctx.empty((M,), np.float32)
    q1, s1 = ctx.empty((M, D1), np.int8), ctx.empty((M,), np.float32)
    y = ctx.empty((M, D2), np.float32)

    def forward():
        ctx.quantize_per_token(x, M, D0, q0, s0)
        ctx.int8_linear_requant_token(q0, s0, layers[0][0], layers[0][1], layers[0][2], "relu", M, D1, D0, q1, s1)
        ctx.int8_linear(q1, s1, layers[1][0], layers[1][1], layers[1][2], "none", M, D2, D1, y)

    l0 = ctx.launch_count()
    for _ in range(5):
        forward()
    ctx.sync()
    launches = (ctx.launch_count() - l0) // 5
    ctx.timer_start()
    for _ in range(iters):
        forward()
    ms_plain = ctx.timer_stop() / iters
    ref = y.download()
    ctx.graph_begin()
    forward()
    graph = ctx.graph_end()
    for _ in range(5):
        ctx.graph_launch(graph)
    ctx.sync()
    ctx.timer_start()
    for _ in range(iters):
        ctx.graph_launch(graph)
    ms_graph = ctx.timer_stop() / iters
    same = bool(np.array_equal(y.download().view(np.uint32), ref.view(np.uint32)))
    ctx.graph_destroy(graph)
    ctx.check_status()
    best = min(ms_plain, ms_graph)
    return {"workload": "c1_mlp_256x512x1024x256_relu", "ms_per_pass_plain_launches": ms_plain, "ms_per_pass_recorded_graph": ms_graph,
            "tokens_per_s": M / (best * 1e-3), "gpu_launches_per_pass": launches, "graph_result_same_bits": same,
            "bound_by": "launch latency: 0.67 GOP and 1.3 MB of traffic per pass"}


def run_roundtrip(ctx, pk, iters, warmup):
    """Standalone quantize -> dequantize of f32 [16384,4096] with 0.1% outliers (HBM bound); per-kernel GB/s."""
    from mlfw_b200 import synth
    M2, K2 = C2_SHAPE
    x2 = c2_input()
    d2 = [ctx.to_device(x2), ctx.to_device(x2[::-1].copy())]      # two sets alternate: 671 MB per set pair, > L2
    q2 = [ctx.empty((M2, K2), np.int8) for _ in range(2)]
    s2 = [ctx.empty((M2,), np.float32) for _ in range(2)]
    y2 = [ctx.empty((M2, K2), np.float32) for _ in range(2)]
    for i in range(warmup):
        ctx.quantize_per_token(d2[i % 2], M2, K2, q2[i % 2], s2[i % 2])
        ctx.dequantize_per_token(q2[i % 2], s2[i % 2], M2, K2, y2[i % 2])
    ctx.profile_enable(True)
    ctx.profile_reset()
    for i in range(iters):
        ctx.quantize_per_token(d2[i % 2], M2, K2, q2[i % 2], s2[i % 2])
        ctx.dequantize_per_token(q2[i % 2], s2[i % 2], M2, K2, y2[i % 2])
    p2 = ctx.profile_read()
    ctx.profile_enable(False)
    ctx.check_status()
    bytes_each = 5.0 * M2 * K2 + 4.0 * M2
    rt = {}
    for name in ("quantize_per_token", "dequantize_per_token"):
        t, n = p2[name]
        gbs = bytes_each / (t / n * 1e-3) / 1e9
        rt[name] = {"achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                    "frac_of_nominal_8000": gbs / 8000.0, "avg_launch_ms": t / n}
    # The same kernels launched back to back (no event between launches: one pair of events around `iters` launches
    # of one kernel, inputs alternating), which is how they run inside a stream of work; the per-launch figures above
    # carry the events' own few microseconds per launch.
    for name, launch in (("quantize_per_token", lambda i: ctx.quantize_per_token(d2[i % 2], M2, K2, q2[i % 2], s2[i % 2])),
                         ("dequantize_per_token", lambda i: ctx.dequantize_per_token(q2[i % 2], s2[i % 2], M2, K2, y2[i % 2]))):
        for i in range(3):
            launch(i)
        ctx.sync()
        ctx.timer_start()
        for i in range(iters):
            launch(i)
        ms = ctx.timer_stop() / iters
        gbs = bytes_each / (ms * 1e-3) / 1e9
        rt[name]["back_to_back"] = {"achieved": gbs, "frac": gbs / pk["hbm_gbs"], "avg_launch_ms": ms, "launches": iters}
    ctx.check_status()
    return {"workload": "quantize -> dequantize, f32 [16384,4096], 0.1% outliers", "algorithmic_bytes": bytes_each, **rt}


C5_M, C5_DIMS, C5_ACTS = 4096, [8192, 28672, 8192, 28672, 8192], ["silu", "silu", "silu", "none"]


class Comm:
    """What the benchmark needs from the ranks: a barrier, max / min over ranks of a host number, all ranks' values,
    and a byte broadcast (torch.distributed when there is more than one rank; identity otherwise)."""

    def __init__(self, dist, local_rank):
        self.dist, self.local_rank = dist, local_rank

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def _reduce(self, v, op):
        if self.dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{self.local_rank}")
        self.dist.all_reduce(t, op=op)
        return float(t.item())

    def max(self, v: float) -> float:
        return self._reduce(v, self.dist.ReduceOp.MAX) if self.dist is not None else v

    def min(self, v: float) -> float:
        return self._reduce(v, self.dist.ReduceOp.MIN) if self.dist is not None else v

    def all(self, v: float):
        if self.dist is None:
            return [v]
        import torch
        world = self.dist.get_world_size()
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{self.local_rank}")
        out = torch.empty(world, dtype=torch.float64, device=t.device)
        self.dist.all_gather_into_tensor(out, t)
        return [float(x) for x in out.cpu()]

    def broadcast_bytes(self, data: bytes, n: int) -> bytes:
        if self.dist is None:
            return data
        import torch
        t = torch.zeros(n, dtype=torch.uint8, device=f"cuda:{self.local_rank}")
        if data is not None:
            t.copy_(torch.frombuffer(bytearray(data), dtype=torch.uint8))
        self.dist.broadcast(t, src=0)
        return bytes(t.cpu().numpy().tobytes())


def timed_steps(ctx, comm, step, steps, warmup):
    """`warmup` untimed steps, then `steps` steps between a barrier + sync on both sides; ms per step, max over ranks."""
    for i in range(warmup):
        step(i)
    ctx.sync()
    ctx.check_status()
    comm.barrier()
    ctx.sync()
    ctx.timer_start()
    for i in range(steps):
        step(i)
    ms = ctx.timer_stop()
    ctx.sync()
    comm.barrier()
    return comm.max(ms) / steps


@functools.lru_cache(maxsize=1)
def c5_layers():
    """Weights of the four wide linears, the same on every rank (numpy's PCG64, seed 5; scales ~U(1e-3,1e-2)/sqrt(K)
    so that activations stay O(1))."""
    gen = np.random.default_rng(5)
    layers = []
    for i in range(4):
        K, N = C5_DIMS[i], C5_DIMS[i + 1]
        w = gen.integers(-127, 128, size=(N, K), dtype=np.int8)
        ws = (gen.uniform(1e-3, 1e-2, N) / np.sqrt(K)).astype(np.float32)
        layers.append((w, ws, C5_ACTS[i]))
    return layers


def run_c5_records(ctx, comm, rank, world, steps, warmup, modes=("mshard", "nshard"), chunk_choices=(1, 2, 4)):
    """Config 5 at fixed total size (M = 4096 rows): unsharded on this rank's GPU (the yardstick and the expected
    values), rows split over the ranks (no collective), and output channels split over the ranks (one max-reduction
    of the row-range keys and one int8 all-gather per layer, NCCL inside the library, b200q_group_linear_nshard).
    Every sharded result is compared bit for bit with the unsharded one."""
    import mlfw_b200
    from mlfw_b200 import sharding, synth
    M, dims = C5_M, C5_DIMS
    x = synth.normal(synth.tensor_seed(5, 0), (M, dims[0]))
    layers = c5_layers()
    ops_total = sum(2.0 * M * dims[i] * dims[i + 1] for i in range(4))
    dx = ctx.to_device(x)
    dls = [(ctx.to_device(w), ctx.to_device(ws), a) for w, ws, a in layers]
    q = [ctx.empty((M, d), np.int8) for d in dims[:-1]]
    sc = [ctx.empty((M,), np.float32) for _ in dims[:-1]]
    ref_out = ctx.empty((M, dims[-1]), np.float32)

    def chain(xbuf, rows, out):
        ctx.quantize_per_token(xbuf, rows, dims[0], q[0], sc[0])
        for i, (dw, dws, a) in enumerate(dls):
            if i < 3:
                ctx.int8_linear_requant_token(q[i], sc[i], dw, dws, None, a, rows, dims[i + 1], dims[i], q[i + 1], sc[i + 1])
            else:
                ctx.int8_linear(q[i], sc[i], dw, dws, None, a, rows, dims[i + 1], dims[i], out)

    l0 = ctx.launch_count()
    chain(dx, M, ref_out)
    launches_per_step = ctx.launch_count() - l0
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    if rank == 0:
        sampler.start()
    ms_unsharded = timed_steps(ctx, comm, lambda i: chain(dx, M, ref_out), steps, warmup)
    clocks = sampler.stop() if rank == 0 else None
    ref_host = ref_out.download()
    # the same steps once more with an event pair around every kernel: where the step's time goes
    ctx.profile_enable(True)
    ctx.profile_reset()
    for _ in range(min(steps, 5)):
        chain(dx, M, ref_out)
    fam = ctx.profile_read()
    ctx.profile_enable(False)
    pk = peaks()
    records = {"unsharded_on_each_gpu": {"ms_per_step": ms_unsharded, "tokens_per_s": M / (ms_unsharded * 1e-3),
                                         "tops": ops_total / (ms_unsharded * 1e-3) / 1e12, "gpu_launches_per_step": launches_per_step,
                                         "frac_of_int8_proxy_burst": ops_total / (ms_unsharded * 1e-3) / 1e12 / (2 * pk["bf16_tflops"]),
                                         "frac_of_int8_proxy_sustained": ops_total / (ms_unsharded * 1e-3) / 1e12 / (2 * pk["bf16_tflops_sustained"]),
                                         "kernel_ms_per_step": {k: v[0] / min(steps, 5) for k, v in fam.items()},
                                         "clocks": clocks}}

    def record(ms, extra):
        return {"ms_per_step": ms, "tokens_per_s": M / (ms * 1e-3), "tops": ops_total / (ms * 1e-3) / 1e12,
                "efficiency_vs_n1": ms_unsharded / (world * ms), "n_gpus": world, **extra}

    if "mshard" in modes:
        r0, rows = sharding.row_block(M, world, rank)
        out = ctx.empty((rows, dims[-1]), np.float32)
        xrows = dx.ptr + r0 * dims[0] * 4
        ms = timed_steps(ctx, comm, lambda i: chain(xrows, rows, out), steps, warmup)
        same = bool((out.download().view(np.uint32) == ref_host[r0:r0 + rows].view(np.uint32)).all())
        records["c5_mshard"] = record(ms, {"matches_unsharded": bool(comm.min(1.0 if same else 0.0) == 1.0), "rows_per_gpu": rows,
                                           "parallelism": f"rows split x{world}, weights replicated, no collective",
                                           "bound_by": "tensor pipe + the f32 round trip of the per-token requantize; weight reads of 235 MB per layer per GPU stay below it"})
        out.free()

    if "nshard" in modes:
        uid = mlfw_b200.Group.unique_id() if rank == 0 else None
        uid = comm.broadcast_bytes(uid, 128)
        group = mlfw_b200.Group.join(ctx, uid, rank, world)
        try:
            cols = [d // world for d in dims[1:]]
            W = [dls[i][0].ptr + rank * cols[i] * dims[i] for i in range(4)]          # rows [rank*cols, ...) of the K-major weight
            WS = [dls[i][1].ptr + rank * cols[i] * 4 for i in range(4)]
            gq = [q[0]] + [ctx.empty((M, d), np.int8) for d in dims[1:-1]]
            gs = [sc[0]] + [ctx.empty((M,), np.float32) for _ in dims[1:-1]]
            out = ctx.empty((M, cols[3]), np.float32)

            def nstep(i):
                ctx.quantize_per_token(dx, M, dims[0], gq[0], gs[0])
                blocks = 1
                for li in range(4):
                    act = C5_ACTS[li]
                    if li < 3:
                        group.linear_nshard([gq[li]], [gs[li]], blocks, [W[li]], [WS[li]], None, act, M, dims[li + 1], dims[li],
                                            q_out=[gq[li + 1]], out_scales=[gs[li + 1]])
                    else:
                        group.linear_nshard([gq[li]], [gs[li]], blocks, [W[li]], [WS[li]], None, act, M, dims[li + 1], dims[li], out_f32=[out])
                    blocks = world

            by_chunks = {}
            all_same = True
            for ch in chunk_choices:
                group.set_chunks(ch)
                ms = timed_steps(ctx, comm, nstep, steps, warmup)
                group.sync()
                c0 = rank * cols[3]
                same = bool((out.download().view(np.uint32) == np.ascontiguousarray(ref_host[:, c0:c0 + cols[3]]).view(np.uint32)).all())
                same = bool(comm.min(1.0 if same else 0.0) == 1.0)
                all_same = all_same and same
                by_chunks[str(ch)] = {"ms_per_step": ms, "matches_unsharded": same}
            best = min(by_chunks, key=lambda k: by_chunks[k]["ms_per_step"])
            up_bytes = M * dims[1] * (world - 1) / world
            records["c5_nshard"] = record(by_chunks[best]["ms_per_step"], {
                "matches_unsharded": all_same, "row_chunks": int(best), "by_row_chunks": by_chunks, "nccl_version": group.nccl_version(),
                "parallelism": f"output channels split x{world}; per layer one max-reduction of 2*M range keys and one int8 all-gather (NCCL, inside libb200q.so)",
                "bytes_received_per_gpu_per_step": (2 * M * dims[1] + M * dims[2]) * (world - 1) / world,
                "bound_by": ("NVLink: the all-gather of the 28672-wide layers delivers %.0f MB to every GPU, as long as its GEMM share at %d GPUs"
                             % (up_bytes / 1e6, world)) if world > 1 else "same kernels as unsharded"})
        finally:
            group.close()
    for buf in [dx, ref_out] + q + sc:
        buf.free()
    return records


def run_c3_strong(ctx, comm, rank, world, steps, warmup, act="gelu_tanh"):
    """Config 3 at its fixed size: the 8192 rows split evenly over the ranks, weights replicated, no collective.
    Each rank cycles through all row blocks of the full input (its own first), so every step reads and writes
    memory that the previous steps have pushed out of L2 (the full input and output are 134 MB each)."""
    from mlfw_b200 import sharding, synth
    M, K, N = 8192, 4096, 4096
    x = synth.normal(synth.tensor_seed(0, 300), (M, K))
    W = synth.randint_i8(synth.tensor_seed(0, 1), (N, K))
    ws = synth.uniform(synth.tensor_seed(0, 2), (N,), 1e-3, 1e-2)
    bias = synth.normal(synth.tensor_seed(0, 3), (N,), 0.0, 0.01)
    dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
    ref, out = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
    ms_unsharded = timed_steps(ctx, comm, lambda i: ctx.linear_f32(dx, dW, dws, db, act, M, N, K, ref), steps, warmup)
    blocks = [sharding.row_block(M, world, r) for r in range(world)]

    def shard_step(i):
        r0, rows = blocks[(rank + i) % world]
        ctx.linear_f32(dx.ptr + r0 * K * 4, dW, dws, db, act, rows, N, K, out.ptr + r0 * N * 4)

    ms = timed_steps(ctx, comm, shard_step, steps, warmup)
    # the same cycle recorded once and replayed: one launch per `world` steps instead of two per step
    ms_graph, graph_note = None, None
    try:
        for i in range(world):
            shard_step(i)
        ctx.sync()
        ctx.graph_begin()
        try:
            for i in range(world):
                shard_step(i)
        finally:
            graph = ctx.graph_end()
        cycles = max(1, steps // world)
        ms_graph = timed_steps(ctx, comm, lambda i: ctx.graph_launch(graph), cycles, max(1, warmup // world)) / world
        ctx.graph_destroy(graph)
    except Exception as exc:                                   # the replayed form is an extra; the plain one stands
        graph_note = f"{type(exc).__name__}: {exc}"
    r0, rows = blocks[rank]
    out.fill_bytes(0)
    ctx.linear_f32(dx.ptr + r0 * K * 4, dW, dws, db, act, rows, N, K, out.ptr + r0 * N * 4)
    ctx.sync()
    got = out.download()[r0:r0 + rows]
    same = bool((got.view(np.uint32) == ref.download()[r0:r0 + rows].view(np.uint32)).all())
    same = bool(comm.min(1.0 if same else 0.0) == 1.0)
    best = min(ms, ms_graph) if ms_graph else ms
    rec = {"ms_per_step": best, "tokens_per_s": M / (best * 1e-3), "tops": 2.0 * M * N * K / (best * 1e-3) / 1e12,
           "efficiency_vs_n1": ms_unsharded / (world * best), "matches_unsharded": same, "n_gpus": world, "rows_per_gpu": rows,
           "ms_per_step_plain_launches": ms, "ms_per_step_replayed": ms_graph, "ms_unsharded_on_each_gpu": ms_unsharded,
           "parallelism": f"rows split x{world}, weights replicated, no collective; a step is one rank-local quantize + GEMM launch pair",
           "l2": "each rank cycles through all row blocks of the 134 MB input and output, so no step finds its data in L2",
           "bound_by": ("one wave of %d tiles of 256x256 on 74 CTA pairs plus launch latency: at %d rows per GPU the GEMM is %d tiles"
                        % ((rows + 255) // 256 * 16, rows, (rows + 255) // 256 * 16))}
    if graph_note:
        rec["replay_unavailable"] = graph_note
    for b in (dx, dW, dws, db, ref, out):
        b.free()
    return rec


def run_c4(args, ctx, rank, world, comm):
    barrier, max_over_ranks = comm.barrier, comm.max
    """Config 4: one pre-norm GPT block (d 768, 12 heads, ff 3072) over 32 x 512 tokens per GPU, from token ids to the
    block's output: embedding, LayerNorm + quantize, four int8 linears, causal attention, residual adds."""
    from mlfw_b200.block import GPTBlock, random_block_params
    D, H, FF, B, S, V = 768, 12, 3072, 32, 512, 50257
    M = B * S
    rng = np.random.default_rng(40 + rank)
    blk = GPTBlock(ctx, D, H, FF, random_block_params(D, FF, seed=4))
    table = ctx.to_device((rng.standard_normal((V, D)) * 0.02).astype(np.float32))
    tokens = [ctx.to_device(rng.integers(0, V, size=M).astype(np.int32)) for _ in range(2)]
    h, out = ctx.empty((M, D), np.float32), ctx.empty((M, D), np.float32)

    def step(i):
        ctx.embedding_f32(table, tokens[i % 2], None, M, D, V, S, h)
        blk.forward(h, B, S, out)

    for i in range(max(args.warmup, 3)):
        step(i)
    ctx.sync()
    ctx.check_status()
    launches0 = ctx.launch_count()
    barrier()
    ctx.sync()
    ctx.timer_start()
    for i in range(args.steps):
        step(i)
    ms = ctx.timer_stop()
    ctx.sync()
    barrier()
    launches = ctx.launch_count() - launches0
    # the same steps once more with an event pair around every kernel (kept out of the headline: the events sit
    # between the kernels and switch the dependent launches off)
    time.sleep(0.5)
    step(0)
    ctx.sync()
    ctx.profile_enable(True)
    ctx.profile_reset()
    for i in range(args.steps):
        step(i)
    ctx.sync()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    ctx.check_status()
    ms = max_over_ranks(ms) / args.steps
    gemm_ops = 2.0 * M * D * (3 * D + D + FF + FF)
    attn_flops = 4.0 * B * H * S * (S + 64) / 2 * 64       # causal: about half of the S x S scores, QK^T and PV
    per_kernel = {k: {"ms_per_step": v[0] / args.steps, "launches_per_step": v[1] / args.steps} for k, v in prof.items() if v[1]}
    pk = peaks()
    ln_ms = prof.get("layernorm_quantize", (0.0, 0))[0] / args.steps
    sd_ms = prof.get("sdpa", (0.0, 0))[0] / args.steps
    return {"metric": "int8_linear_tokens_per_s", "value": world * M / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32 linears; f32 LayerNorm, attention, residuals", "data": "synthetic",
            "config": {"workload": C4_WORKLOAD, "tokens_per_gpu": M, "d_model": D, "heads": H, "ff": FF, "batch": B, "seq": S,
                       "activation": "gelu_sigmoid", "parallelism": f"batch-sharded x{world}, weights replicated, no collective"},
            "tops": world * gemm_ops / (ms * 1e-3) / 1e12, "kernels": per_kernel,
            "roofline_layernorm_quantize": {"bound": "hbm", "achieved": (2 * 5.0 + 8.0) * M * D / (ln_ms * 1e-3) / 1e9 if ln_ms else None,
                                            "peak": pk["hbm_gbs"], "unit": "GB/s",
                                            "note": "two launches per step: 5 B/element (read x, write codes) and 13 B/element (read x and the residual, write their sum and the codes)"},
            "roofline_sdpa": {"bound": "tensor (tcgen05.mma kind::tf32, every product three ways)", "achieved": attn_flops / (sd_ms * 1e-3) / 1e12 if sd_ms else None,
                              "unit": "TFLOP/s of binary32-equivalent work", "tf32_tflops_issued": 3 * attn_flops / (sd_ms * 1e-3) / 1e12 if sd_ms else None,
                              "note": "the 1e-5 bar rules out single tf32 products: hi*hi + hi*lo + lo*hi per term, scores and P in tensor memory, two CTAs per SM"},
            "gpu_launches": launches}


def run_sustained(ctx, step, M, N, K, ms_burst, gpu_index, seconds=2.5):
    """The same step back to back for a few seconds, clocks sampled inside: what the part sustains under its power cap.
    No clock is set or reset; the dependence on the clock shows as throughput x (max MHz / median MHz)."""
    n = int(max(50, min(60000, seconds * 1e3 / max(ms_burst, 1e-3))))
    sampler = ClockSampler(gpu_index)
    ctx.sync()
    sampler.start()
    time.sleep(0.1)
    ctx.timer_start()
    for i in range(n):
        step(i)
    ms = ctx.timer_stop()
    clocks = sampler.stop()
    ctx.check_status()
    per = ms / n
    tops = 2.0 * M * N * K / (per * 1e-3) / 1e12
    rec = {"seconds": ms * 1e-3, "steps": n, "ms_per_step": per, "tokens_per_s": M / (per * 1e-3), "tops_step": tops, "clocks": clocks,
           "note": "tops_step counts the GEMM's 2*M*N*K over the whole step (quantize + GEMM); the GEMM's share of a step is in `roofline`"}
    if clocks.get("sm_mhz") and clocks.get("sm_max_mhz"):
        rec["tops_step_scaled_to_max_clock"] = tops * clocks["sm_max_mhz"] / clocks["sm_mhz"]
    return rec


def run_e2e(ctx, comm, rank, world, local_rank, args, M, K, N, act, x_host, dW, dws, db):
    """The step through the host-buffer entry point (b200q_linear_f32_host): page-locked buffers before and after the
    process is bound to its GPU's NUMA node, ordinary pageable numpy arrays (what a caller holding typed arrays has),
    and the bare copy bandwidths of every rank while all ranks copy at once."""
    out = {}
    e2e_steps = max(3, min(args.steps, 10))

    own = [0.0]      # this rank's own time of the last timed() call (the returned figure is the maximum over ranks)

    def timed(hx, hy):
        ctx.linear_f32_host(hx, dW, dws, db, act, M, N, K, hy)
        comm.barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ctx.linear_f32_host(hx, dW, dws, db, act, M, N, K, hy)
        own[0] = (time.perf_counter() - t0) / e2e_steps
        return comm.max(own[0])

    hx, hy = ctx.pinned((M, K), np.float32), ctx.pinned((M, N), np.float32)
    hx.array[...] = x_host
    dt_before = timed(hx, hy)
    own_before = own[0]
    checksum = float(hy.array[::997, ::97].sum())
    sample = hy.array[::997, ::97].copy()

    # bare copies, all ranks at once: where the host side saturates
    dtmp = ctx.empty((M, K), np.float32)
    reps = 3
    comm.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        dtmp.ctx.lib.b200q_upload(ctx.handle, dtmp.ptr, hx.ptr, M * K * 4)
    h2d = M * K * 4 * reps / (time.perf_counter() - t0) / 1e9
    comm.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        dtmp.ctx.lib.b200q_download(ctx.handle, hy.ptr, dtmp.ptr, M * K * 4)
    d2h = M * K * 4 * reps / (time.perf_counter() - t0) / 1e9
    dtmp.free()
    out["copy_bandwidth"] = {"h2d_gbs_per_rank": comm.all(h2d), "d2h_gbs_per_rank": comm.all(d2h),
                             "note": f"134 MB page-locked copies, one direction at a time, all {world} ranks copying at the same moment"}

    # pageable buffers: staged through the context's page-locked ring by its copy threads, in step with the transfers
    host_threads = max(1, min(8, (os.cpu_count() or 2) // (2 * world)))
    ctx.set_host_threads(host_threads)
    px = np.array(x_host, dtype=np.float32, copy=True)
    py = np.empty((M, N), np.float32)
    dt_pageable = timed(px, py)
    same_pageable = bool(np.array_equal(py[::997, ::97], sample))
    # the same two arrays page-locked in place once (b200q_host_register), as a caller that reuses its buffers can do
    t_reg = time.perf_counter()
    ctx.host_register(px)
    ctx.host_register(py)
    t_reg = time.perf_counter() - t_reg
    py[...] = 0.0
    dt_registered = timed(px, py)
    same_registered = bool(np.array_equal(py[::997, ::97], sample))
    ctx.host_unregister(px)
    ctx.host_unregister(py)

    # bound to the GPU's NUMA node: new page-locked buffers allocated after the binding
    numa = gpu_numa_info(local_rank)
    bound = bind_to_numa_node(numa)
    dt_after = None
    if bound.get("bound"):
        hx2, hy2 = ctx.pinned((M, K), np.float32), ctx.pinned((M, N), np.float32)
        hx2.array[...] = x_host
        dt_after = timed(hx2, hy2)
        hx2.free(); hy2.free()
    any_bound = comm.max(1.0 if dt_after is not None else 0.0) == 1.0
    if any_bound and dt_after is None:       # every rank takes part in the timed region's barrier
        dt_after = timed(hx, hy)
    hx.free(); hy.free()
    best = min(dt_before, dt_after) if dt_after else dt_before
    out["copy_bandwidth"]["both_directions_gbs_per_rank_in_the_e2e_step"] = [(M * K + M * N) * 4 / b / 1e9 for b in comm.all(own_before)]
    out["e2e"] = {"value": world * M / best, "unit": "tokens/s", "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4,
                  "ms_per_step": best * 1e3, "steps": e2e_steps, "result_checksum": checksum,
                  "api": "b200q_linear_f32_host (page-locked host input, host output, synchronous; row blocks pipelined over three streams)",
                  "ms_per_step_unbound": dt_before * 1e3, "ms_per_step_numa_bound": dt_after * 1e3 if dt_after else None,
                  "numa": {**{k: v for k, v in numa.items() if k != "gpu"}, **bound}}
    out["e2e_pageable"] = {"value": world * M / dt_pageable, "unit": "tokens/s", "ms_per_step": dt_pageable * 1e3, "steps": e2e_steps,
                           "same_result_as_page_locked": same_pageable,
                           "host_threads": host_threads,
                           "registered_in_place": {"ms_per_step": dt_registered * 1e3, "tokens_per_s": world * M / dt_registered,
                                                   "same_result_as_page_locked": same_registered, "register_ms_once": t_reg * 1e3,
                                                   "api": "b200q_host_register on the caller's two arrays, then the same calls"},
                           "api": "b200q_linear_f32_host with ordinary (pageable) numpy arrays, as a caller holding typed arrays would pass: "
                                  "row blocks staged through a page-locked ring by the context's copy threads"}
    return out


def _cpu_time(fn, reps):
    fn()
    t0 = time.perf_counter()
    for _ in range(reps):
        r = fn()
    return (time.perf_counter() - t0) / reps, r


def run_cpu_baselines(ctx, x, W, ws, bias, act, dout, M):
    """The CPU restatement of the reference timed on this machine's cores for every configuration: configs 1 and 2 in
    full, the large GEMM and the wide stack on their first 64 rows (rows are independent), the transformer block on
    one sequence of 512 tokens.  A reported baseline, not a target."""
    import oracle
    from mlfw_b200 import synth
    oracle.build()
    oracle.set_num_threads(oracle.usable_cores())
    cores = oracle.num_threads()
    res = {}
    rows = min(CPU_SAMPLE_ROWS, M)
    dt, (ref_out, _, _, _) = _cpu_time(lambda: oracle.linear(x[:rows], W, ws, bias, act), 3)
    rows1 = min(8, M)      # the reference's own execution model is one thread
    t0 = time.perf_counter()
    oracle.linear(x[:rows1], W, ws, bias, act, threads=1)
    dt1 = time.perf_counter() - t0
    got = dout.download()[:rows]
    err = float(np.abs(got.astype(np.float64) - ref_out).max() / np.abs(ref_out).max())
    c3 = {"value": rows / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
          "sample": f"first {rows} of {M} rows, all of N and K, 3 repetitions; C++ restatement of the reference's CPU path with OpenMP",
          "gpu_vs_cpu_max_err_over_absmax": err,
          "single_core": {"value": rows1 / dt1, "unit": "tokens/s", "sample": f"first {rows1} rows, one thread, one repetition"}}
    res["cpu_baseline"] = c3
    per = {"c3_gemm_8192x4096x4096": c3}

    # config 1: the two-layer MLP in full
    x1 = synth.normal(synth.tensor_seed(0, 0), (256, 512))
    w1 = synth.normal(synth.tensor_seed(0, 1), (1024, 512), 0.0, 0.02)
    w2 = synth.normal(synth.tensor_seed(0, 3), (256, 1024), 0.0, 0.02)
    b1 = synth.uniform(synth.tensor_seed(0, 2), (1024,), -0.1, 0.1)
    b2 = synth.uniform(synth.tensor_seed(0, 4), (256,), -0.1, 0.1)
    qw = []
    for w in (w1, w2):
        sc = oracle.per_channel_scales(w, w.shape, 0)
        qw.append((oracle.quantize_per_channel(w, w.shape, 0, sc), sc.astype(np.float32)))

    def mlp():
        h, _, _, _ = oracle.linear(x1, qw[0][0], qw[0][1], b1, "relu")
        return oracle.linear(h, qw[1][0], qw[1][1], b2, "none")[0]

    dt, _ = _cpu_time(mlp, 5)
    per["c1_mlp_256x512x1024x256"] = {"value": 256 / dt, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": "in full, 5 repetitions"}

    # config 2: the round trip in full
    M2, K2 = C2_SHAPE
    x2 = c2_input()

    def roundtrip():
        q, _, s32 = oracle.quantize_per_token(x2)
        return oracle.dequantize_per_token_f32(q, s32)

    dt, _ = _cpu_time(roundtrip, 2)
    per["c2_roundtrip_16384x4096"] = {"value": 2 * (5.0 * M2 * K2 + 4.0 * M2) / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                                      "sample": "in full (quantize + dequantize of 67.1 M elements), 2 repetitions; algorithmic bytes as for the GPU kernels"}

    # config 4: one sequence of 512 tokens through the whole block
    from mlfw_b200.block import random_block_params
    D, H, FF, S = 768, 12, 3072, 512
    prm = random_block_params(D, FF, seed=4)
    lin = {}
    for name, w, b in (("qkv", np.concatenate([prm["wq"], prm["wk"], prm["wv"]]), np.concatenate([prm["bq"], prm["bk"], prm["bv"]])),
                       ("o", prm["wo"], prm["bo"]), ("f1", prm["w1"], prm["b1"]), ("f2", prm["w2"], prm["b2"])):
        sc = oracle.per_channel_scales(w, w.shape, 0)
        lin[name] = (oracle.quantize_per_channel(w, w.shape, 0, sc), sc.astype(np.float32), b)
    h0 = (np.random.default_rng(40).standard_normal((S, D)) * 0.02).astype(np.float32)

    def block():
        n1 = oracle.layer_norm(h0, prm["ln1_gamma"], prm["ln1_beta"])
        qkv = oracle.linear(n1, *lin["qkv"], "none")[0]
        a = oracle.sdpa(np.ascontiguousarray(qkv[:, :D]), np.ascontiguousarray(qkv[:, D:2 * D]), np.ascontiguousarray(qkv[:, 2 * D:]),
                        1, H, S, 64, 0.125, True)
        o = oracle.linear(a, *lin["o"], "none")[0]
        n2, xsum = oracle.layer_norm(o, prm["ln2_gamma"], prm["ln2_beta"], add=h0, want_sum=True)
        f1 = oracle.linear(n2, *lin["f1"], "gelu_sigmoid")[0]
        f2 = oracle.linear(f1, *lin["f2"], "none")[0]
        return xsum + f2

    dt, _ = _cpu_time(block, 2)
    per["c4_gpt_block_d768_h12_ff3072"] = {"value": S / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                          "sample": "one sequence of 512 tokens (of 32) through the whole block, 2 repetitions"}

    # config 5: the first 64 rows through the four layers
    x5 = synth.normal(synth.tensor_seed(5, 0), (C5_M, C5_DIMS[0]))[:CPU_SAMPLE_ROWS]
    layers = c5_layers()

    def stack():
        h = x5
        for w, wsc, a in layers:
            h = oracle.linear(h, w, wsc, None, a)[0]
        return h

    dt, _ = _cpu_time(stack, 1)
    per["c5_stack_4096x8192x28672"] = {"value": CPU_SAMPLE_ROWS / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
                                      "sample": f"first {CPU_SAMPLE_ROWS} of {C5_M} rows through the four layers, one repetition after one warm-up"}
    res["cpu_baselines"] = per
    return res


def run_int_mm_peak(gpu_index):
    """One library int8 GEMM (torch._int_mm, cuBLASLt) at 8192^3 on this GPU, outside the product path: a measured int8
    tensor-core figure to hold the proxy denominator (2 x the measured bf16 figure) against."""
    try:
        import torch
        dev = torch.device("cuda", gpu_index)
        n = 8192
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev).t()     # column-major second operand
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize(dev)
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize(dev)
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        del a, b
        torch.cuda.empty_cache()
        return {"tops": 2.0 * n ** 3 / (best * 1e-3) / 1e12, "ms": best, "how": "torch._int_mm 8192^3 (raw int32 result, no tail), best of 10, CUDA events"}
    except Exception as exc:
        return {"tops": None, "unavailable": f"{type(exc).__name__}: {exc}"}


def run_reference_arm(args, rank, world):
    """The reference's CPU path (its C++ restatement: no JavaScript engine exists here) on all host cores."""
    if rank != 0:
        return None
    import oracle
    oracle.build()
    if args.workload not in WORKLOADS:   # the block and stack workloads have no CPU arm of their own: time the headline linear
        args.workload = DEFAULT_WORKLOAD
    M, K, N, act, xs, W, ws, bias = make_case(args.workload, 0)
    rows = min(CPU_SAMPLE_ROWS, M)
    x = xs[0][:rows]
    oracle.set_num_threads(oracle.usable_cores())   # torchrun exports OMP_NUM_THREADS=1; this arm uses every core it may
    cores = oracle.num_threads()
    for _ in range(max(1, min(args.warmup, 2))):
        oracle.linear(x, W, ws, bias, act)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear(x, W, ws, bias, act)
    dt = (time.perf_counter() - t0) / args.steps
    tps = rows / dt
    line = {
        "impl": "reference", "metric": "int8_linear_tokens_per_s", "value": tps, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 tail", "data": "synthetic",
        "config": {"workload": args.workload, "M_per_gpu": M, "K": K, "N": N, "activation": act},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"first {rows} of {M} rows per step, all of N and K; C++ restatement of the reference's "
                                   "TypeScript CPU path with OpenMP (the reference itself is single-threaded JavaScript and "
                                   "cannot run here)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    return line


class _QuietStdout:
    """Libraries (NCCL prints its version) must not add lines to stdout: fd 1 points at stderr until the JSON line."""

    def __enter__(self):
        sys.stdout.flush()
        self.saved = os.dup(1)
        os.dup2(2, 1)
        return self

    def __exit__(self, *exc):
        sys.stdout.flush()
        os.dup2(self.saved, 1)
        os.close(self.saved)


def main():
    with _QuietStdout():
        line = _run()
    if line is not None:
        print(json.dumps(line), flush=True)


def _run():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tail-mode", type=int, default=0, choices=[0, 1],
                    help="0: exact sigmoid tails (default); 1: hardware exp / reciprocal for f32 outputs (within the 1e-5 bar)")
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS) + [C4_WORKLOAD, C5_WORKLOAD])
    ap.add_argument("--mode", default="mshard", choices=["mshard", "nshard"],
                    help="config 5 only: rows split over the GPUs (no collective) or output channels split (NCCL all-gather)")
    ap.add_argument("--chunks", type=int, default=0, help="config 5, nshard: row chunks of the column-sharded call (0: try 1, 2 and 4)")
    ap.add_argument("--requant-variant", type=int, default=0, choices=[0, 1],
                    help="per-token requantize after a linear: 0 ranges from the GEMM epilogue + one-pass encode (default); 1 full quantize kernel")
    ap.add_argument("--epilogue-warps", type=int, default=0, choices=[0, 8, 16],
                    help="epilogue warps of the tensor-core GEMM for f32 output (0: sixteen for K <= 1024, eight otherwise)")
    ap.add_argument("--no-north-star", action="store_true", help="skip the fixed-size multi-GPU records (c3_strong, c5_mshard, c5_nshard)")
    ap.add_argument("--no-extras", action="store_true", help="skip the end-to-end, round-trip and CPU legs (profiler runs)")
    ap.add_argument("--quant-sweep", action="store_true", help="only the per-token quantize over row lengths 768..8192 and 8192 / 16384 rows")
    ap.add_argument("--tile-group", type=int, default=-1, help="tile walking order of the tensor-core GEMM (b200q_set_tile_group)")
    ap.add_argument("--tail-sweep", action="store_true", help="only config 5's up-projection shape with every fused tail")
    ap.add_argument("--conv-bench", action="store_true", help="only quantized_conv2d on ResNet-sized layers (gather + contraction), both layouts")
    ap.add_argument("--roundtrip-only", action="store_true", help="only the standalone quantize -> dequantize round trip (profiler runs)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" and not args.no_extras else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        return run_reference_arm(args, rank, world)

    import mlfw_b200
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    comm = Comm(dist, local_rank)
    barrier, max_over_ranks = comm.barrier, comm.max

    ctx = mlfw_b200.Context(local_rank)
    ctx.set_tail_mode(args.tail_mode)
    ctx.set_requant_variant(args.requant_variant)
    ctx.set_epilogue_warps(args.epilogue_warps)
    ctx.set_tile_group(args.tile_group)
    if args.roundtrip_only:
        line = {"metric": "quantize_dequantize_GBps", "roundtrip_c2": run_roundtrip(ctx, peaks(), args.steps, args.warmup)}
        ctx.close()
        return line
    if args.quant_sweep:
        line = {"metric": "quantize_per_token_GBps", "unit": "GB/s", "timing": "back to back, 40 launches per point",
                "quant_sweep": run_quant_sweep(ctx, peaks())}
        ctx.close()
        return line
    if args.tail_sweep:
        line = {"metric": "int8_linear_TOPs", "unit": "TOP/s", "shape": "M 4096, K 8192, N 28672", "tail_sweep": run_tail_sweep(ctx)}
        ctx.close()
        return line
    if args.conv_bench:
        line = {"metric": "quantized_conv2d_TOPs", "unit": "TOP/s", "timing": "back to back, 20 calls per point", "conv_bench": run_conv_bench(ctx, peaks())}
        ctx.close()
        return line
    if args.workload == C5_WORKLOAD:
        steps = min(args.steps, 50)
        recs = run_c5_records(ctx, comm, rank, world, steps, max(args.warmup, 3), modes=(args.mode,),
                              chunk_choices=(args.chunks,) if args.chunks else (1, 2, 4))
        rec = recs["c5_" + args.mode]
        line = {"metric": "int8_linear_tokens_per_s", "value": rec["tokens_per_s"], "unit": "tokens/s", "n_gpus": world, "steps": steps,
                "warmup": max(args.warmup, 3), "ms_per_step": rec["ms_per_step"], "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 tail", "data": "synthetic (weights from numpy's PCG64, seed 5)",
                "config": {"workload": C5_WORKLOAD, "M_total": C5_M, "dims": C5_DIMS, "activation": "silu", "mode": args.mode,
                           "parallelism": rec["parallelism"]},
                "tops": rec["tops"], "record": rec, "unsharded_on_each_gpu": recs["unsharded_on_each_gpu"]}
        ctx.close()
        if dist is not None:
            dist.destroy_process_group()
        return line if rank == 0 else None
    if args.workload == C4_WORKLOAD:
        line = run_c4(args, ctx, rank, world, comm)
        ctx.close()
        if dist is not None:
            dist.destroy_process_group()
        return line if rank == 0 else None
    M, K, N, act, xs, W, ws, bias = make_case(args.workload, rank)
    dxs = [ctx.to_device(x) for x in xs]
    douts = [ctx.empty((M, N), np.float32) for _ in xs]
    dW, dws, db = ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)

    def step(i):
        ctx.linear_f32(dxs[i % 2], dW, dws, db, act, M, N, K, douts[i % 2])

    for i in range(args.warmup):
        step(i)
    ctx.sync()
    ctx.check_status()

    # ------------------------------------------------------------ timed region (device resident)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count()
    barrier()
    ctx.sync()
    ctx.timer_start()
    for i in range(args.steps):
        step(i)
    ms = ctx.timer_stop()
    ctx.sync()
    barrier()
    launches = ctx.launch_count() - launches0
    # The same steps once more with an event pair around every kernel (the per-kernel figures of the roofline); the
    # events sit between the kernels, so this pass is kept out of the headline.
    time.sleep(0.5)     # both passes start from the same clocks: a long busy stretch runs into the power cap
    for i in range(min(args.warmup, 5)):
        step(i)
    ctx.sync()
    ctx.profile_enable(True)
    ctx.profile_reset()
    for i in range(args.steps):
        step(i)
    ctx.sync()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    clocks = sampler.stop() if rank == 0 else None
    ctx.check_status()
    ms = max_over_ranks(ms)
    ms_per_step = ms / args.steps
    tokens_per_s = world * M / (ms_per_step * 1e-3)

    pk = peaks()
    gemm_ms, gemm_n = prof.get("gemm_tensor_core", (0.0, 0))
    quant_ms, quant_n = prof.get("quantize_per_token", (0.0, 0))
    gemm_avg_ms = gemm_ms / max(gemm_n, 1)
    int8_peak = 2.0 * pk["bf16_tflops"]
    achieved_tops = 2.0 * M * N * K / (gemm_avg_ms * 1e-3) / 1e12 if gemm_n else None
    roofline = {
        "kernel": "gemm_i8_umma_kernel (tcgen05.mma kind::i8 + fused tail)", "bound": "tensor", "achieved": achieved_tops,
        "peak": int8_peak, "unit": "TOP/s", "frac": (achieved_tops / int8_peak) if achieved_tops else None,
        "peak_note": f"2 x bf16_tflops of {pk['source']} peaks (no int8 figure is measured on this pool); nominal dense int8 is 4500",
        # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this size, from an ncu capture
        # at full size (52.0 MB read + 86.0 MB written; the rest of the 134 MB of output is still in L2 when the
        # kernel ends); algorithmic bytes are 184.6 MB
        "traffic": 138.0e6 if (M, K, N) == (8192, 4096, 4096) else None, "avg_launch_ms": gemm_avg_ms, "launches": gemm_n,
        "algorithmic_ops_per_launch": 2.0 * M * N * K,
        # a timed region of a tenth of a second or more runs under the power cap: the sustained figure is its yardstick
        "peak_sustained": 2.0 * pk["bf16_tflops_sustained"],
        "frac_of_sustained": (achieved_tops / (2.0 * pk["bf16_tflops_sustained"])) if achieved_tops else None,
        "regime": "sustained (long timed region, power cap)" if ms >= 100.0 else "burst",
    }
    if quant_n:
        q_avg = quant_ms / quant_n
        roofline_quant = {"kernel": "quantize_per_token_warp_kernel (teams of warps, the row in registers)", "bound": "hbm", "achieved": 5.0 * M * K / (q_avg * 1e-3) / 1e9,
                          "peak": pk["hbm_gbs"], "unit": "GB/s", "avg_launch_ms": q_avg, "launches": quant_n}
        roofline_quant["frac"] = roofline_quant["achieved"] / pk["hbm_gbs"]
    else:
        roofline_quant = None

    line = {
        "metric": "int8_linear_tokens_per_s", "value": tokens_per_s, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x int8 -> int32, f32 tail", "data": "synthetic",
        "config": {"workload": args.workload, "M_per_gpu": M, "K": K, "N": N, "activation": act,
                   "parallelism": f"M-sharded x{world}, weights replicated, no collective",
                   "l2": "each step reads 134 MB of f32 activations and writes 134 MB of f32 results (> 126 MB L2); two buffer sets alternate"},
        "tops": world * 2.0 * M * N * K / (ms_per_step * 1e-3) / 1e12,
        "roofline": roofline, "roofline_quantize": roofline_quant, "gpu_launches": launches, "clocks": clocks,
    }

    if not args.no_extras:
        # -------------------------------------------------------- spread of single steps (each one timed and synchronised by itself)
        samples = []
        for i in range(50):
            ctx.timer_start()
            step(i)
            samples.append(ctx.timer_stop())
        q1, med, q3 = (float(v) for v in np.percentile(samples, [25, 50, 75]))
        line["step_samples_ms"] = {"n": len(samples), "median": med, "iqr": q3 - q1, "min": float(min(samples)), "max": float(max(samples)),
                                   "note": "CUDA events around single synchronised steps; the headline times all steps back to back"}

        # -------------------------------------------------------- the same steps handed over as a queue of independent batches
        # (b200q_linear_f32_many: the quantize of batch i+1 overlaps the GEMM of batch i on a second stream); same buffers,
        # same number of steps, one call; the headline above stays the one-batch-per-call figure
        n_b = args.steps
        bx, bo = [dxs[i % 2] for i in range(n_b)], [douts[i % 2] for i in range(n_b)]
        for _ in range(2):
            ctx.linear_f32_many(bx, dW, dws, db, act, M, N, K, bo)
        ctx.sync()
        ref_bits = douts[0].download()[::509, ::127].copy()
        step(0)
        ctx.sync()
        same = bool(np.array_equal(douts[0].download()[::509, ::127].view(np.uint32), ref_bits.view(np.uint32)))
        barrier()
        ctx.sync()
        ctx.timer_start()
        ctx.linear_f32_many(bx, dW, dws, db, act, M, N, K, bo)
        ms_many = max_over_ranks(ctx.timer_stop())
        barrier()
        line["queued_batches"] = {"ms_per_step": ms_many / n_b, "tokens_per_s": world * M / (ms_many / n_b * 1e-3), "steps": n_b,
                                  "tops": world * 2.0 * M * N * K / (ms_many / n_b * 1e-3) / 1e12, "same_result_as_one_batch_per_call": same,
                                  "api": "b200q_linear_f32_many: one call for all steps, the per-token quantize of batch i+1 on a second stream "
                                         "while the GEMM of batch i runs"}

        if world == 1:
            line["c1_mlp"] = run_c1(ctx)

        # -------------------------------------------------------- sustained regime (N = 1: a seconds-long stretch under the power cap)
        if world == 1:
            line["sustained"] = run_sustained(ctx, step, M, N, K, ms_per_step, local_rank)

        # -------------------------------------------------------- end to end (host buffers)
        line.update(run_e2e(ctx, comm, rank, world, local_rank, args, M, K, N, act, xs[0], dW, dws, db))

        # -------------------------------------------------------- the fixed-size multi-GPU runs (strong scaling, value-checked)
        if not args.no_north_star:
            for b in dxs + douts:
                b.free()
            ns_steps, ns_warm = min(args.steps, 40), min(max(args.warmup, 3), 5)
            ns = {"c3_strong": run_c3_strong(ctx, comm, rank, world, ns_steps, ns_warm)}
            ns.update(run_c5_records(ctx, comm, rank, world, min(ns_steps, 20), 3))
            line["north_star_runs"] = ns
            dxs = [ctx.to_device(x) for x in xs]
            douts = [ctx.empty((M, N), np.float32) for _ in xs]

        if rank == 0 and world == 1:
            line["roundtrip_c2"] = run_roundtrip(ctx, pk, iters=20, warmup=4)
            step(0)
            ctx.sync()
            line.update(run_cpu_baselines(ctx, xs[0], W, ws, bias, act, douts[0], M))
            line["int8_peak_measured"] = run_int_mm_peak(local_rank)
            if line["int8_peak_measured"].get("tops") and roofline["achieved"]:
                roofline["frac_of_int8_peak_measured"] = roofline["achieved"] / line["int8_peak_measured"]["tops"]

    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else None


if __name__ == "__main__":
    main()
