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
`cpu_baseline` the CPU port timed on this machine.
"""
from __future__ import annotations

import argparse
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


def make_case(workload: str, rank: int):
    from mlfw_b200 import synth
    M, K, N, act = WORKLOADS[workload]
    seed = 0
    xs = [synth.normal(synth.tensor_seed(seed, 100 + 10 * rank + i), (M, K)) for i in range(2)]
    W = synth.randint_i8(synth.tensor_seed(seed, 1), (N, K))
    ws = synth.uniform(synth.tensor_seed(seed, 2), (N,), 1e-3, 1e-2)
    bias = synth.normal(synth.tensor_seed(seed, 3), (N,), 0.0, 0.01)
    return M, K, N, act, xs, W, ws, bias


def run_roundtrip(ctx, pk, iters, warmup):
    """Standalone quantize -> dequantize of f32 [16384,4096] with 0.1% outliers (HBM bound); per-kernel GB/s."""
    from mlfw_b200 import synth
    M2, K2 = C2_SHAPE
    x2 = synth.with_outliers(synth.normal(synth.tensor_seed(0, 20), (M2, K2)), synth.tensor_seed(0, 21), synth.tensor_seed(0, 22))
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


def run_c5(args, ctx, dist, rank, world, local_rank, barrier, max_over_ranks):
    """Config 5: four int8 linears 8192 <-> 28672 with SiLU and a per-token requantize between them, M = 4096 rows in
    total (strong scaling).  mshard: each rank takes M / world rows of every layer, weights replicated, no
    collective.  nshard: each rank takes N / world output channels of every layer; per layer two [M]-float
    all-reduces (row ranges) and one int8 all-gather of the column blocks over NVLink."""
    import torch
    from mlfw_b200 import sharding, synth
    M, dims, acts = 4096, [8192, 28672, 8192, 28672, 8192], ["silu", "silu", "silu", "none"]
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    gen = np.random.default_rng(5)                               # same weights on every rank
    x = synth.normal(synth.tensor_seed(5, 0), (M, dims[0]))
    layers = []
    for i in range(4):
        K, N = dims[i], dims[i + 1]
        w = gen.integers(-127, 128, size=(N, K), dtype=np.int8)
        ws = (gen.uniform(1e-3, 1e-2, N) / np.sqrt(K)).astype(np.float32)
        layers.append((w, ws, acts[i]))
    ops_total = sum(2.0 * M * dims[i] * dims[i + 1] for i in range(4))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    if args.mode == "mshard":
        r0, rows = sharding.row_block(M, world, rank)
        dx = ctx.to_device(x[r0:r0 + rows])
        dls = [(ctx.to_device(w), ctx.to_device(ws), a) for w, ws, a in layers]
        q = [ctx.empty((rows, d), np.int8) for d in dims[:-1]]
        sc = [ctx.empty((rows,), np.float32) for _ in dims[:-1]]
        out = ctx.empty((rows, dims[-1]), np.float32)

        def step():
            ctx.quantize_per_token(dx, rows, dims[0], q[0], sc[0])
            for i, (dw, dws, a) in enumerate(dls):
                if i < 3:
                    ctx.int8_linear_requant_token(q[i], sc[i], dw, dws, None, a, rows, dims[i + 1], dims[i], q[i + 1], sc[i + 1])
                else:
                    ctx.int8_linear(q[i], sc[i], dw, dws, None, a, rows, dims[i + 1], dims[i], out)
            ctx.sync()
    else:
        shards = []
        for i, (w, ws, a) in enumerate(layers):
            c0, cols = sharding.column_block(dims[i + 1], world, rank)
            shards.append(sharding.ShardedLayer(dims[i], dims[i + 1], c0, cols, torch.from_numpy(np.ascontiguousarray(w[c0:c0 + cols])).to(dev),
                                                torch.from_numpy(ws[c0:c0 + cols].copy()).to(dev), None, a))
        stack = sharding.ColumnShardedStack(sharding.DeviceOps(ctx, torch), dist, rank, world, shards)
        tx = torch.from_numpy(x).to(dev)
        tq = torch.empty((M, dims[0]), dtype=torch.int8, device=dev)
        ts = torch.empty((M,), dtype=torch.float32, device=dev)

        def step():
            torch.cuda.current_stream(dev).synchronize()
            ctx.quantize_per_token(tx.data_ptr(), M, dims[0], tq.data_ptr(), ts.data_ptr())
            ctx.sync()
            stack.forward(tq, ts, M, last_f32=True)
            torch.cuda.current_stream(dev).synchronize()

    del layers
    for _ in range(max(args.warmup, 3)):
        step()
    ctx.check_status()
    launches0 = ctx.launch_count()
    barrier()
    torch.cuda.synchronize(dev)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize(dev)
    ms = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    ctx.check_status()
    return {"metric": "int8_linear_tokens_per_s", "value": M / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "int8 x int8 -> int32, f32 tail", "data": "synthetic (weights from numpy's PCG64, seed 5)",
            "config": {"workload": C5_WORKLOAD, "M_total": M, "dims": dims, "activation": "silu", "mode": args.mode,
                       "parallelism": (f"M-sharded x{world}, weights replicated, no collective" if args.mode == "mshard" else
                                       f"N-sharded x{world}: per layer 2 all-reduces of [M] floats + 1 int8 all-gather (NCCL)")},
            "tops": ops_total / (ms * 1e-3) / 1e12, "gpu_launches": ctx.launch_count() - launches0}


def run_c4(args, ctx, rank, world, barrier, max_over_ranks):
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
            "roofline_sdpa": {"bound": "fp32 CUDA cores", "achieved": attn_flops / (sd_ms * 1e-3) / 1e12 if sd_ms else None, "unit": "TFLOP/s",
                              "note": "binary32 FMA on CUDA cores (the 1e-5 bar rules out tf32 tensor-core products)"},
            "gpu_launches": launches}


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
    ap.add_argument("--no-extras", action="store_true", help="skip the end-to-end, round-trip and CPU legs (profiler runs)")
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

    def barrier():
        if dist is not None:
            dist.barrier()

    def max_over_ranks(v: float) -> float:
        if dist is None:
            return v
        import torch
        t = torch.tensor([v], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    ctx = mlfw_b200.Context(local_rank)
    ctx.set_tail_mode(args.tail_mode)
    if args.roundtrip_only:
        line = {"metric": "quantize_dequantize_GBps", "roundtrip_c2": run_roundtrip(ctx, peaks(), args.steps, args.warmup)}
        ctx.close()
        return line
    if args.workload == C5_WORKLOAD:
        line = run_c5(args, ctx, dist, rank, world, local_rank, barrier, max_over_ranks)
        ctx.close()
        if dist is not None:
            dist.destroy_process_group()
        return line if rank == 0 else None
    if args.workload == C4_WORKLOAD:
        line = run_c4(args, ctx, rank, world, barrier, max_over_ranks)
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
        roofline_quant = {"kernel": "quantize_per_token_staged_kernel", "bound": "hbm", "achieved": 5.0 * M * K / (q_avg * 1e-3) / 1e9,
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

        # -------------------------------------------------------- end to end (host buffers)
        hx = ctx.pinned((M, K), np.float32)
        hy = ctx.pinned((M, N), np.float32)
        hx.array[...] = xs[0]
        e2e_steps = max(3, min(args.steps, 10))
        ctx.linear_f32_host(hx, dW, dws, db, act, M, N, K, hy)
        barrier()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            ctx.linear_f32_host(hx, dW, dws, db, act, M, N, K, hy)
        dt = max_over_ranks((time.perf_counter() - t0) / e2e_steps)
        checksum = float(hy.array[::997, ::97].sum())
        line["e2e"] = {"value": world * M / dt, "unit": "tokens/s", "h2d_bytes_per_step": M * K * 4, "d2h_bytes_per_step": M * N * 4,
                       "ms_per_step": dt * 1e3, "steps": e2e_steps, "result_checksum": checksum,
                       "api": "b200q_linear_f32_host (pinned host input, host output, synchronous)"}

        if rank == 0 and world == 1:
            line["roundtrip_c2"] = run_roundtrip(ctx, pk, iters=20, warmup=4)

            # ---------------------------------------------------- CPU baseline (bounded sample)
            import oracle
            oracle.build()
            rows = min(CPU_SAMPLE_ROWS, M)
            oracle.set_num_threads(oracle.usable_cores())
            cores = oracle.num_threads()
            oracle.linear(xs[0][:rows], W, ws, bias, act)
            t0 = time.perf_counter()
            reps = 3
            for _ in range(reps):
                ref_out, _, _, _ = oracle.linear(xs[0][:rows], W, ws, bias, act)
            dt_cpu = (time.perf_counter() - t0) / reps
            rows1 = min(8, M)      # the reference's own execution model is one thread
            t0 = time.perf_counter()
            oracle.linear(xs[0][:rows1], W, ws, bias, act, threads=1)
            dt_cpu1 = time.perf_counter() - t0
            step(0)
            ctx.sync()
            got = douts[0].download()[:rows]
            err = float(np.abs(got.astype(np.float64) - ref_out).max() / np.abs(ref_out).max())
            line["cpu_baseline"] = {"value": rows / dt_cpu, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"first {rows} of {M} rows, all of N and K, {reps} repetitions; C++ restatement of the "
                                              "reference's CPU path with OpenMP", "gpu_vs_cpu_max_err_over_absmax": err,
                                    "single_core": {"value": rows1 / dt_cpu1, "unit": "tokens/s", "sample": f"first {rows1} rows, one thread, one repetition"}}

    ctx.close()
    if dist is not None:
        dist.destroy_process_group()
    return line if rank == 0 else None


if __name__ == "__main__":
    main()
