"""The allocation-free entry point against the ordinary one (through the C ABI).

Some callers of libb200q.so may not allocate device memory inside a call: their own pool owns the whole device,
or they sit in a latency-bound loop where an allocation could stall every stream.  For them
b200q_linear_f32_noalloc keeps its scratch (int8 activations, per-token scales) in a fixed array inside the
library.  The array is shared between calls and keeps the previous call's contents, so the check runs two calls
in a row with different inputs and shapes: stale contents must not leak into the second result.  A second case
enqueues several calls back to back on one context with nothing between them (the array is reused while the
previous call's GEMM may still be running unless the kernels order themselves), and a third checks that a warmed
call leaves the device's free memory where it was.

This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _case(seed, M, N, K):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal((M, K)).astype(np.float32)
    W = rng.integers(-127, 128, size=(N, K)).astype(np.int8)
    ws = (rng.uniform(1e-3, 1e-2, size=N) / np.sqrt(K) * 8).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    return x, W, ws, bias


def test_noalloc_matches_allocating_entry_point_twice_in_a_row():
    import mlfw_b200
    with mlfw_b200.Context(0) as ctx:
        # second case is smaller than the first: whatever the first left behind in the scratch lies beyond it
        for seed, (M, N, K), act in [(1, (640, 768, 1024), "relu"), (2, (130, 260, 144), "gelu_sigmoid")]:
            x, W, ws, bias = _case(seed, M, N, K)
            dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
            ref, out = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
            out.fill_bytes(0xFF)
            ctx.linear_f32(dx, dW, dws, db, act, M, N, K, ref)
            ctx.linear_f32_noalloc(dx, dW, dws, db, act, M, N, K, out)
            ctx.sync()
            ctx.check_status()
            a, b = out.download(), ref.download()
            # same kernels, same inputs: the two entry points agree bit for bit (the suite's bar is 1e-5 of absmax)
            assert np.abs(a.astype(np.float64) - b).max() <= 1e-5 * np.abs(b).max()
            assert (a.view(np.uint32) == b.view(np.uint32)).all()


def test_noalloc_calls_enqueued_back_to_back():
    """Three calls on one context with no synchronisation and no other call between them, different inputs, shapes and
    outputs: a staged-quantize shape (M >= 64, rows of at most 16 KB), a register-path shape (M = 32) and a CTA-pair
    shape (M >= 1024).  Each result must equal b200q_linear_f32's, computed separately, bit for bit."""
    import mlfw_b200
    with mlfw_b200.Context(0) as ctx:
        cases = [(11, (1024, 512, 2048), "gelu_sigmoid"), (12, (32, 256, 4096), "relu"), (13, (640, 768, 1024), "silu")]
        held = []
        for seed, (M, N, K), act in cases:
            x, W, ws, bias = _case(seed, M, N, K)
            dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
            ref, out = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
            out.fill_bytes(0xFF)
            ctx.linear_f32(dx, dW, dws, db, act, M, N, K, ref)
            held.append((dx, dW, dws, db, act, M, N, K, ref, out))
        ctx.sync()
        for _ in range(2):                                  # twice over, so every shape also follows every other
            for dx, dW, dws, db, act, M, N, K, ref, out in held:
                ctx.linear_f32_noalloc(dx, dW, dws, db, act, M, N, K, out)
        ctx.sync()
        ctx.check_status()
        for *_, ref, out in held:
            assert (out.download().view(np.uint32) == ref.download().view(np.uint32)).all()


def test_noalloc_leaves_free_device_memory_unchanged():
    """After one warm-up call of the same kind, a call must not change the device's free memory (cudaMemGetInfo)."""
    import torch
    import mlfw_b200
    for device in range(min(2, torch.cuda.device_count())):      # the address cache is per device ordinal
        with mlfw_b200.Context(device) as ctx:
            M, N, K = 512, 512, 1024
            x, W, ws, bias = _case(21 + device, M, N, K)
            dx, dW, dws, db = ctx.to_device(x), ctx.to_device(W), ctx.to_device(ws), ctx.to_device(bias)
            ref, out = ctx.empty((M, N), np.float32), ctx.empty((M, N), np.float32)
            ctx.linear_f32(dx, dW, dws, db, "relu", M, N, K, ref)
            ctx.linear_f32_noalloc(dx, dW, dws, db, "relu", M, N, K, out)       # warm-up: kernel code and attributes
            ctx.sync()
            free0, _ = torch.cuda.mem_get_info(device)
            for _ in range(3):
                ctx.linear_f32_noalloc(dx, dW, dws, db, "relu", M, N, K, out)
            ctx.sync()
            free1, _ = torch.cuda.mem_get_info(device)
            assert free1 == free0, f"device {device}: free memory moved by {free0 - free1} bytes across allocation-free calls"
            assert (out.download().view(np.uint32) == ref.download().view(np.uint32)).all()


def test_noalloc_rejects_what_does_not_fit():
    import mlfw_b200
    with mlfw_b200.Context(0) as ctx:
        d = ctx.empty((16,), np.float32)
        with pytest.raises(mlfw_b200.B200QError, match="exceeds the fixed scratch"):
            ctx.linear_f32_noalloc(d, d, d, None, "none", 2048, 256, 4096, d)      # 8 Mi activation elements
        with pytest.raises(mlfw_b200.B200QError, match="exceeds the fixed scratch"):
            ctx.linear_f32_noalloc(d, d, d, None, "none", 20000, 256, 16, d)       # too many rows
        with pytest.raises(mlfw_b200.B200QError, match="exceeds the fixed scratch"):
            ctx.linear_f32_noalloc(d, d, d, None, "none", 16384, 256, 2 ** 50, d)  # M * K would overflow 64 bits
        with pytest.raises(mlfw_b200.B200QError, match="CUDA-core kernel"):
            ctx.linear_f32_noalloc(d, d, d, None, "none", 8, 8, 10, d)             # K not a multiple of 16
