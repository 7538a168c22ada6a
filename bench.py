#!/usr/bin/env python
"""Benchmark of the quantized-linear decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config.workload): the int4 group-128 decode linear at the Llama-70B
MLP shape — x float32 [1, 8192] ~ N(0, 1), W float32 [28672, 8192]
~ N(0, 0.015) quantized asymmetric uint4 per group of 128 — seeded synthetic
data standing in for a checkpoint. At N = 1 the whole layer runs on one GPU; at
N > 1 it is column-sharded (rank r owns output features [r n/N, (r+1) n/N))
and every call ends with the full y[1, 28672] on every rank: the gather is
part of the call (this library's own, fused into the GEMV's epilogue). One STEP
is one pass of x through R distinct device copies of the (sharded) weight, R
chosen so that a rank's copies exceed twice the L2 (every call streams its
weight from HBM), replayed as one CUDA graph the way a captured decode step
runs. Total work is fixed as N grows: strong scaling.

metric / value : algorithmic GB/s = whole-layer bytes (packed weight + scales +
                 zero points + x + y, each counted once) per call / device
                 time per call, inputs resident in HBM, timed with CUDA events
                 on the launching stream, max over ranks.
e2e            : the same pass through the public API with HOST buffers: per
                 step x is copied from pinned host memory, the graph replayed,
                 the R outputs (one contiguous buffer) copied back and waited
                 for (host wall clock, max over ranks).
roofline       : achieved = this rank's algorithmic bytes per launch / average
                 launch duration over the timed region; peak = measured HBM
                 copy bandwidth from MEASURED_PEAKS.json (else the fallback).
cpu_baseline   : the CPU oracle (a port of the reference's shader arithmetic)
                 timed on the host cores on a bounded sample of the workload.
extras         : the other configurations (C1, C2, C3 at more rows, C4 prefill,
                 C5 decode step) and, at N > 1, the sharded layer's variants
                 with their parity against the unsharded layer.

--impl reference times that CPU implementation alone, on the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GROUP = 128
C2 = {"n": 14336, "k": 4096, "sigma": 0.02, "seed": 1}   # Llama-8B MLP up-projection
C3 = {"n": 28672, "k": 8192, "sigma": 0.015, "seed": 2}  # Llama-70B MLP up-projection: the headline
SIGMA, SEED = 0.02, 1
METRIC, UNIT = "int4_g128_decode_linear_algorithmic_bandwidth", "GB/s"


def algorithmic_bytes(m: int, n: int, k: int, group: int = GROUP) -> int:
    words = -(-k // 32) * 4
    groups = -(-k // group)
    return n * words * 4 + 2 * n * groups * 4 + m * k * 4 + m * n * 4


def replicas_for(world: int) -> int:
    """Weight copies per rank so that a rank's copies exceed 2 x 126 MB of L2."""
    per_rank = algorithmic_bytes(1, C3["n"] // world, C3["k"])
    return max(4, -(-256_000_000 // per_rank))


def shard_weight(rank: int, world: int) -> np.ndarray:
    """The rows rank `rank` of `world` owns, seeded per shard so that any rank can rebuild any shard."""
    rng = np.random.default_rng(C3["seed"] * 1000 + world * 10 + rank)
    return (rng.standard_normal((C3["n"] // world, C3["k"])) * C3["sigma"]).astype(np.float32)


def c3_x(m: int) -> np.ndarray:
    return np.random.default_rng(C3["seed"]).standard_normal((16, C3["k"])).astype(np.float32)[:m]


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples taken while the GPU is under load."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index, self.proc, self.path = index, None, f"/tmp/gq_clocks_{os.getpid()}.csv"

    def start(self) -> None:
        try:
            self.out = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)], stdout=self.out, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.out.close()
        sm, mx, reasons = [], [], set()
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.remove(self.path)
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


def cpu_inputs(world: int):
    """What the CPU arms multiply: the first rank's shard of the layer (the same rows the GPU arm's rank 0 holds),
    quantized by the oracle. A bounded sample: 1/world of the layer, scaled up in the value."""
    import oracle
    w = shard_weight(0, world)
    q, scale, zero = oracle.quantize_q4(w, GROUP)
    return c3_x(1), q, scale, zero


def cpu_run(seconds: float, world: int = 1, threads: int | None = None):
    """The oracle's int4 linear on one shard of the layer, all host threads, repeated for about `seconds`:
    returns (whole-layer-equivalent GB/s, calls, threads, seconds)."""
    import oracle
    oracle.set_threads(threads or os.cpu_count() or 1)
    x, q, scale, zero = cpu_inputs(world)
    k = C3["k"]
    oracle.linear_q4(x, q, scale, zero, None, k, GROUP)  # warm
    calls, t0 = 0, time.perf_counter()
    while True:
        oracle.linear_q4(x, q, scale, zero, None, k, GROUP)
        calls += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return algorithmic_bytes(1, C3["n"] // world, k) * calls / dt / 1e9, calls, oracle.threads(), dt


def run_reference(args) -> None:
    """The CPU implementation alone, on the GPU arm's metric and config. torchrun exports OMP_NUM_THREADS=1 to its
    workers; the thread count is set here, to every host core, so the launcher cannot shrink the baseline. Each of
    the K steps is a whole number of M = 1 calls over one shard, chosen after the warm-up so that the K steps take
    at least three seconds."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    world = max(args.gpus, 1)
    oracle.set_threads(os.cpu_count() or 1)
    x, q, scale, zero = cpu_inputs(world)
    k = C3["k"]
    for _ in range(max(args.warmup, 1)):
        oracle.linear_q4(x, q, scale, zero, None, k, GROUP)
    t0 = time.perf_counter()
    oracle.linear_q4(x, q, scale, zero, None, k, GROUP)
    t_call = max(time.perf_counter() - t0, 1e-6)
    steps = max(args.steps, 1)
    calls_per_step = max(1, int(np.ceil(3.0 / (steps * t_call))))
    t0 = time.perf_counter()
    for _ in range(steps * calls_per_step):
        oracle.linear_q4(x, q, scale, zero, None, k, GROUP)
    dt = time.perf_counter() - t0
    value = algorithmic_bytes(1, C3["n"] // world, k) * steps * calls_per_step / dt / 1e9
    sample = (f"each step = {calls_per_step} M=1 call(s) over rank 0's shard of the packed weight (1/{world} of the layer, "
              f"{algorithmic_bytes(1, C3['n'] // world, k) / 1e6:.0f} MB), {oracle.threads()} OpenMP threads, {dt:.1f} s in all")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own CPU route is Vulkan on a software renderer, unavailable on this box; this is the CPU port of its shader arithmetic (oracle/oracle.c)",
    }))


def workload_config(n_gpus: int) -> dict:
    r = replicas_for(n_gpus)
    how = "the whole layer on one GPU" if n_gpus == 1 else (
        f"column-sharded over {n_gpus} GPUs ({C3['n'] // n_gpus} output features per rank), every call ends with the full y on "
        f"every rank: GEMV and gather in one kernel (value-and-step words stored to every peer from the epilogue)")
    return {"workload": f"C3: int4 group-{GROUP} decode linear, x[1,{C3['k']}] . W[{C3['n']},{C3['k']}]^T, {how}; {r} weight copies per "
                        f"rank and step ({r * algorithmic_bytes(1, C3['n'] // n_gpus, C3['k']) / 1e6:.0f} MB per rank > 2 x L2, so "
                        f"inputs larger than L2: no flush needed)",
            "m": 1, "n": C3["n"], "k": C3["k"], "group_size": GROUP, "replicas": r,
            "launch": f"one CUDA graph of {r} calls per step",
            "parallelism": "single GPU" if n_gpus == 1 else f"tp{n_gpus} column sharding + all-gather of y"}


def _stream_of(lib, ctx, local=None):
    import ctypes
    import torch
    sp = ctypes.c_void_p()
    from grilly2_b200 import _lib
    _lib.check(lib.gq_stream(ctx, ctypes.byref(sp)))
    if local is None:
        return torch.cuda.ExternalStream(sp.value)
    return torch.cuda.ExternalStream(sp.value, device=torch.device("cuda", local))


def measure_prefill(rows: int, steps: int, warmup: int, with_cublas: bool) -> dict:
    """Config 4: x float32 [rows, 4096] ~ N(0,1), W [14336, 4096] ~ N(0, 0.02) int8 per row; one step = one
    call of the tensor-core GEMM through GQ_KERNEL_AUTO: the exact integer kernel (tcgen05 kind::i8 against three
    int8 digit planes of x; two launches per call, the conversion of x included in the time). 2 M N K flops per
    step; the peak is the int8 tensor rate (twice the measured bf16 rate: 8192 multiply-adds per clock and SM in
    an instruction-rate loop) divided by the three planes. The library's tf32 kernel (GQ_KERNEL_TENSOR) and
    cuBLAS's own tf32 rate on the same shape with float32 weights are measured beside it, with the tf32 peak (half
    the measured bf16 rate). Median and best of five timed batches."""
    import torch
    from grilly2_b200 import _C, _lib
    m, n, k = rows, C2["n"], C2["k"]
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((n, k)) * SIGMA).astype(np.float32)
    x_np = rng.standard_normal((m, k)).astype(np.float32)
    wt = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    x = _C.Tensor.from_numpy(x_np)
    lib, ctx = _lib.load(), _C.context()
    stream = _stream_of(lib, ctx)
    y = _C.Tensor.empty((m, n), "float32")
    per_batch = max(steps // 5, 1)

    def timed(kernel):
        for _ in range(max(warmup, 3)):
            wt.linear(x, None, kernel, out=y)
        _C.synchronize()
        out = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(per_batch):
                wt.linear(x, None, kernel, out=y)
            e1.record(stream)
            _C.synchronize()
            out.append(e0.elapsed_time(e1) / per_batch)
        return out

    times = timed(_lib.KERNEL_AUTO)
    ms = statistics.median(times)
    tflops = 2.0 * m * n * k / ms / 1e9
    tf32_kernel = 2.0 * m * n * k / statistics.median(timed(_lib.KERNEL_TENSOR)) / 1e9
    cublas = None
    if with_cublas:
        torch.backends.cuda.matmul.allow_tf32 = True
        a, b = torch.from_numpy(x_np).cuda(), torch.from_numpy(w).cuda()
        for _ in range(3):
            c = a @ b.t()
        torch.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0.record()
            c = a @ b.t()
            t1.record()
            torch.cuda.synchronize()
            best = min(best, t0.elapsed_time(t1))
        cublas = 2.0 * m * n * k / best / 1e9
        del a, b, c
        torch.cuda.empty_cache()
    try:
        bf16, src = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]), "measured"
    except Exception:
        bf16, src = 1590.0, "fallback"
    peak, kind = bf16 * 2 / 3, f"{src} bf16 x 2 (int8 rate) / 3 digit planes"
    return {"m": m, "n": n, "k": k, "ms_median": ms, "ms_best": min(times), "tflops_median": tflops,
            "tflops_best": 2.0 * m * n * k / min(times) / 1e9, "peak": peak, "peak_kind": kind, "frac": tflops / peak,
            "tf32_peak": bf16 / 2, "frac_of_tf32_peak": tflops / (bf16 / 2), "tf32_kernel_tflops_median": tf32_kernel,
            "cublas_tf32_same_shape_fp32_weights": cublas, "launches": 2 * 5 * per_batch}


def run_decode_rows(args) -> None:
    """Config 2 (int4 g128, 14336 x 4096) at `--rows` rows of x (1 to 16) through GQ_KERNEL_AUTO: 8 weight copies
    (264 MB > 2 x L2) in one CUDA graph per step. The workload of the tcgen05 decode kernel's ncu summary."""
    import torch
    from grilly2_b200 import _C, _lib
    m, n, k = max(1, min(args.rows, 16)), C2["n"], C2["k"]
    rng = np.random.default_rng(C2["seed"])
    base = _C.Int4Weight.quantize(_C.Tensor.from_numpy((rng.standard_normal((n, k)) * C2["sigma"]).astype(np.float32)), GROUP)
    ws = []
    for _ in range(8):
        q = _C.Tensor.empty(base.packed().shape, "int32", persistent=True)
        sc = _C.Tensor.empty(base.scale().shape, "float32", persistent=True)
        z = _C.Tensor.empty(base.zero().shape, "float32", persistent=True)
        q.copy_(base.packed()), sc.copy_(base.scale()), z.copy_(base.zero())
        ws.append(_C.Int4Weight(q, sc, z, base.shape, GROUP))
    x = _C.Tensor.from_numpy(rng.standard_normal((m, k)).astype(np.float32))
    lib, ctx = _lib.load(), _C.context()
    stream = _stream_of(lib, ctx)
    ws[0].linear(x)  # first sighting eagerly (the context's scratch may grow), the second is recorded
    _C.begin_capture()
    keep = [w.linear(x) for w in ws]
    graph = _C.end_capture()
    steps, warm = min(args.steps, 500), max(args.warmup, 3)
    for _ in range(warm):
        graph.replay()
    _C.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        graph.replay()
    e1.record(stream)
    _C.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (steps * len(ws))
    peak, kind = measured_peak()
    b = algorithmic_bytes(m, n, k)
    print(json.dumps({
        "metric": METRIC, "value": b / (us * 1e-6) / 1e9, "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": us * len(ws) / 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"C2: int4 group-128 decode linear, x[{m},{k}] . W[{n},{k}]^T, 8 weight copies per step (inputs larger than L2)",
                   "m": m, "n": n, "k": k, "group_size": GROUP},
        "roofline": {"bound": "hbm", "achieved": b / (us * 1e-6) / 1e9, "peak": peak, "unit": "GB/s", "frac": b / (us * 1e-6) / 1e9 / peak, "traffic": None,
                     "peak_kind": kind, "algorithmic_bytes_per_launch": b, "us_per_launch": us},
        "gpu_launches": steps * len(keep),
    }))


def run_prefill(args) -> None:
    r = measure_prefill(args.rows, min(args.steps, 200), args.warmup, not args.no_extras)
    m, n, k = r["m"], r["n"], r["k"]
    print(json.dumps({
        "metric": "int8_weight_only_prefill_gemm", "value": r["tflops_median"], "unit": "TFLOP/s", "n_gpus": 1, "steps": r["launches"] // 2,
        "warmup": max(args.warmup, 3), "ms_per_step": r["ms_median"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "i8 (x as three int8 digit planes of a 23-bit fixed point per row, int32 accumulation, exact)", "data": "synthetic",
        "config": {"workload": f"C4: int8 weight-only prefill GEMM, x[{m},{k}] . W[{n},{k}]^T, fp32 out (inputs "
                               f"{(m * k * 4 + n * k) / 1e6:.0f} MB + output {m * n * 4 / 1e6:.0f} MB per step)", "m": m, "n": n, "k": k},
        "roofline": {"bound": "tensor", "achieved": r["tflops_median"], "peak": r["peak"], "unit": "TFLOP/s", "frac": r["frac"], "traffic": None,
                     "peak_kind": r["peak_kind"], "kernel": "gemm_i8_q8_kernel (with x_planes_kernel ahead of it, inside the time)",
                     "flops_per_launch": 2.0 * m * n * k, "best_of_five_batches": r["tflops_best"], "tf32_peak": r["tf32_peak"],
                     "frac_of_tf32_peak": r["frac_of_tf32_peak"], "tf32_kernel_tflops_median": r["tf32_kernel_tflops_median"],
                     "cublas_tf32_same_shape_fp32_weights": r["cublas_tf32_same_shape_fp32_weights"]},
        "gpu_launches": r["launches"],
    }))


def measure_decode_step(steps: int, warmup: int, cpu_seconds: float) -> dict:
    """Config 5: one decode step of a random-init Qwen2.5-0.5B-architecture model, int8 weight-only on every
    linear, float32 KV cache of length 1024, batch 1, the whole step one CUDA graph. Every replay decodes at
    position 1023 over 1024 cached positions: the graph begins by copying the cursor back to 1023, so the work
    per step is constant. Weights + cache (about 520 MB) exceed L2, so successive steps are L2-cold for them."""
    import ctypes
    import torch
    from grilly2_b200 import _C, _lib
    from grilly2_b200.infer import llama
    cfg = llama.qwen25_05b(1024)
    model = llama.LlamaDecoder(cfg, llama.random_weights(cfg, seed=SEED))
    rng = np.random.default_rng(SEED)
    shape = (cfg.num_hidden_layers, cfg.num_key_value_heads, 1023, cfg.head_dim)
    model.cache.fill(rng.standard_normal(shape).astype(np.float32), rng.standard_normal(shape).astype(np.float32), 1023)
    lens0 = _C.Tensor.from_numpy(np.full(cfg.num_hidden_layers, 1023, dtype=np.int32), persistent=True)
    token = _C.Tensor.from_numpy(np.array([12345], dtype=np.int32), persistent=True)
    lib, ctx = _lib.load(), _C.context()
    stream = _stream_of(lib, ctx)

    def step():
        model.cache.lens.copy_(lens0)
        return model.step(token)

    step()  # eager once: first-use set-up happens outside the capture
    before = _C.submit_stats()["launches"]
    _C.begin_capture()
    logits, nxt = step()
    graph = _C.end_capture()
    launches = _C.submit_stats()["launches"] - before
    warm = max(warmup, 3)
    for _ in range(warm):
        graph.replay()
    _C.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        graph.replay()
    e1.record(stream)
    _C.synchronize()
    ms = e0.elapsed_time(e1) / steps
    first = int(nxt.numpy()[0])

    # end to end: the autoregressive loop a caller runs - token in from pinned host memory, next token out
    hp = ctypes.c_void_p()
    _lib.check(lib.gq_host_alloc(ctx, 8, ctypes.byref(hp)))
    tok_in = (ctypes.c_int32 * 2).from_address(hp.value)
    tok_in[0] = 12345

    def e2e_step():
        _lib.check(lib.gq_upload_async(ctx, token.storage.handle, 0, hp, 4))
        graph.replay()
        _lib.check(lib.gq_download_async(ctx, nxt.storage.handle, 0, hp.value + 4, 4))
        _C.synchronize()
        tok_in[0] = tok_in[1]

    e2e_steps = min(steps, 500)
    for _ in range(3):
        e2e_step()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    peak, peak_kind = measured_peak()
    nbytes = model.bytes_per_token()
    achieved = nbytes["total"] / (ms * 1e-3) / 1e9

    cpu = None
    if cpu_seconds > 0:
        import oracle
        oracle.set_threads(os.cpu_count() or 1)
        shapes = [(cfg.q_size + 2 * cfg.kv_size, cfg.hidden_size), (cfg.hidden_size, cfg.q_size),
                  (2 * cfg.intermediate_size, cfg.hidden_size), (cfg.hidden_size, cfg.intermediate_size)]
        packed = []
        for n, k in shapes + [(cfg.vocab_size, cfg.hidden_size)]:
            w = (np.random.default_rng(n + k).standard_normal((n, k)) * SIGMA).astype(np.float32)
            q, sc = oracle.quantize_q8(w)
            packed.append((np.random.default_rng(k).standard_normal((1, k)).astype(np.float32), q, sc, k))

        def cpu_token():
            for _ in range(cfg.num_hidden_layers):
                for x, q, sc, k in packed[:4]:
                    oracle.linear_q8(x, q, sc, None, k)
            x, q, sc, k = packed[4]
            oracle.linear_q8(x, q, sc, None, k)

        cpu_token()
        n_tok, t0 = 0, time.perf_counter()
        while True:
            cpu_token()
            n_tok += 1
            dt = time.perf_counter() - t0
            if dt >= cpu_seconds:
                break
        cpu = {"value": n_tok / dt, "unit": "tokens/s", "cores": oracle.threads(), "kind": "port",
               "sample": f"{n_tok} tokens in {dt:.1f} s; the 97 int8 linears of a step only (norms, rotary, attention over the "
                         f"cache and argmax left out: under 6 % of the step's bytes), one weight copy per shape reused across layers"}
    del graph
    return {"tokens_per_s": 1e3 / ms, "ms_per_step": ms, "launches_per_step": launches, "steps": steps, "warmup": warm,
            "e2e_tokens_per_s": e2e_steps / e2e_s, "e2e_steps": e2e_steps, "achieved_GBps": achieved, "peak": peak, "peak_kind": peak_kind,
            "frac_of_hbm": achieved / peak, "algorithmic_bytes_per_step": nbytes, "cpu": cpu, "first_greedy_token": first}


def run_decode_step(args) -> None:
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
    r = measure_decode_step(min(args.steps, 2000), args.warmup, args.cpu_seconds)
    clocks = sampler.stop()
    print(json.dumps({
        "metric": "decode_tokens_per_s", "value": r["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": r["steps"], "warmup": r["warmup"],
        "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C5: full decode step, Qwen2.5-0.5B architecture (24 layers, hidden 896, 14 q / 2 kv heads, head_dim 64, "
                               "inter 4864, vocab 151936 tied int8 lm_head), int8 weight-only linears, fp32 KV cache length 1024 "
                               "(position 1023 every step), batch 1, one CUDA graph per step; weights + cache exceed L2",
                   "published_reference_other_hardware": "168.4 tokens/s on one RX 6750 XT (docs/inference.md:840)"},
        "roofline": {"bound": "hbm", "achieved": r["achieved_GBps"], "peak": r["peak"], "unit": "GB/s", "frac": r["frac_of_hbm"], "traffic": None,
                     "peak_kind": r["peak_kind"], "kernel": f"whole step ({r['launches_per_step']} launches)",
                     "algorithmic_bytes_per_step": r["algorithmic_bytes_per_step"]},
        "cpu_baseline": r["cpu"],
        "e2e": {"value": r["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": r["launches_per_step"] * r["steps"], "launches_per_step": r["launches_per_step"], "clocks": clocks,
        "first_greedy_token": r["first_greedy_token"],
    }))


def traffic_of(kernel_key: str):
    """DRAM bytes per launch from the ncu capture summarised under profiles/ (a small JSON beside the summary)."""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json")))[kernel_key]
    except Exception:
        return None


def _quiet_stdout():
    """Libraries (NCCL's version banner) write to file descriptor 1; the contract is ONE JSON line on stdout.
    Point fd 1 at stderr for the run and hand back a file on the real stdout for the result line."""
    real = os.fdopen(os.dup(1), "w")
    sys.stdout.flush()
    os.dup2(2, 1)
    return real


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "decode_step", "decode_rows"],
                    help="decode: the headline int4 layer; prefill: the int8 tensor-core GEMM of config 4; decode_step: config 5; "
                         "decode_rows: config 2 at --rows rows of x (1 to 16)")
    ap.add_argument("--rows", type=int, default=2048, help="rows of x for --workload prefill (default 2048) and decode_rows (1 to 16)")
    args = ap.parse_args()
    global print
    _real = _quiet_stdout()
    _builtin_print = print

    def print(*a, **kw):  # noqa: A001 - every result line of this file goes to the real stdout
        kw.setdefault("file", _real)
        kw.setdefault("flush", True)
        _builtin_print(*a, **kw)

    if args.impl == "reference":
        run_reference(args)
        return
    if args.workload == "prefill":
        run_prefill(args)
        return
    if args.workload == "decode_rows":
        if int(os.environ.get("RANK", "0")) == 0:
            run_decode_rows(args)
        return
    if args.workload == "decode_step":
        if int(os.environ.get("RANK", "0")) == 0:
            run_decode_step(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("GQ_DEVICE", str(local))

    import ctypes

    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import grilly2_b200 as g  # noqa: F401
    from grilly2_b200 import _C, _lib

    lib, ctx = _lib.load(), _C.context()
    stream = _stream_of(lib, ctx, local)
    n, k = C3["n"], C3["k"]
    ns = n // world
    reps = replicas_for(world)
    steps, warm = args.steps, max(args.warmup, 3)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        _C.synchronize()

    def timed(graph, nsteps: int, nwarm: int) -> float:
        """Device milliseconds for `nsteps` replays, max over ranks."""
        for _ in range(nwarm):
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(nsteps):
            graph.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def replicate(base, count):
        out = []
        for _ in range(count):
            q = _C.Tensor.empty(base.packed().shape, "int32", persistent=True)
            s = _C.Tensor.empty(base.scale().shape, "float32", persistent=True)
            z = _C.Tensor.empty(base.zero().shape, "float32", persistent=True)
            q.copy_(base.packed()), s.copy_(base.scale()), z.copy_(base.zero())
            out.append(_C.Int4Weight(q, s, z, base.shape, GROUP))
        return out

    # this rank's rows of the layer, and R copies of them
    base = _C.Int4Weight.quantize(_C.Tensor.from_numpy(shard_weight(rank, world)), GROUP)
    weights = replicate(base, reps)
    peers = comm = None
    if world > 1:
        from grilly2_b200.sharded import Comm, PeerGather

        def exchange(obj):
            out = [None] * world
            dist.all_gather_object(out, obj)
            return out

        comm = Comm.from_torch_distributed()
        peers = {m: PeerGather(world, rank, m, n, exchange) for m in (1, 8, 16)}

    def capture(m: int, ws, variant: str, out_all=None):
        """One graph: x[m] through every weight of `ws`. variant: 'linear' (this rank's rows only), 'fused'
        (linear + gather in one kernel), 'nccl', 'peer' (linear, then that gather). out_all: a [len(ws), m, n]
        tensor whose rows receive the outputs (one contiguous buffer)."""
        x = _C.Tensor.from_numpy(c3_x(m))
        outs = [None if out_all is None else out_all.window_rows(i, 1).reshape((m, out_all.shape[-1])) for i in range(len(ws))]
        if variant != "fused":
            ws[0].linear(x)  # first sighting of the shape runs eagerly (the context's scratch may grow), the second is recorded
        _C.begin_capture()
        ys = []
        for wt, o in zip(ws, outs):
            if variant == "fused":
                ys.append(peers[m].linear_gather(wt, x, None, out=o))
                continue
            y = wt.linear(x, out=o if variant == "linear" else None)
            if variant == "nccl":
                y = comm.all_gather(y, out=o)
            elif variant == "peer":
                y = peers[m].gather(y, out=o)
            ys.append(y)
        return x, ys, _C.end_capture()

    headline_variant = "linear" if world == 1 else "fused"
    out_all = _C.Tensor.empty((reps, 1, n), "float32", persistent=True)
    x1, ys1, g1 = capture(1, weights, headline_variant, out_all)
    peak, peak_kind = measured_peak()
    sampler = ClockSampler(local)
    launches_before = _C.submit_stats()["graph_nodes_replayed"]
    if rank == 0:
        sampler.start()
    ms = timed(g1, steps, warm)
    clocks = sampler.stop() if rank == 0 else None
    gpu_launches = (_C.submit_stats()["graph_nodes_replayed"] - launches_before) - warm * reps
    per_call_us = ms * 1e3 / (steps * reps)
    layer_bytes = algorithmic_bytes(1, n, k)
    rank_bytes = algorithmic_bytes(1, ns, k) + (n - ns) * 4  # this rank's weights and x once, the whole y written here
    value = layer_bytes / (per_call_us * 1e-6) / 1e9
    achieved = rank_bytes / (per_call_us * 1e-6) / 1e9

    # end to end with host buffers: pinned x in, the R outputs (one contiguous buffer) out, waited for each step
    hx, hy = ctypes.c_void_p(), ctypes.c_void_p()
    y_bytes = reps * n * 4
    _lib.check(lib.gq_host_alloc(ctx, k * 4, ctypes.byref(hx)))
    _lib.check(lib.gq_host_alloc(ctx, y_bytes, ctypes.byref(hy)))
    ctypes.memmove(hx.value, c3_x(1).ctypes.data, k * 4)

    def e2e_step():
        _lib.check(lib.gq_upload_async(ctx, x1.storage.handle, 0, hx, k * 4))
        g1.replay()
        _lib.check(lib.gq_download_async(ctx, out_all.storage.handle, 0, hy, y_bytes))
        _C.synchronize()

    e2e_steps = min(steps, 500)
    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = layer_bytes * reps * e2e_steps / e2e_s / 1e9
    host_y = np.ctypeslib.as_array((ctypes.c_float * (reps * n)).from_address(hy.value)).reshape(reps, n)
    assert np.array_equal(host_y[0], host_y[-1]) and np.isfinite(host_y).all() and np.abs(host_y).max() > 0, "replicas disagree"

    extras = {"weight_only_GBps": (n * k // 2 + 2 * n * (k // GROUP) * 4) / (per_call_us * 1e-6) / 1e9,  # the reference's own convention
              "frac_of_nominal_8TBps": achieved / 8000.0, "us_per_call": per_call_us}
    steps2 = max(steps // 4, 10)

    def time_variant(m, variant, ws=None, nsteps=None):
        ws = weights if ws is None else ws
        _, ys, gm = capture(m, ws, variant)
        nsteps = nsteps or steps2
        us = timed(gm, nsteps, 3) * 1e3 / (nsteps * len(ws))
        del gm
        return us, ys

    if world > 1 and not args.no_extras:
        # The sharded layer's variants, per call, max over ranks; and, outside the timed region, each variant's y_full
        # against the same layer computed unsharded on this rank by the plain linear over every shard's rows (each
        # rank rebuilds all shards from their seeds), and on rank 0 against the CPU oracle at m = 1.
        full = _C.Int4Weight.cat([_C.Int4Weight.quantize(_C.Tensor.from_numpy(shard_weight(r, world)), GROUP) for r in range(world)])
        sh = {"world": world, "rows_per_rank": ns, "replicas": reps}
        for m in (1, 8, 16):
            want = full.linear(_C.Tensor.from_numpy(c3_x(m))).numpy()
            for variant in ("linear", "nccl", "peer", "fused"):
                us, ys = time_variant(m, variant)
                key = f"m{m}_{variant}"
                sh[key + "_us"] = us
                sh[key + "_layer_GBps"] = algorithmic_bytes(m, n, k) / (us * 1e-6) / 1e9
                if variant != "linear":
                    worst = max(float(np.abs(y.numpy() - want).max() / np.abs(want).max()) for y in (ys[0], ys[-1]))
                    if dist is not None:
                        t = torch.tensor([worst], device="cuda")
                        dist.all_reduce(t, op=dist.ReduceOp.MAX)
                        worst = float(t.item())
                    sh[key + "_parity_max_rel"] = worst
                del ys
            if m == 1 and rank == 0:
                import oracle
                oracle.set_threads(os.cpu_count() or 1)
                qs, ss, zs = zip(*[oracle.quantize_q4(shard_weight(r, world), GROUP) for r in range(world)])
                ref = oracle.linear_q4(c3_x(1), np.concatenate(qs), np.concatenate(ss), np.concatenate(zs), None, k, GROUP)
                sh["m1_unsharded_vs_cpu_oracle_max_rel"] = float(np.abs(want - ref).max() / np.abs(ref).max())
        del full
        extras["sharded_c3"] = sh

    if world == 1 and not args.no_extras:
        # C3 at more rows, one GPU
        for m in (8, 16):
            us, _ = time_variant(m, "linear")
            extras[f"c3_m{m}_us"] = us
            extras[f"c3_m{m}_GBps"] = algorithmic_bytes(m, n, k) / (us * 1e-6) / 1e9
            extras[f"c3_m{m}_frac_of_measured_hbm"] = extras[f"c3_m{m}_GBps"] / peak
            # the same through the warp-level ring kernel alone (passes of four rows): what AUTO ran before the tcgen05 kernel
            xr = _C.Tensor.from_numpy(c3_x(m))
            weights[0].linear(xr, None, _lib.KERNEL_RING)
            _C.begin_capture()
            keep = [wt.linear(xr, None, _lib.KERNEL_RING) for wt in weights]
            gr = _C.end_capture()
            extras[f"c3_m{m}_ring_passes_us"] = timed(gr, steps2, 3) * 1e3 / (steps2 * len(weights))
            del gr, keep
        us, _ = time_variant(1, "linear", [weights[0]] * reps)
        extras["c3_m1_l2_hot_us"] = us
        del weights[1:]
        # C2: int4 14336 x 4096, 16 weight copies (528 MB), m = 1, 4, 8, 16; L2-hot; the older kernels
        rng2 = np.random.default_rng(C2["seed"])
        x2 = rng2.standard_normal((16, C2["k"])).astype(np.float32)
        base2 = _C.Int4Weight.quantize(_C.Tensor.from_numpy((rng2.standard_normal((C2["n"], C2["k"])) * C2["sigma"]).astype(np.float32)), GROUP)
        ws2 = replicate(base2, 16)

        def c2_graph(m, ws, kernel=_lib.KERNEL_AUTO):
            xx = _C.Tensor.from_numpy(x2[:m])
            ws[0].linear(xx, None, kernel)  # first sighting eagerly, as above
            _C.begin_capture()
            keep = [w.linear(xx, None, kernel) for w in ws]
            return keep, _C.end_capture()

        for m in (1, 4, 8, 16):
            keep, gm = c2_graph(m, ws2)
            us = timed(gm, steps2, 3) * 1e3 / (steps2 * 16)
            b = algorithmic_bytes(m, C2["n"], C2["k"])
            extras[f"c2_m{m}_us"], extras[f"c2_m{m}_GBps"], extras[f"c2_m{m}_frac_of_measured_hbm"] = us, b / (us * 1e-6) / 1e9, b / (us * 1e-6) / 1e9 / peak
            del gm, keep
        keep, gm = c2_graph(1, [ws2[0]] * 16)
        extras["c2_m1_l2_hot_us"] = timed(gm, steps2, 3) * 1e3 / (steps2 * 16)
        del gm, keep
        keep, gm = c2_graph(16, ws2, _lib.KERNEL_RING)
        extras["c2_m16_ring_passes_us"] = timed(gm, max(steps2 // 4, 5), 3) * 1e3 / (max(steps2 // 4, 5) * 16)
        del gm, keep
        for label, kern in (("imma_streaming", _lib.KERNEL_IMMA), ("dp4a", _lib.KERNEL_DP4A), ("reference_order_float", _lib.KERNEL_GEMV)):
            keep, gm = c2_graph(1, ws2, kern)
            ns_ = max(steps2 // 4, 5)
            extras[f"c2_m1_{label}_kernel_us"] = timed(gm, ns_, 3) * 1e3 / (ns_ * 16)
            del gm, keep
        del ws2, base2
        # config 1: int8 per-row x[1,896] . W[4864,896]^T, 64 weight copies per graph (280 MB > L2) and one copy (L2-hot)
        rng1 = np.random.default_rng(0)
        x1c = _C.Tensor.from_numpy(rng1.standard_normal((1, 896)).astype(np.float32))
        w1 = _C.Int8Weight.quantize(_C.Tensor.from_numpy((rng1.standard_normal((4864, 896)) * SIGMA).astype(np.float32)))

        def copy8():
            q8 = _C.Tensor.empty(w1.packed().shape, "int32", persistent=True)
            s8 = _C.Tensor.empty(w1.scale().shape, "float32", persistent=True)
            q8.copy_(w1.packed()), s8.copy_(w1.scale())
            return _C.Int8Weight(q8, s8, w1.shape)

        c1_bytes = w1.nbytes + 4 * 896 + 4 * 4864
        for label, ws8 in (("c1_int8_4864x896_m1", [copy8() for _ in range(64)]), ("c1_int8_4864x896_m1_l2_hot", [w1] * 64)):
            _C.begin_capture()
            keep = [wt.linear(x1c) for wt in ws8]
            g8 = _C.end_capture()
            ns_ = max(steps2 // 4, 5)
            t = timed(g8, ns_, 3) * 1e3 / (ns_ * 64)
            extras[label + "_us"], extras[label + "_GBps"], extras[label + "_frac_of_measured_hbm"] = t, c1_bytes / (t * 1e-6) / 1e9, c1_bytes / (t * 1e-6) / 1e9 / peak
            del g8, keep, ws8
        # config 4 (prefill) and config 5 (decode step), measured in this same run
        extras["c4_prefill"] = {f"m{m}": measure_prefill(m, 50 if m < 8192 else 20, 3, m == 2048) for m in (256, 2048, 8192)}
        r5 = measure_decode_step(300, 5, 0.0)
        extras["c5_decode_step"] = {key: r5[key] for key in ("tokens_per_s", "ms_per_step", "launches_per_step", "e2e_tokens_per_s", "frac_of_hbm", "first_greedy_token")}

    if peers:
        barrier()
        for pg in peers.values():
            pg.close()
        comm.close()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and args.cpu_seconds > 0:
        gbps, calls, threads, dt = cpu_run(args.cpu_seconds)
        cpu = {"value": gbps, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{calls} M=1 calls over one copy of the packed weight in {dt:.1f} s ({calls / reps:.2f} GPU steps)"}

    kernel_name = "gemv_q4_ring_kernel<1 row of x, 4 groups per warp>" + ("" if world == 1 else " with the gather in its epilogue")
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(world),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": traffic_of("gemv_q4_ring_c3_m1") if world == 1 else None,
                     "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture summarised under profiles/ (dram_traffic.json)",
                     "peak_kind": peak_kind, "kernel": kernel_name,
                     "algorithmic_bytes_per_launch": rank_bytes, "us_per_launch": per_call_us},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": k * 4, "d2h_bytes_per_step": y_bytes,
                "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3},
        "gpu_launches": int(gpu_launches), "clocks": clocks, "extras": extras,
    }))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
