#!/usr/bin/env python
"""Benchmark of the quantized-linear decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (config.workload): the int4 group-128 decode linear of a Llama-8B MLP
up-projection — x float32 [1, 4096] ~ N(0, 1), W float32 [14336, 4096]
~ N(0, 0.02) quantized asymmetric uint4 per group of 128 — seeded synthetic
data standing in for a checkpoint. One STEP is one pass of x through R = 16
distinct device copies of the packed weight (528 MB, four times the 126 MB L2,
so every call streams its weight from HBM): 16 dequant-fused GEMV launches,
replayed as one CUDA graph the way a captured decode step runs.

metric / value : algorithmic GB/s = (packed weight + scales + zero points +
                 x + y bytes, each counted once) x launches / device time,
                 inputs resident in HBM, timed with CUDA events on the
                 launching stream, max over ranks. N ranks each stream their
                 own copies (weak scaling, no collective on the data path).
e2e            : the same pass through the public API with HOST buffers: per
                 step x is copied from pinned host memory, the graph replayed,
                 all R outputs copied back and waited for (host wall clock).
roofline       : achieved = algorithmic bytes per launch / average launch
                 duration over the timed region; peak = measured HBM copy
                 bandwidth from MEASURED_PEAKS.json (else the fallback 6650).
cpu_baseline   : the CPU oracle (a port of the reference's shader arithmetic)
                 timed on the host cores on a bounded sample of the workload.

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

N_OUT, K_IN, GROUP, SIGMA, SEED = 14336, 4096, 128, 0.02, 1
REPLICAS = 16
METRIC, UNIT = "int4_g128_decode_linear_algorithmic_bandwidth", "GB/s"


def algorithmic_bytes(m: int, n: int = N_OUT, k: int = K_IN, group: int = GROUP) -> int:
    words = -(-k // 32) * 4
    groups = -(-k // group)
    return n * words * 4 + 2 * n * groups * 4 + m * k * 4 + m * n * 4


def make_inputs(m: int):
    rng = np.random.default_rng(SEED)
    x = rng.standard_normal((16, K_IN)).astype(np.float32)[:m]
    w = (rng.standard_normal((N_OUT, K_IN)) * SIGMA).astype(np.float32)
    return x, w


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


def cpu_run(seconds: float, m: int = 1):
    """The oracle's int4 linear on the full weight, all host threads, repeated
    for about `seconds`: returns (GB/s, calls, threads)."""
    import oracle
    x, w = make_inputs(m)
    q, scale, zero = oracle.quantize_q4(w, GROUP)
    oracle.linear_q4(x, q, scale, zero, None, K_IN, GROUP)  # warm
    calls, t0 = 0, time.perf_counter()
    while True:
        oracle.linear_q4(x, q, scale, zero, None, K_IN, GROUP)
        calls += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return algorithmic_bytes(m) * calls / dt / 1e9, calls, oracle.threads(), dt


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    x, w = make_inputs(1)
    q, scale, zero = oracle.quantize_q4(w, GROUP)
    for _ in range(max(args.warmup, 1)):
        oracle.linear_q4(x, q, scale, zero, None, K_IN, GROUP)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear_q4(x, q, scale, zero, None, K_IN, GROUP)
    dt = time.perf_counter() - t0
    value = algorithmic_bytes(1) * args.steps / dt / 1e9
    sample = f"each step = one M=1 call over one copy of the packed weight (1/{REPLICAS} of a GPU step), {oracle.threads()} OpenMP threads"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(1),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own CPU route is Vulkan on a software renderer, unavailable on this box; this is the CPU port of its shader arithmetic (oracle/oracle.c)",
    }))


def run_prefill(args) -> None:
    """Config 4: x float32 [rows, 4096] ~ N(0,1), W [14336, 4096] ~ N(0, 0.02) int8 per row; one step = one
    call of the tensor-core GEMM. 2 M N K flops per step; the peak is half the measured bf16 rate (tf32 runs
    at half of bf16 on these tensor cores), with cuBLAS's own tf32 rate on the same shape measured beside it."""
    import ctypes
    import torch
    from grilly2_b200 import _C, _lib
    m, n, k = args.rows, N_OUT, K_IN
    rng = np.random.default_rng(3)
    w = (rng.standard_normal((n, k)) * SIGMA).astype(np.float32)
    x_np = rng.standard_normal((m, k)).astype(np.float32)
    wt = _C.Int8Weight.quantize(_C.Tensor.from_numpy(w))
    x = _C.Tensor.from_numpy(x_np)
    lib, ctx = _lib.load(), _C.context()
    sp = ctypes.c_void_p()
    _lib.check(lib.gq_stream(ctx, ctypes.byref(sp)))
    stream = torch.cuda.ExternalStream(sp.value)
    for _ in range(max(args.warmup, 3)):
        y = wt.linear(x, None, _lib.KERNEL_TENSOR)
    _C.synchronize()
    steps = min(args.steps, 200)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        y = wt.linear(x, None, _lib.KERNEL_TENSOR)
    e1.record(stream)
    _C.synchronize()
    ms = e0.elapsed_time(e1) / steps
    tflops = 2.0 * m * n * k / ms / 1e9
    cublas = None
    if not args.no_extras:
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
    try:
        peak, kind = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]) / 2, "measured bf16 / 2"
    except Exception:
        peak, kind = 1590.0 / 2, "fallback bf16 / 2"
    print(json.dumps({
        "metric": "int8_weight_only_prefill_gemm_tf32", "value": tflops, "unit": "TFLOP/s", "n_gpus": 1, "steps": steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "tf32", "data": "synthetic",
        "config": {"workload": f"C4: int8 weight-only prefill GEMM, x[{m},{k}] . W[{n},{k}]^T, fp32 out (inputs "
                               f"{(m * k * 4 + n * k) / 1e6:.0f} MB + output {m * n * 4 / 1e6:.0f} MB per step)", "m": m, "n": n, "k": k},
        "roofline": {"bound": "tensor", "achieved": tflops, "peak": peak, "unit": "TFLOP/s", "frac": tflops / peak, "traffic": None,
                     "peak_kind": kind, "kernel": "gemm_tf32_q8_kernel", "flops_per_launch": 2.0 * m * n * k,
                     "cublas_tf32_same_shape_fp32_weights": cublas},
        "gpu_launches": steps,
    }))


def run_decode_step(args) -> None:
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
    sp = ctypes.c_void_p()
    _lib.check(lib.gq_stream(ctx, ctypes.byref(sp)))
    stream = torch.cuda.ExternalStream(sp.value)

    def step():
        model.cache.lens.copy_(lens0)
        return model.step(token)

    step()  # eager once: first-use set-up happens outside the capture
    before = _C.submit_stats()["launches"]
    _C.begin_capture()
    logits, nxt = step()
    graph = _C.end_capture()
    launches = _C.submit_stats()["launches"] - before
    warm = max(args.warmup, 3)
    steps = min(args.steps, 2000)
    for _ in range(warm):
        graph.replay()
    _C.synchronize()
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))
    sampler.start()
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
    clocks = sampler.stop()
    peak, peak_kind = measured_peak()
    nbytes = model.bytes_per_token()
    achieved = nbytes["total"] / (ms * 1e-3) / 1e9

    cpu = None
    if args.cpu_seconds > 0:
        import oracle
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
            if dt >= args.cpu_seconds:
                break
        cpu = {"value": n_tok / dt, "unit": "tokens/s", "cores": oracle.threads(), "kind": "port",
               "sample": f"{n_tok} tokens in {dt:.1f} s; the 97 int8 linears of a step only (norms, rotary, attention over the "
                         f"cache and argmax left out: under 6 % of the step's bytes), one weight copy per shape reused across layers"}

    print(json.dumps({
        "metric": "decode_tokens_per_s", "value": 1e3 / ms, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warm,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C5: full decode step, Qwen2.5-0.5B architecture (24 layers, hidden 896, 14 q / 2 kv heads, head_dim 64, "
                               "inter 4864, vocab 151936 tied int8 lm_head), int8 weight-only linears, fp32 KV cache length 1024 "
                               "(position 1023 every step), batch 1, one CUDA graph per step; weights + cache exceed L2",
                   "published_reference_other_hardware": "168.4 tokens/s on one RX 6750 XT (docs/inference.md:840)"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None,
                     "peak_kind": peak_kind, "kernel": f"whole step ({launches} launches)", "algorithmic_bytes_per_step": nbytes},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
        "gpu_launches": launches * steps, "launches_per_step": launches, "clocks": clocks,
        "first_greedy_token": first,
    }))


def sharded_c3(world, rank, dist, timed_fn, capture_mod, lib):
    """Config 3: int4 g128 W[28672, 8192] column-sharded over `world` ranks, x[1, 8192] replicated. Times, per
    call, this rank's GEMV alone, GEMV + NCCL all-gather of y, GEMV + the put-and-signal peer gather, and the GEMV
    whose epilogue does the gather itself (CUDA graphs of 8 calls over distinct weight copies; max over ranks). Weights are seeded per rank: timing only."""
    from grilly2_b200.sharded import Comm, PeerGather
    _C = capture_mod
    n, k, reps = 28672, 8192, 8
    ns = n // world
    rng = np.random.default_rng(2000 + rank)
    w = (rng.standard_normal((ns, k)) * 0.015).astype(np.float32)
    base = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w), GROUP)
    del w

    def replica():
        q = _C.Tensor.empty(base.packed().shape, "int32", persistent=True)
        sc = _C.Tensor.empty(base.scale().shape, "float32", persistent=True)
        z = _C.Tensor.empty(base.zero().shape, "float32", persistent=True)
        q.copy_(base.packed()), sc.copy_(base.scale()), z.copy_(base.zero())
        return _C.Int4Weight(q, sc, z, base.shape, GROUP)

    ws = [replica() for _ in range(reps)]
    x = _C.Tensor.from_numpy(np.random.default_rng(2).standard_normal((1, k)).astype(np.float32))
    comm = Comm.from_torch_distributed()

    def exchange(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    peers = PeerGather(world, rank, 1, n, exchange)
    out = {"world": world, "rows_per_rank": ns, "bytes_per_rank": base.nbytes + 4 * k + 4 * ns}
    for name in ("gemv_only", "gemv_nccl_all_gather", "gemv_peer_gather", "gemv_fused_gather"):
        _C.begin_capture()
        for wt in ws:
            if name == "gemv_fused_gather":  # one kernel: the GEMV's epilogue stores into every rank's y_full and signals
                peers.linear_gather(wt, x)
                continue
            y = wt.linear(x)
            if name == "gemv_nccl_all_gather":
                comm.all_gather(y)
            elif name == "gemv_peer_gather":
                peers.gather(y)
        graph = _C.end_capture()
        us = timed_fn(graph, 200, 5) * 1e3 / (200 * reps)
        out[name + "_us"] = us
        out[name + "_GBps_per_rank"] = out["bytes_per_rank"] / (us * 1e-6) / 1e9
        del graph
    _C.synchronize()
    dist.barrier()
    peers.close()
    comm.close()
    return out


def workload_config(n_gpus: int) -> dict:
    return {"workload": f"C2: int4 group-{GROUP} decode linear, x[1,{K_IN}] . W[{N_OUT},{K_IN}]^T, {REPLICAS} weight copies per step "
                        f"({REPLICAS * algorithmic_bytes(1) / 1e6:.0f} MB > L2, so inputs larger than L2: no flush needed)",
            "m": 1, "n": N_OUT, "k": K_IN, "group_size": GROUP, "replicas": REPLICAS, "launch": "one CUDA graph of 16 GEMV nodes per step",
            "parallelism": f"{n_gpus} independent rank(s), each streaming its own weight copies"}


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
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "decode_step"],
                    help="decode: the headline int4 GEMV sweep; prefill: the int8 tf32 tensor-core GEMM of config 4")
    ap.add_argument("--rows", type=int, default=2048, help="rows of x for --workload prefill")
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
    if args.workload == "decode_step":
        if int(os.environ.get("RANK", "0")) == 0:
            run_decode_step(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("GQ_DEVICE", str(local))

    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    import grilly2_b200 as g  # noqa: F401
    from grilly2_b200 import _C, _lib
    import ctypes

    lib, ctx = _lib.load(), _C.context()
    sp = ctypes.c_void_p()
    _lib.check(lib.gq_stream(ctx, ctypes.byref(sp)))
    stream = torch.cuda.ExternalStream(sp.value, device=torch.device("cuda", local))

    x_np, w_np = make_inputs(16)
    base = _C.Int4Weight.quantize(_C.Tensor.from_numpy(w_np), GROUP)

    def replica():
        q = _C.Tensor.empty(base.packed().shape, "int32", persistent=True)
        s = _C.Tensor.empty(base.scale().shape, "float32", persistent=True)
        z = _C.Tensor.empty(base.zero().shape, "float32", persistent=True)
        q.copy_(base.packed()), s.copy_(base.scale()), z.copy_(base.zero())
        return _C.Int4Weight(q, s, z, base.shape, GROUP)

    weights = [replica() for _ in range(REPLICAS)]

    def capture(m: int, ws, kernel=_lib.KERNEL_AUTO):
        x = _C.Tensor.from_numpy(x_np[:m])
        _C.begin_capture()
        ys = [w.linear(x, None, kernel) for w in ws]
        return x, ys, _C.end_capture()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        _C.synchronize()

    def timed(graph, steps: int, warmup: int) -> float:
        """Device milliseconds for `steps` replays, max over ranks."""
        for _ in range(warmup):
            graph.replay()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            graph.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    peak, peak_kind = measured_peak()
    sampler = ClockSampler(local)
    x1, ys1, g1 = capture(1, weights)
    launches_before = _C.submit_stats()["graph_nodes_replayed"]
    if rank == 0:
        sampler.start()
    ms = timed(g1, args.steps, max(args.warmup, 3))
    clocks = sampler.stop() if rank == 0 else None
    gpu_launches = (_C.submit_stats()["graph_nodes_replayed"] - launches_before) - max(args.warmup, 3) * REPLICAS
    per_launch_us = ms * 1e3 / (args.steps * REPLICAS)
    bytes_launch = algorithmic_bytes(1)
    achieved = bytes_launch / (per_launch_us * 1e-6) / 1e9
    value = achieved * world

    # end to end with host buffers: pinned x in, every y out, waited for each step
    hx, hy = ctypes.c_void_p(), ctypes.c_void_p()
    y_bytes = N_OUT * 4
    _lib.check(lib.gq_host_alloc(ctx, K_IN * 4, ctypes.byref(hx)))
    _lib.check(lib.gq_host_alloc(ctx, REPLICAS * y_bytes, ctypes.byref(hy)))
    ctypes.memmove(hx.value, x_np[:1].ctypes.data, K_IN * 4)

    def e2e_step():
        _lib.check(lib.gq_upload_async(ctx, x1.storage.handle, 0, hx, K_IN * 4))
        g1.replay()
        for r, y in enumerate(ys1):
            _lib.check(lib.gq_download_async(ctx, y.storage.handle, 0, hy.value + r * y_bytes, y_bytes))
        _C.synchronize()

    e2e_steps = min(args.steps, 500)
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
    e2e_value = bytes_launch * REPLICAS * e2e_steps / e2e_s / 1e9 * world
    host_y = np.ctypeslib.as_array((ctypes.c_float * (REPLICAS * N_OUT)).from_address(hy.value)).reshape(REPLICAS, N_OUT)
    assert np.array_equal(host_y[0], host_y[-1]) and np.isfinite(host_y).all(), "replicas disagree"

    extras = {}
    if not args.no_extras:
        steps2 = max(args.steps // 4, 10)
        for m in (4, 16):
            _, _, gm = capture(m, weights)
            t = timed(gm, steps2, 3) * 1e3 / (steps2 * REPLICAS)
            extras[f"m{m}_us_per_launch"] = t
            extras[f"m{m}_GBps"] = algorithmic_bytes(m) / (t * 1e-6) / 1e9
            extras[f"m{m}_frac_of_measured_hbm"] = extras[f"m{m}_GBps"] / peak
        _, _, ghot = capture(1, [weights[0]] * REPLICAS)
        t = timed(ghot, steps2, 3) * 1e3 / (steps2 * REPLICAS)
        extras["m1_l2_hot_us_per_launch"] = t
        extras["m1_l2_hot_GBps"] = bytes_launch / (t * 1e-6) / 1e9
        _, _, gim = capture(1, weights, _lib.KERNEL_IMMA)
        t = timed(gim, max(steps2 // 4, 5), 3) * 1e3 / (max(steps2 // 4, 5) * REPLICAS)
        extras["m1_imma_streaming_kernel_us_per_launch"] = t
        _, _, g2 = capture(2, weights)
        t = timed(g2, steps2, 3) * 1e3 / (steps2 * REPLICAS)
        extras["m2_us_per_launch"] = t
        extras["m2_GBps"] = algorithmic_bytes(2) / (t * 1e-6) / 1e9
        _, _, gdp = capture(1, weights, _lib.KERNEL_DP4A)
        t = timed(gdp, max(steps2 // 4, 5), 3) * 1e3 / (max(steps2 // 4, 5) * REPLICAS)
        extras["m1_dp4a_kernel_us_per_launch"] = t
        _, _, gexact = capture(1, weights, _lib.KERNEL_GEMV)
        t = timed(gexact, max(steps2 // 4, 5), 3) * 1e3 / (max(steps2 // 4, 5) * REPLICAS)
        extras["m1_reference_order_float_kernel_us_per_launch"] = t
        extras["weight_only_GBps"] = base.nbytes / (per_launch_us * 1e-6) / 1e9  # the reference's own convention
        extras["frac_of_nominal_8TBps"] = achieved / 8000.0
        # config 1: int8 per-row x[1,896] . W[4864,896]^T, 64 weight copies per graph (280 MB > L2) and one copy (L2-hot)
        rng1 = np.random.default_rng(SEED + 1)
        w1 = _C.Int8Weight.quantize(_C.Tensor.from_numpy((rng1.standard_normal((4864, 896)) * SIGMA).astype(np.float32)))
        x1c = _C.Tensor.from_numpy(rng1.standard_normal((1, 896)).astype(np.float32))

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
            t = timed(g8, max(steps2 // 4, 5), 3) * 1e3 / (max(steps2 // 4, 5) * 64)
            extras[label + "_us_per_launch"] = t
            extras[label + "_GBps"] = c1_bytes / (t * 1e-6) / 1e9
            del g8, keep

    if world > 1 and not args.no_extras:
        extras["sharded_c3"] = sharded_c3(world, rank, dist, timed_fn=timed, capture_mod=_C, lib=_lib)

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    cpu = None
    if world == 1 and args.cpu_seconds > 0:
        gbps, calls, threads, dt = cpu_run(args.cpu_seconds)
        cpu = {"value": gbps, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": f"{calls} M=1 calls over one copy of the packed weight in {dt:.1f} s ({calls / REPLICAS:.2f} GPU steps)"}

    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(world),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": 33071872, "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch, ncu capture summarised in profiles/gemv_q4_ring_int4_m1_decode_c2.md", "peak_kind": peak_kind, "kernel": "gemv_q4_ring_kernel<1 row of x, 2 groups per warp>",
                     "algorithmic_bytes_per_launch": bytes_launch, "us_per_launch": per_launch_us},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": K_IN * 4, "d2h_bytes_per_step": REPLICAS * y_bytes,
                "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3},
        "gpu_launches": int(gpu_launches), "clocks": clocks, "extras": extras,
    }))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
