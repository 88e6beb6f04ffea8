#!/usr/bin/env python3
"""Benchmark of the ternary contraction hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): the ternary GEMV sweep at LLaMA-3-8B projection shapes, batch 1
-- one "step" is one decode-style pass over all 32 layers x 7 projection matrices
(224 GEMVs, 1.85 GB of packed weights, every matrix distinct so the pass is cold in
L2).  Weights are seeded synthetic: W = 0.02*randn ternarised per 128 along K
(threshold 0.7*mean|w|), activations randn FP16.  The metric is algorithmic bytes
(masks + scales + activations + outputs) per second.

Prints ONE JSON line (rank 0).  `value` is timed with the inputs resident in HBM
(CUDA-graph replay, CUDA events); `e2e` repeats the measurement through the same
public API with the step's activations copied from pinned host memory and its
outputs copied back inside the timed region.  `roofline` times the dominant
kernel (the 14336x4096 gate/up GEMV) alone over distinct cold matrices.
`--impl reference` times the reference's scalar CPU matvec on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# (name, rows N, cols K) of one LLaMA-3-8B decoder layer's ternary projections
SHAPES_8B = [("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096), ("o", 4096, 4096),
             ("gate", 14336, 4096), ("up", 14336, 4096), ("down", 4096, 14336)]
LAYERS_8B = 32
METRIC = "ternary_gemv_hbm_throughput_llama3_8b_shapes_batch1"
UNIT = "GB/s"


def gemv_bytes(n: int, k: int, b: int = 1) -> int:
    """Algorithmic bytes of one GEMV: masks N*K/4 + scales N*K/64 + 2B(K+N)."""
    return n * k // 4 + n * k // 64 + 2 * b * (k + n)


LAYER_BYTES = sum(gemv_bytes(n, k) for _, n, k in SHAPES_8B)
STEP_BYTES = LAYER_BYTES * LAYERS_8B
# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of one [gate|up] launch
# (28672 x 4096), taken from an ncu capture of that launch on cold weights; the capture's
# command and figures are kept with the other profile summaries of this repository.
ROOF_TRAFFIC = 31235840


def measured_peak_hbm():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def measured_peak_bf16():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["bf16_tflops"])
    except Exception:
        return 1590.0


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
                for nme, v in zip(names, r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            except Exception:
                continue
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------
# CPU legs (the only place bench.py touches oracle/)
# --------------------------------------------------------------------------
def cpu_layer_sample(reps: int, threads: int):
    """Times the reference's scalar matvec over one 8B layer (7 GEMVs) on host
    cores.  Returns (GB/s of algorithmic bytes, kind, threads, description)."""
    from oracle import cpu
    from ternary_llm_b200 import pack
    kind = "reference" if cpu.have_ref() else "port"
    mats = []
    rng = np.random.default_rng(0)
    for i, (_, n, k) in enumerate(SHAPES_8B):
        nz, sg, sc = pack.random_ternary_weight(n, k, seed=1000 + i)
        x = rng.standard_normal(k).astype(np.float16).astype(np.float32)
        mats.append((nz, sg, sc.astype(np.float32), x))
    best = None
    for _ in range(max(1, reps)):
        t0 = time.perf_counter()
        for nz, sg, sc, x in mats:
            cpu.matvec_f32(nz, sg, sc, x, 128, threads=threads, use_ref=(kind == "reference"))
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    what = ("cpu_reference compiled from the reference's tests/test_ternary_gemv.cu, rows split over host threads"
            if kind == "reference" else "C restatement of the reference's cpu_reference (oracle/cpu_reference.c), OpenMP over rows")
    return LAYER_BYTES / best / 1e9, best, kind, what


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores: its scalar matvec
    over one layer of the arm's workload per step (8B shapes at N = 1, the 70B shapes of the
    tensor-parallel arm at N > 1).  Under torchrun only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    from oracle import cpu
    from ternary_llm_b200 import pack
    kind = "reference" if cpu.have_ref() else "port"
    if args.gpus > 1:
        shapes = [("q", 8192, 8192), ("k", 1024, 8192), ("v", 1024, 8192), ("o", 8192, 8192),
                  ("gate", 28672, 8192), ("up", 28672, 8192), ("down", 8192, 28672)]
        metric, n_layers = "ternary_gemv_hbm_throughput_llama70b_shapes_tp_batch1", 80
        workload = "LLaMA-70B-shape ternary projection stack, batch 1, CPU scalar matvec"
    else:
        shapes, metric, n_layers = SHAPES_8B, METRIC, LAYERS_8B
        workload = "llama3-8b projection shapes, batch 1, CPU scalar matvec"
    layer_bytes = sum(gemv_bytes(n, k) for _, n, k in shapes)
    mats = []
    rng = np.random.default_rng(0)
    for i, (_, n, k) in enumerate(shapes):
        nz, sg, sc = pack.random_ternary_weight(n, k, seed=1000 + i)
        mats.append((nz, sg, sc.astype(np.float32), rng.standard_normal(k).astype(np.float16).astype(np.float32)))

    def step():
        for nz, sg, sc, x in mats:
            cpu.matvec_f32(nz, sg, sc, x, 128, threads=threads, use_ref=(kind == "reference"))

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = layer_bytes / dt / 1e9
    sample = f"one layer (7 GEMVs, {layer_bytes / 1e6:.1f} MB of packed weights) per step = 1/{n_layers} of the GPU arm's step"
    print(json.dumps({
        "impl": "reference", "metric": metric, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# --------------------------------------------------------------------------
# GPU arm, N > 1: tensor-parallel LLaMA-70B-shape layer stack
# --------------------------------------------------------------------------
H70, Q70, KV70, I70, LAYERS_70B = 8192, 8192, 1024, 28672, 80
METRIC_TP = "ternary_gemv_hbm_throughput_llama70b_shapes_tp_batch1"


def tp_shapes(tp: int):
    """Per-rank (name, rows, cols) of one layer: q/k/v/gate/up are column-parallel
    (rows split), o/down are row-parallel (cols split on 128-aligned boundaries)."""
    assert Q70 % (64 * tp) == 0 and KV70 % (64 * tp) == 0 and I70 % (128 * tp) == 0 and H70 % (128 * tp) == 0
    return [("q", Q70 // tp, H70), ("k", KV70 // tp, H70), ("v", KV70 // tp, H70), ("o", H70, Q70 // tp),
            ("gate", I70 // tp, H70), ("up", I70 // tp, H70), ("down", H70, I70 // tp)]


def tp_parity(torch, dist, rank, world, dev, src, calls, row_parallel, n_rows=512):
    """Checks the row-parallel path (GEMV + all-reduce, whichever route is selected) on layer 0's
    o and down: every rank runs the call, the shards' sampled rows are gathered on rank 0, which
    compares the reduced FP16 result with the oracle's float64 sum over ranks and the bound
    2e-3 * sum|scale*t*x| (+ half an FP16 ulp).  Returns {"max_err_over_tol": ...} on rank 0."""
    out = {}
    worst = 0.0
    idx = torch.from_numpy(np.random.default_rng(5).choice(H70, n_rows, replace=False).astype(np.int64)).to(dev)
    for name, (w, x_local, y) in calls.items():
        row_parallel(w, x_local, y)
        torch.cuda.synchronize()
        nz, sg, sc = (t[idx].contiguous() for t in src[name])
        parts = []
        for t in (nz, sg, sc, x_local.contiguous()):
            buf = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
            dist.gather(t, buf, dst=0)
            parts.append(buf)
        if rank == 0:
            from oracle import oracle
            y64 = np.zeros(n_rows)
            bound = np.zeros(n_rows)
            for r in range(world):
                hnz = parts[0][r].cpu().numpy().view(np.uint32)
                hsg = parts[1][r].cpu().numpy().view(np.uint32)
                hsc = parts[2][r].cpu().numpy()
                hx = parts[3][r].cpu().numpy()
                y64 += oracle.ternary_matvec(hnz, hsg, hsc, hx, 128, np.float64).reshape(-1)
                bound += oracle.tolerance_bound(hnz, hsg, hsc, hx, 128, 2e-3).reshape(-1)
            got = y[idx].float().cpu().numpy().astype(np.float64)
            half_ulp = 0.5 * 2.0 ** (np.floor(np.log2(np.maximum(np.abs(y64), 2.0 ** -14))) - 10)
            ratio = float(np.max(np.abs(got - y64) / (bound + half_ulp)))
            out[name] = ratio
            worst = max(worst, ratio)
    if rank != 0:
        return None
    return {"max_err_over_tol": worst, "per_matrix": out, "rows_sampled": n_rows,
            "what": "layer 0 o and down: all-reduced FP16 result vs float64 oracle over the gathered shards"}


def ar_phase_table(rec, launches_per_step):
    """Median microseconds per phase of the fused all-reduce launches of the last traced step,
    for the o (odd launch numbers) and down (even) projections, from the library's time stamps."""
    if rec is None:
        return None
    rec = rec[rec[:, 5] > 0]
    if len(rec) == 0:
        return None
    last = rec[:, 5].max()
    rec = rec[rec[:, 5] > last - launches_per_step]
    out = {}
    for name, odd in (("o", 1), ("down", 0)):
        r = rec[(rec[:, 5] % 2) == odd].astype(np.float64)
        if len(r) == 0:
            continue
        d = np.diff(r[:, :5], axis=1) / 1e3
        out[name] = {"launches": int(len(r)),
                     "stream_order_wait": float(np.median(d[:, 0])),
                     "staging_and_tiles": float(np.median(d[:, 1])),
                     "partial_sums_to_peer_stores_issued": float(np.median(d[:, 2])),
                     "wait_for_all_ranks_and_sum": float(np.median(d[:, 3])),
                     "kernel_total": float(np.median((r[:, 4] - r[:, 0]) / 1e3))}
    out["note"] = "CTA 0 of each launch, GPU nanosecond timer; stream_order_wait overlaps the previous kernel of the stream"
    return out



def _log(rank, msg):
    if rank == 0 and os.environ.get("TLLM_BENCH_VERBOSE"):
        print(f"[bench {time.strftime('%H:%M:%S')}] {msg}", file=sys.stderr, flush=True)


def run_tp(args, torch, dist, tl, synth, rank, world, local, dev):
    """N > 1: the LLaMA-70B-shape layer stack (norms, q/k/v, RoPE + KV append, attention over a
    2048-token FP16 cache, o, SwiGLU, down) tensor-parallel over the ranks, one token per step.
    Headline: batch 1 with the all-reduce fused into the row-parallel GEMV.  Beside it: the same
    stack at batch 32 (library all-reduce) and the projections alone (the weight stream without
    attention and element-wise kernels)."""
    from ternary_llm_b200.tp_stack import StackConfig, TpLayerStack
    KV_LEN = 2048
    shapes = tp_shapes(world)
    n_layers = args.layers if args.layers > 0 else LAYERS_70B
    cfg = StackConfig(hidden=H70, n_heads=Q70 // 128, n_kv_heads=KV70 // 128, head_dim=128, intermediate=I70,
                      max_seq_len=KV_LEN)
    assert [(n, r, c) for n, r, c in cfg.shard_shapes(world)] == shapes
    full = [("q", Q70, H70), ("k", KV70, H70), ("v", KV70, H70), ("o", H70, Q70), ("gate", I70, H70),
            ("up", I70, H70), ("down", H70, I70)]
    weight_bytes = n_layers * sum(gemv_bytes(n, k) for _, n, k in full)
    kv_bytes = n_layers * 2 * KV70 * KV_LEN * 2                 # K and V of every layer, read once per token
    step_bytes = weight_bytes + kv_bytes
    parity_src = {}
    ones = torch.ones(H70, dtype=torch.float16, device=dev)

    def layer_sources():
        for li in range(n_layers):
            src = {"attn_norm": ones, "ffn_norm": ones}
            for mi, (name, n, k) in enumerate(shapes):
                src[name] = synth.random_ternary_weight(n, k, seed=1_000_000 * rank + 100 * li + mi, device=dev)
            if li == 0:
                parity_src.update({"o": src["o"], "down": src["down"]})     # this rank's shards, reference layout
            yield src

    _log(rank, f"generating {n_layers} layers of tp{world} shards")
    fused = args.allreduce == "fused"
    stack = TpLayerStack(cfg, layer_sources(), rank, world, dev, dist.group.WORLD, allreduce=args.allreduce, batch=1)
    gen = torch.Generator(device=dev).manual_seed(99)
    stack.k_cache.copy_(torch.randn(stack.k_cache.shape, generator=gen, device=dev, dtype=torch.float16))
    stack.v_cache.copy_(torch.randn(stack.v_cache.shape, generator=gen, device=dev, dtype=torch.float16))
    x_h = (torch.randn(1, H70, generator=gen, device=dev) * 0.5).half()   # the token's embedding (replicated)
    x_attn = torch.randn(Q70 // world, generator=gen, device=dev).half()  # inputs of the projections-only pass
    x_ffn = torch.randn(I70 // world, generator=gen, device=dev).half()
    yq, yk, yv, yo, yg, yu, yd = (stack.q[0], stack.k[0], stack.v[0], stack.yo[0], stack.g[0], stack.u[0], stack.yd[0])

    def row_parallel(w, x_local, y):
        stack._row(w, x_local, y)

    def projections_only():
        for (qkv, o, gu, down, _, _) in stack.layers:
            tl.ternary_gemv_packed_multi(qkv, x_h[0], [yq, yk, yv])     # column shards, one input
            row_parallel(o, x_attn, yo)
            tl.ternary_gemv_packed_multi(gu, x_h[0], [yg, yu])
            row_parallel(down, x_ffn, yd)

    def launch_step():
        stack.step(x_h, KV_LEN - 1)

    _log(rank, "weights ready; first eager step")
    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        launch_step()
        torch.cuda.synchronize()
        tl.check_device_errors()
        assert bool(torch.isfinite(stack.out).all()), "non-finite residual stream"
        # parity of the exchange, outside every timed region: layer 0's o and down through the
        # same row-parallel path, rank 0 compares sampled rows with the CPU oracle on the
        # gathered shards (sum over ranks of W_r x_r)
        parity = tp_parity(torch, dist, rank, world, dev, parity_src,
                           {"o": (stack.layers[0][1], x_attn, yo), "down": (stack.layers[0][3], x_ffn, yd)}, row_parallel)
        parity_src.clear()
        _log(rank, "eager step done; capturing")

        def capture(fn):
            if args.no_graph:
                return None, "eager launches (graph disabled)"
            try:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    fn()
                return g, "CUDA graph replay of the whole step"
            except Exception as e:      # capture of the collective is not available: launch eagerly
                torch.cuda.synchronize()
                return None, f"eager launches (graph capture failed: {type(e).__name__})"

        graph, mode = capture(launch_step)
        _log(rank, f"launch mode: {mode}")

        def step():
            if graph is not None:
                graph.replay()
            else:
                launch_step()

        def barrier():
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()

        def timed(fn, reps):
            barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                fn()
            b.record(stream)
            barrier()
            t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())

        sampler = ClockSampler(local)
        sampler.__enter__()          # samples from warm-up to the end of the timed regions
        for _ in range(max(args.warmup, 3)):
            step()
        t_load = time.perf_counter()
        n_extra = torch.zeros(1, dtype=torch.int32, device=dev)
        while True:                                   # keep the GPUs under load until clock samples exist
            step()
            torch.cuda.synchronize()
            n_extra[0] = 1 if time.perf_counter() - t_load < 0.5 else 0
            dist.all_reduce(n_extra, op=dist.ReduceOp.MAX)   # all ranks leave the loop together
            if int(n_extra.item()) == 0:
                break
        ms = timed(step, args.steps)
        # end to end: the step's input vector comes from pinned host memory and the
        # step's output vector goes back to it, inside the timed region
        x_host = x_h.cpu().pin_memory()
        y_host = torch.empty(1, H70, dtype=torch.float16).pin_memory()

        def step_e2e():
            x_h.copy_(x_host, non_blocking=True)
            step()
            y_host.copy_(stack.out, non_blocking=True)
        for _ in range(2):
            step_e2e()
        ms_e2e = timed(step_e2e, args.steps)
        sampler.__exit__(None, None, None)
        clocks = sampler.summary()
        launches = stack.launches_per_step

        # beside the headline: the projections alone, and the same stack at batch 32
        g_proj, _ = capture(projections_only)
        reps = max(3, args.steps // 4)
        (g_proj.replay if g_proj is not None else projections_only)()
        ms_proj = timed(g_proj.replay if g_proj is not None else projections_only, reps) / reps
        phases = None
        if fused and g_proj is not None:
            # where a fused all-reduce launch spends its time: a graph of the projections-only
            # pass captured with the library's time stamps switched on, outside the timed regions
            stack.ar.trace(4096)
            g2, _ = capture(projections_only)
            if g2 is not None:
                for _ in range(3):
                    g2.replay()
            barrier()
            phases = ar_phase_table(stack.ar.trace(0), 2 * n_layers)
            g2 = None
        g_proj = None
        batch32 = None
        try:
            B = 32
            s32 = TpLayerStack(cfg, None, rank, world, dev, dist.group.WORLD, allreduce="nccl", batch=B, weights_from=stack)
            s32.k_cache.copy_(torch.randn(s32.k_cache.shape, generator=gen, device=dev, dtype=torch.float16))
            s32.v_cache.copy_(torch.randn(s32.v_cache.shape, generator=gen, device=dev, dtype=torch.float16))
            x32 = (torch.randn(B, H70, generator=gen, device=dev) * 0.5).half()
            s32.step(x32, KV_LEN - 1)
            torch.cuda.synchronize()
            tl.check_device_errors()
            finite = bool(torch.isfinite(s32.out).all())
            g32, mode32 = capture(lambda: s32.step(x32, KV_LEN - 1))
            fn32 = g32.replay if g32 is not None else (lambda: s32.step(x32, KV_LEN - 1))
            fn32()
            ms32 = timed(fn32, reps) / reps
            batch32 = {"ms_per_step": ms32, "tok_per_s": B * 1000.0 / ms32, "allreduce": "NCCL, FP16 [32, 8192]",
                       "launch": mode32, "finite": finite,
                       "gemv_route": "tcgen05 GEMM kernel (more than 8 vectors)"}
            g32 = None
            s32 = None
        except Exception as e:          # reported, never fatal for the headline
            batch32 = {"failed": f"{type(e).__name__}: {e}"[:300]}
    tl.check_device_errors()
    if rank == 0:
        peak, peak_kind = measured_peak_hbm()
        value = step_bytes * args.steps / (ms * 1e-3) / 1e9
        per_gpu_bytes = n_layers * sum(gemv_bytes(n, k) for _, n, k in shapes)
        print(json.dumps({
            "metric": METRIC_TP, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": "s8 MMA (exact s32 group sums), f32 accumulate", "data": "synthetic",
            "config": {"workload": "LLaMA-70B-shape ternary layer stack (hidden 8192, 64 heads / 8 KV heads of 128, intermediate 28672, %d layers): one decode token at batch 1 through norms, q/k/v, RoPE + KV append, attention over a %d-token FP16 KV cache, o, SwiGLU, down" % (n_layers, KV_LEN),
                       "parallelism": f"tp{world}: q/k/v/gate/up column-sharded (heads and KV cache with them), o/down row-sharded, all-reduce of the 8192-vector after o and after down ({2 * n_layers} per step): " + ("fused into the row-parallel GEMV kernel (peer stores over NVLink, flags, local sum)" if fused else "NCCL"),
                       "kernel_launches_per_step_per_gpu": launches,
                       "bytes_per_step": step_bytes, "weight_bytes_per_step": weight_bytes, "kv_bytes_per_step": kv_bytes,
                       "l2": f"{per_gpu_bytes/1e9:.2f} GB of distinct weights per GPU per step (> 126 MB L2), no flush needed",
                       "launch": mode},
            "roofline": {"bound": "hbm", "achieved": value / world, "peak": peak, "unit": "GB/s",
                         "frac": value / world / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "whole sharded step per GPU (GEMVs with all-reduces, attention, norms)"},
            "e2e": {"value": step_bytes * args.steps / (ms_e2e * 1e-3) / 1e9, "unit": UNIT,
                    "h2d_bytes_per_step": 2 * H70 * world, "d2h_bytes_per_step": 2 * H70 * world,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": launches * args.steps, "clocks": clocks,
            "decode": {"batch1": {"ms_per_token": ms / args.steps, "tok_per_s": 1000.0 * args.steps / ms},
                       "batch32": batch32, "kv_len": KV_LEN},
            "projections_only": {"ms_per_step": ms_proj, "gbs": weight_bytes / (ms_proj * 1e-3) / 1e9,
                                 "kernel_launches_per_step_per_gpu": 4 * n_layers + (0 if fused else 2 * n_layers),
                                 "what": "the seven projections of every layer with their all-reduces, fixed inputs"},
            "parity": parity, "ar_phases_us": phases,
        }), flush=True)
    # Tearing down a process group whose collectives were captured in a CUDA graph can
    # block forever: drop the graph, drain the device, meet at a barrier, then leave
    # without the destructor path.
    graph = None
    torch.cuda.synchronize()
    dist.barrier()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)



# --------------------------------------------------------------------------
# Rows reported beside the headline (N = 1)
# --------------------------------------------------------------------------
class ColdTimer:
    """Times a CUDA graph with cold caches: a buffer larger than the 126 MB L2 is rewritten
    before every timed replay, and the median of the replays is reported."""

    def __init__(self, torch, dev, stream):
        self.torch, self.stream = torch, stream
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def median_ms(self, graph, reps=5, warm=2):
        torch = self.torch
        times = []
        for i in range(warm + reps):
            self.flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            graph.replay()
            e1.record(self.stream)
            torch.cuda.synchronize()
            if i >= warm:
                times.append(e0.elapsed_time(e1))
        return statistics.median(times)


def gemv_batch_rows(torch, tl, synth, prepared, dev, stream, cold):
    """Configuration "GEMV sweep at batch 1/4/16" shape by shape, and the single-GEMV
    configuration (8192 x 2048): each row is one launch per distinct matrix (32 of them) as a
    CUDA graph, weights cold.  Batch 16 runs on the tcgen05 kernel (the library's routing)."""
    rows = []
    per_layer = len(SHAPES_8B)
    cases = [("q", 0), ("k/v", 1), ("o", 3), ("gate/up", 4), ("down", 6)]
    mats = {name: [prepared[li * per_layer + mi] for li in range(LAYERS_8B)] for name, mi in cases}
    cfg0 = []
    for i in range(LAYERS_8B):
        nz, sg, sc = synth.random_ternary_weight(8192, 2048, seed=77_000 + i, device=dev)
        cfg0.append(tl.PreparedWeight(nz, sg, sc, 8192, 2048, register=False, keep_source=False))
    mats["single-GEMV configuration (1B up_proj)"] = cfg0
    for name, ws in mats.items():
        n, k = ws[0].rows, ws[0].cols
        for b in ((1,) if name.startswith("single") else (1, 4, 16)):
            x = torch.randn(b, k, device=dev).half()
            y = torch.zeros(b, n, dtype=torch.float16, device=dev)
            for w in ws[:2]:
                tl.ternary_gemv_packed(w, x, y, b)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for w in ws:
                    tl.ternary_gemv_packed(w, x, y, b)
            us = cold.median_ms(g) * 1e3 / len(ws)
            wbytes = n * k // 4 + n * k // 64
            rows.append({"shape": name, "N": n, "K": k, "batch": b, "us_per_launch": us,
                         "gbs_algorithmic": gemv_bytes(n, k, b) / us / 1e3, "gbs_weights": wbytes / us / 1e3,
                         "vs_batch1": None})
            del g
    for r in rows:
        base = [q for q in rows if q["shape"] == r["shape"] and q["batch"] == 1][0]
        r["vs_batch1"] = r["us_per_launch"] / base["us_per_launch"]
    return rows


def reference_cuda_rows(torch, layers, dev, cold, stream):
    """The reference's own CUDA kernels (its sources compiled unmodified for sm_100 into the
    checker library under oracle/_ref) on the SAME seeded weights and the same cold-cache
    harness: a reported baseline beside this library's kernels, never part of it."""
    try:
        from oracle import cpu
        if not cpu.have_ref():
            return {"unavailable": "oracle/_ref/libref.so is not built on this machine"}
        ref = cpu.ref()
    except Exception as e:      # pragma: no cover
        return {"unavailable": f"{type(e).__name__}: {e}"}
    st = stream.cuda_stream
    out = []
    for name, mi in (("q/o", 0), ("gate/up", 4), ("down", 6)):
        _, n, k = SHAPES_8B[mi]
        ws = [layers[li][mi] for li in range(8)]               # 8 distinct matrices, reference layout
        x = torch.randn(k, device=dev).half()
        xq = torch.randint(-127, 128, (k,), device=dev, dtype=torch.int8)
        y = torch.zeros(n, dtype=torch.float16, device=dev)
        m = 128
        a_act = torch.randn(m, k, device=dev).half()
        c_out = torch.zeros(m, n, dtype=torch.float16, device=dev)

        def gemv():
            for a, b, c in ws:
                ref.ref_ternary_gemv(a.data_ptr(), b.data_ptr(), c.data_ptr(), x.data_ptr(), y.data_ptr(), n, k, 128, st)

        def gemv_i8():
            for a, b, c in ws:
                ref.ref_ternary_gemv_int8(a.data_ptr(), b.data_ptr(), c.data_ptr(), xq.data_ptr(), 0.01, y.data_ptr(), n, k, 128, st)

        def gemm():
            a, b, c = ws[0]
            ref.ref_ternary_gemm(a_act.data_ptr(), a.data_ptr(), b.data_ptr(), c.data_ptr(), c_out.data_ptr(), m, n, k, 128, st)

        row = {"shape": name, "N": n, "K": k}
        for label, fn, launches in (("ternary_gemv", gemv, len(ws)), ("ternary_gemv_int8", gemv_i8, len(ws)), ("ternary_gemm_M128", gemm, 1)):
            fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                fn()
            us = cold.median_ms(g, reps=3, warm=1) * 1e3 / launches
            if label == "ternary_gemm_M128":
                row[label] = {"us": us, "tflops": 2.0 * m * n * k / us / 1e6}
            else:
                row[label] = {"us": us, "gbs": gemv_bytes(n, k) / us / 1e3}
        out.append(row)
    return {"kernels": "kernels/ternary_gemv.cu and kernels/ternary_gemm.cu of the reference, compiled unmodified for sm_100",
            "harness": "same seeded weights (reference layout), CUDA graph, L2 flushed before every timed replay, median of 3",
            "rows": out}


def tp70b_single_gpu(torch, tl, synth, dev, stream, n_layers=LAYERS_70B):
    """The workload of the N > 1 arm -- the LLaMA-70B-shape projection stack, batch 1 -- on ONE
    GPU (18.2 GB of packed weights), so that the 2/4/8-GPU lines have a one-GPU anchor of the
    same work."""
    full = [("q", Q70, H70), ("k", KV70, H70), ("v", KV70, H70), ("o", H70, Q70), ("gate", I70, H70),
            ("up", I70, H70), ("down", H70, I70)]
    layers = []
    for li in range(n_layers):
        src = []
        for mi, (_, n, k) in enumerate(full):
            nz, sg, sc = synth.random_ternary_weight(n, k, seed=5_000_000 + 100 * li + mi, device=dev)
            src.append((nz, sg, sc, n, k))
        mats = tl.prepare_group(src[0:3])
        mats.append(tl.PreparedWeight(*src[3], register=False, keep_source=False))
        mats += tl.prepare_group(src[4:6])
        mats.append(tl.PreparedWeight(*src[6], register=False, keep_source=False))
        del src
        layers.append(mats)
    x_h = torch.randn(H70, device=dev).half()
    x_q = torch.randn(Q70, device=dev).half()
    x_i = torch.randn(I70, device=dev).half()
    yq, yk, yv = (torch.zeros(n, dtype=torch.float16, device=dev) for n in (Q70, KV70, KV70))
    yo, yd = (torch.zeros(H70, dtype=torch.float16, device=dev) for _ in range(2))
    yg, yu = (torch.zeros(I70, dtype=torch.float16, device=dev) for _ in range(2))

    def step():
        for q, k, v, o, g, u, d in layers:
            tl.ternary_gemv_packed_multi([q, k, v], x_h, [yq, yk, yv])
            tl.ternary_gemv_packed(o, x_q, yo, 1)
            tl.ternary_gemv_packed_multi([g, u], x_h, [yg, yu])
            tl.ternary_gemv_packed(d, x_i, yd, 1)

    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=stream):
        step()
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record(stream)
    for _ in range(reps):
        g.replay()
    e1.record(stream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    step_bytes = n_layers * sum(gemv_bytes(n, k) for _, n, k in full)
    del g, layers
    return {"workload": "LLaMA-70B-shape ternary projection stack (%d layers), batch 1, one GPU, no all-reduce" % n_layers,
            "ms_per_step": ms, "gbs": step_bytes / (ms * 1e-3) / 1e9, "bytes_per_step": step_bytes,
            "kernel_launches_per_step": 4 * n_layers}


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    import ternary_llm_b200 as tl
    from ternary_llm_b200 import synth

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path in this library")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    tl.lib()   # fail loudly here if the shared library is missing
    if world > 1:
        return run_tp(args, torch, dist, tl, synth, rank, world, local, dev)

    # ---- weights: 32 layers x 7 distinct matrices, seeded, on the device ----
    # q,k,v and gate,up share their input vector: each group is packed back to back at load time
    # (tl.prepare_group) so that the fused entry point streams it as one matrix in one launch.
    layers, prepared = [], []
    for li in range(LAYERS_8B):
        mats = []
        for mi, (_, n, k) in enumerate(SHAPES_8B):
            nz, sg, sc = synth.random_ternary_weight(n, k, seed=10_000 * rank + 100 * li + mi, device=dev)
            mats.append((nz, sg, sc, n, k))
        # load-time repack; registering makes the reference-signature calls below use the packed copy
        pw = tl.prepare_group(mats[0:3], register=True)
        pw.append(tl.PreparedWeight(*mats[3], register=True))
        pw += tl.prepare_group(mats[4:6], register=True)
        pw.append(tl.PreparedWeight(*mats[6], register=True))
        prepared += pw
        layers.append([m[:3] for m in mats])

    # ---- activations and outputs: one contiguous device buffer each ----------
    x_off, y_off, xo, yo = [], [], 0, 0
    for _ in range(LAYERS_8B):
        for _, n, k in SHAPES_8B:
            x_off.append(xo)
            y_off.append(yo)
            xo += k
            yo += n
    gen = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn(xo, generator=gen).to(torch.float16).pin_memory()
    y_host = torch.empty(yo, dtype=torch.float16).pin_memory()
    x_dev = x_host.to(dev)
    y_dev = torch.zeros(yo, dtype=torch.float16, device=dev)

    # a second set of device buffers: the end-to-end loop overlaps the copies of one step with
    # the kernels of the next (ping-pong), as a serving loop would
    x_dev2 = torch.empty_like(x_dev)
    y_dev2 = torch.zeros_like(y_dev)
    y_host2 = torch.empty(yo, dtype=torch.float16).pin_memory()

    def launch_step(xbuf=None, ybuf=None):
        xbuf = x_dev if xbuf is None else xbuf
        ybuf = y_dev if ybuf is None else ybuf

        def xs(i, k):
            return xbuf[x_off[i]:x_off[i] + k]

        def ys(i, n):
            return ybuf[y_off[i]:y_off[i] + n]

        return _launch_step(xs, ys)

    def _launch_step(xs, ys):
        """One decode-style pass.  q/k/v read the same vector (as do gate/up), so they go
        through the fused entry point; o and down through the reference-signature call,
        which finds the prepared copy by the registered weight pointer."""
        i = 0
        for li in range(LAYERS_8B):
            pw = prepared[li * 7:(li + 1) * 7]
            tl.ternary_gemv_packed_multi(pw[0:3], xs(i, 4096), [ys(i + j, SHAPES_8B[j][1]) for j in range(3)])
            nz, sg, sc = layers[li][3]
            tl.ternary_gemv(nz, sg, sc, xs(i + 3, 4096), ys(i + 3, 4096), 4096, 4096)
            tl.ternary_gemv_packed_multi(pw[4:6], xs(i + 4, 4096), [ys(i + 4, 14336), ys(i + 5, 14336)])
            nz, sg, sc = layers[li][6]
            tl.ternary_gemv(nz, sg, sc, xs(i + 6, 14336), ys(i + 6, 4096), 4096, 14336)
            i += 7
        return i, 4 * LAYERS_8B      # GEMVs computed, kernels launched ([q|k|v]; o; [gate|up]; down)

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        gemvs_per_step, launches_per_step = launch_step()   # also warms caches / attributes before capture
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            launch_step()
        graph2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph2, stream=stream):
            launch_step(x_dev2, y_dev2)

        # roofline kernel: the dominant launch of the step, [gate|up] (28672 x 4096 as one matrix),
        # alone over the 32 distinct gate|up groups
        n_r, k_r = 2 * 14336, 4096
        rgraph = torch.cuda.CUDAGraph()
        xr = x_dev[:k_r]
        yr = [torch.zeros(14336, dtype=torch.float16, device=dev) for _ in range(2)]
        with torch.cuda.graph(rgraph, stream=stream):
            for li in range(LAYERS_8B):
                tl.ternary_gemv_packed_multi(prepared[li * 7 + 4:li * 7 + 6], xr, yr)
        roof_launches = LAYERS_8B
        # the same launch on ONE group over and over: the 31 MB stay in the 126 MB L2 (warm figure)
        wgraph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(wgraph, stream=stream):
            for _ in range(LAYERS_8B):
                tl.ternary_gemv_packed_multi(prepared[4:6], xr, yr)

        def barrier():
            torch.cuda.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        ev = lambda: torch.cuda.Event(enable_timing=True)

        # ---- device-resident timing -------------------------------------------
        sampler = ClockSampler(local)
        sampler.__enter__()          # samples from warm-up to the end of the timed regions
        t_load = time.perf_counter()
        for _ in range(args.warmup):
            graph.replay()
        while time.perf_counter() - t_load < 0.5:      # keep the GPU under load until samples exist
            graph.replay()
            torch.cuda.synchronize()
        barrier()
        e0, e1 = ev(), ev()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)

        # ---- end to end: pinned host -> device, run, device -> pinned host, every step ------------
        # Three streams and two buffer sets: while step i computes, the inputs of step i+1 are
        # copied in and the outputs of step i-1 are copied out.
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        bufs = [(x_dev, y_dev, y_host, graph), (x_dev2, y_dev2, y_host2, graph2)]
        plain = lambda: torch.cuda.Event()

        def e2e_loop(n):
            done_c = [None, None]      # kernels of the last step that used buffer set b
            done_o = [None, None]      # its outputs copied out
            for i in range(n):
                b = i & 1
                xb, yb, yh, g = bufs[b]
                if done_c[b] is not None:
                    s_in.wait_event(done_c[b])          # the step that read xb has finished
                with torch.cuda.stream(s_in):
                    xb.copy_(x_host, non_blocking=True)
                    ev_in = plain()
                    ev_in.record(s_in)
                stream.wait_event(ev_in)
                if done_o[b] is not None:
                    stream.wait_event(done_o[b])        # yb has been copied out
                g.replay()
                done_c[b] = plain()
                done_c[b].record(stream)
                s_out.wait_event(done_c[b])
                with torch.cuda.stream(s_out):
                    yh.copy_(yb, non_blocking=True)
                    done_o[b] = plain()
                    done_o[b].record(s_out)

        e2e_loop(max(2, args.warmup // 2))
        barrier()
        f0, f1 = ev(), ev()
        f0.record(s_in)
        e2e_loop(args.steps)
        stream.wait_stream(s_out)
        f1.record(stream)
        barrier()
        ms_e2e = f0.elapsed_time(f1)

        # ---- dominant kernel alone ----------------------------------------------
        for _ in range(3):
            rgraph.replay()
        barrier()
        r0, r1 = ev(), ev()
        reps = 5
        r0.record(stream)
        for _ in range(reps):
            rgraph.replay()
        r1.record(stream)
        barrier()
        ms_roof = r0.elapsed_time(r1) / (reps * roof_launches)
        for _ in range(3):
            wgraph.replay()
        barrier()
        w0, w1 = ev(), ev()
        w0.record(stream)
        for _ in range(reps):
            wgraph.replay()
        w1.record(stream)
        barrier()
        ms_warm = w0.elapsed_time(w1) / (reps * roof_launches)
        # ---- prefill GEMM at the same shapes, M = 128, 512, 2048 (reported beside the headline):
        # 8 distinct matrices per timed pass, median of 5 passes, clock sampler still running ----
        gemm_rows = []
        for m_tok in (128, 512, 2048):          # the token counts of the benchmark definition's prefill configuration
            for name, mi in (("q/o", 0), ("k/v", 1), ("gate/up", 4), ("down", 6)):
                _, n, k = SHAPES_8B[mi]
                a_act = torch.randn(m_tok, k, device=dev).half()
                c_out = torch.empty(m_tok, n, dtype=torch.float16, device=dev)
                ws = [prepared[li * len(SHAPES_8B) + mi] for li in range(8)]     # 8 distinct matrices
                for w in ws[:3]:
                    tl.ternary_gemm_packed(a_act, w, c_out, m_tok)
                torch.cuda.synchronize()
                samples = []
                for _ in range(5):
                    g0, g1 = ev(), ev()
                    g0.record(stream)
                    for w in ws:
                        tl.ternary_gemm_packed(a_act, w, c_out, m_tok)
                    g1.record(stream)
                    torch.cuda.synchronize()
                    samples.append(g0.elapsed_time(g1) * 1e3 / len(ws))
                us = statistics.median(samples)
                gemm_rows.append({"shape": name, "M": m_tok, "N": n, "K": k, "us": us, "us_min": min(samples),
                                  "us_max": max(samples), "tflops": 2.0 * m_tok * n * k / us / 1e6})
                del a_act, c_out
        batch_rows = None if args.no_extras else gemv_batch_rows(torch, tl, synth, prepared, dev, stream, ColdTimer(torch, dev, stream))
        sampler.__exit__(None, None, None)
        clocks = sampler.summary()
        ref_cuda = None if (args.no_extras or world > 1) else reference_cuda_rows(torch, layers, dev, ColdTimer(torch, dev, stream), stream)

    t = torch.tensor([ms, ms_e2e, ms_roof], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_e2e, ms_roof = (float(v) for v in t.tolist())
    tl.check_device_errors()

    if rank == 0:
        peak, peak_kind = measured_peak_hbm()
        total_bytes = STEP_BYTES * world
        value = total_bytes * args.steps / (ms * 1e-3) / 1e9
        e2e = total_bytes * args.steps / (ms_e2e * 1e-3) / 1e9
        rb = gemv_bytes(n_r, k_r)
        achieved = rb / (ms_roof * 1e-3) / 1e9
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "s8 MMA (exact s32 group sums), f32 accumulate", "data": "synthetic",
            "config": {"workload": "ternary GEMV sweep, LLaMA-3-8B projection shapes (q,k,v,o,gate,up,down) x 32 layers, batch 1",
                       "gemv_per_step": gemvs_per_step, "kernel_launches_per_step": launches_per_step, "bytes_per_step": STEP_BYTES,
                       "l2": "1.85 GB of distinct weights per step (> 126 MB L2), no flush needed",
                       "launch": "CUDA graph replay of the whole step; q|k|v and gate|up are packed back to back at load time and each group is streamed as one matrix in one launch (they share the input vector); o and down one launch each (down, 14336 columns, as clusters of two CTAs that split the columns)",
                       "parallelism": "independent replicas per GPU" if world > 1 else "single GPU"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": ROOF_TRAFFIC, "peak_kind": peak_kind,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one launch from an ncu capture of the same launch on cold weights (a constant in this script, not measured by this run)",
                         "kernel": "gemv [gate|up] 28672x4096 batch 1 (gemv_packed_kernel<0>)", "bytes_per_launch": rb,
                         "us_per_launch": ms_roof * 1e3,
                         "warm_l2_us_per_launch": ms_warm * 1e3, "warm_l2_gbs": rb / (ms_warm * 1e-3) / 1e9,
                         "frac_of_nominal_8000": achieved / 8000.0},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel() * 2),
                    "d2h_bytes_per_step": int(y_host.numel() * 2), "ms_per_step": ms_e2e / args.steps,
                    "overlap": "copies of neighbouring steps overlap the kernels (two buffer sets, three streams)"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "prefill_gemm": {"kernel": "tcgen05 kind::f16, weights expanded to exact FP16 in tensor memory",
                             "peak_tflops": measured_peak_bf16(), "peak_kind": "measured bf16 cuBLAS burst",
                             "rows": gemm_rows},
        }
        if batch_rows is not None:
            out["gemv_batch"] = {"note": "one launch per distinct matrix (32), CUDA graph, L2 flushed before every timed replay, median of 5; "
                                         "batch <= 8 is the streaming GEMV (one or two vectors on 24-bit block fixed point; three and four vectors per weight pass on 16-bit block fixed point, within the 2e-3 bound for any input), batch 16 the tcgen05 kernel",
                                 "rows": batch_rows}
        if ref_cuda is not None:
            out["reference_cuda"] = ref_cuda
        if world == 1 and not args.no_decode:
            out["decode"] = decode_sample(torch, tl, dev)
        if world == 1 and not args.no_extras:
            # free the 8B sweep's weights first: the 70B stack needs 18 GB packed plus its sources in flight
            for w in prepared:
                w.release()
            prepared.clear()
            layers.clear()
            torch.cuda.empty_cache()
            with torch.cuda.stream(stream):
                out["tp70b_one_gpu"] = tp70b_single_gpu(torch, tl, synth, dev, stream)
            tl.check_device_errors()
        if world == 1 and not args.no_cpu:
            v, dt, kind, what = cpu_layer_sample(reps=3, threads=os.cpu_count() or 1)
            out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": kind,
                                   "sample": f"one layer (7 GEMVs, 57.9 MB) = 1/32 of a step, best of 3, {dt*1e3:.1f} ms; {what}"}
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


DECODE_ARCH_1B = dict(vocab_size=128256, hidden_dim=2048, intermediate_dim=8192, n_layers=16, n_heads=32, n_kv_heads=8,
                      head_dim=64, max_seq_len=1024, rope_theta=500000.0, rms_norm_eps=1e-5)


def decode_sample(torch, tl, dev, n_prompt=512, n_steps=128):
    """Decode tok/s of the library's decoder on the benchmark's 1B architecture (16 layers, hidden
    2048, 32/8 heads of 64, intermediate 8192, vocab 128256, FP16 embedding and lm_head) with seeded
    random weights drawn on the device: a 512-token prefill, then 128 greedy steps replayed as one
    CUDA graph per step (position, token and activation scales stay on the device).  Both
    arithmetic paths of a single-token step are reported: INT8 activations (what the reference
    engine runs) and FP16 activations (what the parity statement of the benchmark is written for)."""
    from ternary_llm_b200 import synth
    from ternary_llm_b200 import tllm_format as tf
    cfg = tf.TllmConfig(**DECODE_ARCH_1B)
    model = synth.random_device_model(cfg, 2026, dev)
    prompt = torch.from_numpy(np.random.default_rng(0).integers(0, cfg.vocab_size, n_prompt).astype(np.int32)).to(dev)
    layer_bytes = sum(gemv_bytes(o, i) for _, o, i in cfg.proj_shapes())
    step_bytes = layer_bytes * cfg.n_layers + cfg.vocab_size * cfg.hidden_dim * 2
    out = {"workload": "LLaMA-3.2-1B architecture, seeded random weights, 512-token prefill then 128 greedy steps, batch 1",
           "weight_bytes_per_token": step_bytes}
    for key, int8 in (("int8_activations", True), ("fp16_activations", False)):
        dec = tl.Decoder(model, int8_decode=int8)
        logits = dec.forward(prompt, 0)
        first = int(logits.float().argmax().item())
        dec.generate(first, n_prompt, 4)             # captures the step graph
        dec.reset()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dec.forward(prompt, 0)
        e1.record()
        torch.cuda.synchronize()
        _, ms = dec.generate(first, n_prompt, n_steps)
        tl.check_device_errors()
        dec.close()
        out[key] = {"prefill_ms": e0.elapsed_time(e1), "decode_ms_per_token": ms, "tok_per_s": 1e3 / ms,
                    "hbm_gbs": step_bytes / (ms * 1e-3) / 1e9}
    # the headline keys keep their meaning: the engine's own path (INT8 activations)
    out.update({"prefill_ms": out["int8_activations"]["prefill_ms"],
                "decode_ms_per_token": out["int8_activations"]["decode_ms_per_token"],
                "tok_per_s": out["int8_activations"]["tok_per_s"], "hbm_gbs": out["int8_activations"]["hbm_gbs"],
                "arithmetic": "tok_per_s is the INT8-activation path (the reference engine's choice for single-token steps); "
                              "fp16_activations is the same loop on FP16 activations; the prefill is FP16 + tcgen05 GEMM in both"})
    return out


def run_case(args):
    """A small single-kernel case for profilers: `gemv:NxK[:copies]`, `gemv_int8:NxK[:copies]`
    `gemm:MxNxK`, or `decode:ARCH[:prompt[:steps[:eager]]]` (the decoder on a random model).
    Distinct matrices are cycled so that the weights come from HBM."""
    import torch

    import ternary_llm_b200 as tl
    from ternary_llm_b200 import synth
    kind, dims, *rest = args.case.split(":")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if kind in ("gemv", "gemv_int8"):
        n, k = (int(v) for v in dims.split("x"))
        copies = int(rest[0]) if rest else 12
        ws = []
        for i in range(copies):
            nz, sg, sc = synth.random_ternary_weight(n, k, seed=i, device=dev)
            ws.append(tl.PreparedWeight(nz, sg, sc, n, k, register=False, keep_source=False))
        x = torch.randn(k, device=dev).half()
        xq = torch.randint(-127, 128, (k,), device=dev, dtype=torch.int8)
        y = torch.zeros(n, device=dev, dtype=torch.float16)
        for _ in range(2):
            for w in ws:
                if kind == "gemv":
                    tl.ternary_gemv_packed(w, x, y, 1)
                else:
                    tl.ternary_gemv_int8_packed(w, xq, 0.01, y)
    elif kind == "gemv_group":
        # gemv_group:N1+N2[+N3]xK[:copies] -- matrices packed back to back, one launch per group
        ns, k = dims.split("x")
        ns, k = [int(v) for v in ns.split("+")], int(k)
        copies = int(rest[0]) if rest else 6
        groups = []
        for c in range(copies):
            mats = []
            for i, n in enumerate(ns):
                nz, sg, sc = synth.random_ternary_weight(n, k, seed=10 * c + i, device=dev)
                mats.append((nz, sg, sc, n, k))
            groups.append(tl.prepare_group(mats))
        x = torch.randn(k, device=dev).half()
        ys = [torch.zeros(n, device=dev, dtype=torch.float16) for n in ns]
        for _ in range(2):
            for g in groups:
                tl.ternary_gemv_packed_multi(g, x, ys)
    elif kind == "gemm":
        m, n, k = (int(v) for v in dims.split("x"))
        nz, sg, sc = synth.random_ternary_weight(n, k, seed=0, device=dev)
        w = tl.PreparedWeight(nz, sg, sc, n, k, register=False, keep_source=False)
        a = torch.randn(m, k, device=dev).half()
        c = torch.zeros(m, n, device=dev, dtype=torch.float16)
        for _ in range(4):
            tl.ternary_gemm_packed(a, w, c, m)
    elif kind == "decode_batch":
        # decode_batch:1b|1b-4l:B[:prompt[:steps]] -- B sequences decoded in lock step (graph-replayed step)
        from ternary_llm_b200 import tllm_format as tf
        arch = dict(DECODE_ARCH_1B)
        if dims == "1b-4l":
            arch.update(n_layers=4, vocab_size=32000)
        bsz = int(rest[0]) if rest else 8
        n_prompt = int(rest[1]) if len(rest) > 1 else 512
        n_steps = int(rest[2]) if len(rest) > 2 else 32
        cfg = tf.TllmConfig(**arch)
        dec = tl.Decoder(tf.random_model(cfg, seed=2026), int8_decode=True, max_batch=bsz)
        rng = np.random.default_rng(0)
        for b in range(bsz):
            dec.forward_seq(b, torch.from_numpy(rng.integers(0, cfg.vocab_size, n_prompt).astype(np.int32)).to(dev), 0)
        toks = torch.from_numpy(rng.integers(0, cfg.vocab_size, bsz).astype(np.int32)).to(dev)
        dec.forward_batch(toks, n_prompt)
        torch.cuda.synchronize()
        stream = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(stream):
            graphs = []
            for i in range(n_steps):            # one graph per position (the position is a launch argument here)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    dec.forward_batch(toks, n_prompt + i)
                graphs.append(g)
            for g in graphs[:3]:
                g.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for g in graphs:
                g.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n_steps
        tl.check_device_errors()
        print(json.dumps({"case": args.case, "status": "ok", "batch": bsz, "ms_per_step": ms,
                          "tok_per_s_all_sequences": bsz * 1e3 / ms}))
        return
    elif kind == "decode":
        # decode:ARCH[:prompt[:steps[:eager]]] -- the library's decoder on a seeded random model of
        # the benchmark's 1B architecture (`1b`, 16 layers) or a 4-layer cut of it (`1b-4l`)
        from ternary_llm_b200 import tllm_format as tf
        arch = dict(DECODE_ARCH_1B)
        if dims == "1b-4l":
            arch.update(n_layers=4, vocab_size=32000)
        elif dims == "8b":      # LLaMA-3-8B architecture (the benchmark's GEMV shapes), weights drawn on the device
            arch.update(hidden_dim=4096, intermediate_dim=14336, n_layers=32, n_heads=32, n_kv_heads=8, head_dim=128)
        elif dims != "1b":
            raise SystemExit(f"unknown decode architecture {dims}")
        n_prompt = int(rest[0]) if len(rest) > 0 else 512
        n_steps = int(rest[1]) if len(rest) > 1 else 128
        eager = len(rest) > 2 and rest[2] == "eager"
        cfg = tf.TllmConfig(**arch)
        model = synth.random_device_model(cfg, 2026, dev) if dims == "8b" else tf.random_model(cfg, seed=2026)
        dec = tl.Decoder(model, int8_decode=True)
        del model
        prompt = torch.from_numpy(np.random.default_rng(0).integers(0, cfg.vocab_size, n_prompt).astype(np.int32)).to(dev)
        logits = dec.forward(prompt, 0)
        first = int(logits.float().argmax().item())
        info = {}
        if eager:
            tok = first
            for i in range(n_steps):
                lg = dec.forward(torch.tensor([tok], dtype=torch.int32, device=dev), n_prompt + i)
                tok = int(lg.float().argmax().item())
        else:
            dec.generate(first, n_prompt, min(4, n_steps))
            dec.reset()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            dec.forward(prompt, 0)
            e1.record()
            torch.cuda.synchronize()
            toks, ms = dec.generate(first, n_prompt, n_steps)
            info = {"prefill_ms": e0.elapsed_time(e1), "decode_ms_per_token": ms, "tok_per_s": 1e3 / ms}
        torch.cuda.synchronize()
        tl.check_device_errors()
        print(json.dumps({"case": args.case, "status": "ok", **info}))
        return
    else:
        raise SystemExit(f"unknown case {args.case}")
    torch.cuda.synchronize()
    tl.check_device_errors()
    print(json.dumps({"case": args.case, "status": "ok"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-decode", action="store_true", help="skip the decoder tok/s sample (N=1 only)")
    ap.add_argument("--no-extras", action="store_true",
                    help="N=1 only: skip the rows beside the headline (batch sweep, reference CUDA kernels, 70B stack on one GPU)")
    ap.add_argument("--layers", type=int, default=0, help="N>1 only: layer count override for quick checks (0 = the full 80)")
    ap.add_argument("--allreduce", default="fused", choices=["fused", "nccl"],
                    help="N>1 only: all-reduce fused into the row-parallel GEMV (default) or GEMV + NCCL")
    ap.add_argument("--no-graph", action="store_true", help="N>1 only: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--case", default="", help="run one small kernel case instead of the benchmark (for ncu): "
                    "gemv:NxK[:copies] | gemv_int8:NxK[:copies] | gemv_group:N1+N2xK[:copies] | gemm:MxNxK | decode:1b|1b-4l|8b[:prompt[:steps[:eager]]] | decode_batch:1b|1b-4l:B[:prompt[:steps]]")
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
