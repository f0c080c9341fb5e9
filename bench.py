#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path: Q4_K / Q6_K decode GEMV at 9B shapes, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Workload ("ffn9b_b1"): the feed-forward projections of a 9B-shaped decoder, per layer
  ffn_gate Q4_K 12288x4096, ffn_up Q4_K 12288x4096, ffn_down Q6_K 4096x12288, batch 1,
on seeded synthetic GGUF superblocks (cogni_ml_b200.synth) that stand in for the model file the
reference measures on.  One step = one pass over L layers (3L GEMV launches); the L layers are
distinct device buffers totalling far more than L2, so every launch streams its weights from HBM.

Printed JSON (one line, rank 0):
  value     weight GB/s with inputs resident in HBM (CUDA events on the launching stream)
  e2e       the same pass through the resident runner with HOST activations: pinned H2D of the
            step's inputs, the GEMVs, D2H of the step's result, every step
  roofline  the dominant kernel (Q4_K GEMV) against the measured copy bandwidth
  cpu_baseline  the CPU restatement of the reference's QuantMatmul timed on this host

N > 1: each rank holds the row shard [rank*N_out/G, (rank+1)*N_out/G) of every matrix of a model
G times wider per GPU (weak scaling: per-GPU bytes fixed), followed by the all-gather of the
row-sharded outputs over NCCL, as the multi-GPU split of the path prescribes.
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

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

HIDDEN, FFN = 4096, 12288
Q4_K, Q6_K = 12, 14
Q4K_BYTES = FFN * (HIDDEN // 256) * 144      # 28,311,552
Q6K_BYTES = HIDDEN * (FFN // 256) * 210      # 41,287,680


# dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture summarised in
# profiles/gemv_imma_q4k_q6k_ffn9b_b1.md (batch 1; traffic does not depend on the layer count)
NCU_TRAFFIC_BYTES = {"q4k_12288x4096_b1": 28_356_608 + 65_536, "q6k_4096x12288_b1": 41_368_576 + 65_536}


def algorithmic_bytes(weight_bytes: int, in_dim: int, out_dim: int, batch: int) -> int:
    """Weights once + activations in + outputs out, per GEMV launch."""
    return weight_bytes + batch * in_dim * 4 + batch * out_dim * 4


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled every 100 ms while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def cpu_baseline(seconds: float, threads: int):
    """Times the C restatement of QuantMatmul.matmul_add on one layer's three projections."""
    from cogni_ml_b200 import synth
    from oracle import loader as oracle
    gate = synth.make_weight(Q4_K, FFN, HIDDEN, seed=0, tensor_id=1)
    down = synth.make_weight(Q6_K, HIDDEN, FFN, seed=0, tensor_id=3)
    xh = synth.make_activation(1, HIDDEN, seed=0, tensor_id=10)
    xf = synth.make_activation(1, FFN, seed=0, tensor_id=11)
    zf, zh = np.zeros(FFN, np.float32), np.zeros(HIDDEN, np.float32)
    oracle.matmul_add(xh, 1, HIDDEN, gate, Q4_K, FFN, zf, threads=threads)  # warm
    t0, passes = time.perf_counter(), 0
    while True:
        oracle.matmul_add(xh, 1, HIDDEN, gate, Q4_K, FFN, zf, threads=threads)   # ffn_gate
        oracle.matmul_add(xh, 1, HIDDEN, gate, Q4_K, FFN, zf, threads=threads)   # ffn_up
        oracle.matmul_add(xf, 1, FFN, down, Q6_K, HIDDEN, zh, threads=threads)   # ffn_down
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    layer_bytes = 2 * Q4K_BYTES + Q6K_BYTES
    return {"value": passes * layer_bytes / dt / 1e9, "unit": "GB/s", "cores": threads,
            "kind": "port",
            "sample": f"{passes} passes of one layer (ffn_gate+ffn_up Q4_K 12288x4096, ffn_down "
                      f"Q6_K 4096x12288, batch 1) in {dt:.1f} s; C restatement of "
                      "QuantMatmul.matmul_add, f64 accumulate, OpenMP over output rows"}


def run_reference(args):
    """--impl reference: the reference's CPU QuantMatmul for the same workload.  The reference is
    Crystal and cannot be compiled in this image, so its line-for-line C restatement (oracle/) is
    what runs, on all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import loader as oracle
    threads = oracle.max_threads()
    per_step = max(1.0, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_baseline(per_step / 4, threads)
    vals = [cpu_baseline(per_step, threads) for _ in range(args.steps)]
    value = float(np.mean([v["value"] for v in vals]))
    layer_bytes = 2 * Q4K_BYTES + Q6K_BYTES
    base = dict(vals[-1], value=value)
    print(json.dumps({
        "impl": "reference", "metric": "q4k_q6k_gemv_weight_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": layer_bytes / value / 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic",
        "config": {"workload": "ffn9b_b1", "batch": 1, "sample": "one layer per pass, bounded time",
                   "note": "reference CPU QuantMatmul restated in C (Crystal toolchain absent)"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def measure_extras(dev, gate_h, down_h, peaks):
    """The path's other two kernels at their benchmark shapes (reported beside the headline):
    prefill dequant-fused GEMM (TFLOP/s) and the fused vocab-sized lm_head GEMV + top-1 (GB/s)."""
    import torch

    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth

    def timed(fn, reps, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    out = {"prefill": [], "lm_head": None, "swiglu_down": None, "ffn_block_fused": None,
           "batched_ffn": None}
    tf_burst, tf_sust = peaks.get("bf16_tflops"), peaks.get("bf16_tflops_sustained")
    for qtype, raw, n, k in ((Q4_K, gate_h, FFN, HIDDEN), (Q6_K, down_h, HIDDEN, FFN)):
        dw = DeviceQuantWeight.upload(QuantWeight(raw, qtype, n, k), dev)
        for m in (512, 4096):
            x = torch.randn(m, k, device=dev).bfloat16()
            y = torch.empty(m, n, dtype=torch.float32, device=dev)
            ms = timed(lambda: dw.gemm(x, out=y), 10)
            tf = 2.0 * m * n * k / ms / 1e9
            out["prefill"].append({"type": "Q4_K" if qtype == Q4_K else "Q6_K", "M": m, "N": n,
                                   "K": k, "ms": ms, "tflops": tf,
                                   "frac_of_measured_burst": tf / tf_burst if tf_burst else None,
                                   "frac_of_measured_sustained": tf / tf_sust if tf_sust else None})
        del dw
    # ffn_down with the SwiGLU product fused into its activation pass, against the product written
    # by a separate elementwise kernel and then the plain GEMV; four weight copies (165 MB) defeat L2
    downs = [DeviceQuantWeight.upload(QuantWeight(down_h, Q6_K, HIDDEN, FFN), dev) for _ in range(4)]
    gate_v = torch.from_numpy(synth.make_activation(1, FFN, seed=3, tensor_id=21)).to(dev)
    up_v = torch.from_numpy(synth.make_activation(1, FFN, seed=3, tensor_id=22)).to(dev)
    yv = torch.empty(1, HIDDEN, dtype=torch.float32, device=dev)
    prod = torch.empty_like(gate_v)

    def fused():
        for d in downs:
            d.gemv_swiglu(gate_v, up_v, out=yv)

    def separate():
        for d in downs:
            torch.mul(torch.nn.functional.silu(gate_v), up_v, out=prod)
            d.gemv(prod, out=yv)

    out["swiglu_down"] = {"kernel": "Q6_K 4096x12288 b1: y = W (silu(gate) * up)",
                          "fused_us": timed(fused, 20) * 1e3 / len(downs),
                          "separate_us": timed(separate, 20) * 1e3 / len(downs)}
    # a whole FFN block per layer in two launches: RMSNorm fused into ffn_gate + ffn_up, SwiGLU and
    # the residual add fused into ffn_down; four layers of weights (390 MB) defeat L2
    from cogni_ml_b200 import GemvMany
    gates = [DeviceQuantWeight.upload(QuantWeight(gate_h, Q4_K, FFN, HIDDEN), dev) for _ in range(8)]
    hidden = torch.from_numpy(synth.make_activation(1, HIDDEN, seed=5, tensor_id=31)).to(dev)
    hidden2 = torch.empty_like(hidden)
    norm_w = torch.ones(HIDDEN, dtype=torch.float32, device=dev)
    g_out = torch.empty(1, FFN, dtype=torch.float32, device=dev)
    u_out = torch.empty(1, FFN, dtype=torch.float32, device=dev)
    calls = [GemvMany([gates[2 * i], gates[2 * i + 1]], hidden, [g_out, u_out], norm_weight=norm_w)
             for i in range(4)]

    def ffn_blocks():
        for i in range(4):
            calls[i].run()
            downs[i].gemv_swiglu(g_out, u_out, out=hidden2, residual=hidden)

    out["ffn_block_fused"] = {"kernel": "per layer: RMSNorm + ffn_gate/ffn_up (1 launch), SwiGLU + ffn_down + residual (1 launch), b1",
                              "us_per_layer": timed(ffn_blocks, 20) * 1e3 / 4}
    # the same four layers replayed from a CUDA graph (as the headline is), against the unfused
    # sequence of the same work: RMSNorm kernel, dual GEMV, SwiGLU kernel, GEMV with residual
    xn = torch.empty_like(hidden)
    plain_calls = [GemvMany([gates[2 * i], gates[2 * i + 1]], xn, [g_out, u_out]) for i in range(4)]

    def ffn_blocks_unfused():
        for i in range(4):
            ms = hidden.pow(2).mean(dim=-1, keepdim=True)
            torch.mul(hidden * torch.rsqrt(ms + 1e-6), norm_w, out=xn)
            plain_calls[i].run()
            torch.mul(torch.nn.functional.silu(g_out), u_out, out=prod)
            downs[i].gemv(prod, out=hidden2, residual=hidden)

    for name, fn in (("us_per_layer_graph", ffn_blocks), ("us_per_layer_unfused_graph", ffn_blocks_unfused)):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            fn()
        out["ffn_block_fused"][name] = timed(graph.replay, 20) * 1e3 / 4
        del graph
    del plain_calls
    del calls
    # the speculative verifier's row batches: one layer's ffn_gate + ffn_up (one launch) and ffn_down
    # at batch 2 .. 16, weight bytes per second; four layers of weights (390 MB) defeat L2
    out["batched_ffn"] = []
    for batch in (2, 4, 8, 16):
        xb = torch.from_numpy(synth.make_activation(batch, HIDDEN, seed=6, tensor_id=41)).to(dev)
        hb = torch.from_numpy(synth.make_activation(batch, FFN, seed=6, tensor_id=42)).to(dev)
        gb = torch.empty(batch, FFN, dtype=torch.float32, device=dev)
        ub = torch.empty(batch, FFN, dtype=torch.float32, device=dev)
        yb = torch.empty(batch, HIDDEN, dtype=torch.float32, device=dev)
        bcalls = [GemvMany([gates[2 * i], gates[2 * i + 1]], xb, [gb, ub]) for i in range(4)]

        def gate_up():
            for c in bcalls:
                c.run()

        def down():
            for d in downs:
                d.gemv(hb, out=yb)

        us_gu = timed(gate_up, 20) * 1e3 / 4
        us_dn = timed(down, 20) * 1e3 / 4
        out["batched_ffn"].append({"batch": batch, "gate_up_q4k_us": us_gu,
                                   "gate_up_gbs": 2 * gates[0].nbytes / us_gu / 1e3,
                                   "down_q6k_us": us_dn, "down_gbs": downs[0].nbytes / us_dn / 1e3})
        del bcalls
    del downs, gates
    vocab, hid = 151936, 5120
    head = DeviceQuantWeight.upload(
        QuantWeight(synth.make_weight(Q6_K, vocab, hid, seed=7, tensor_id=9), Q6_K, vocab, hid), dev)
    xh = torch.from_numpy(synth.make_activation(1, hid, seed=7, tensor_id=12)).to(dev)
    ms = timed(lambda: head.gemv_top1(xh), 20)
    nbytes = head.nbytes + hid * 4 + 8
    hbm = peaks.get("hbm_gbs")
    out["lm_head"] = {"kernel": "Q6_K 151936x5120 GEMV + top-1, batch 1", "ms": ms,
                      "achieved_gbs": nbytes / ms / 1e6, "algorithmic_bytes": nbytes,
                      "frac_of_measured": nbytes / ms / 1e6 / hbm if hbm else None}
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    from cogni_ml_b200 import DeviceQuantWeight, GemvMany, QuantWeight, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if args.kernel_choice:
        from cogni_ml_b200 import lib
        lib.cogni_qmm_set_kernel_choice(args.kernel_choice)
    L, B = args.layers, args.batch
    # One layer's bytes are generated on the host (rank-keyed seed), then replicated into L distinct
    # device buffers: timing depends on addresses, not on contents.
    gate_h = synth.make_weight(Q4_K, FFN, HIDDEN, seed=rank, tensor_id=1)
    up_h = synth.make_weight(Q4_K, FFN, HIDDEN, seed=rank, tensor_id=2)
    down_h = synth.make_weight(Q6_K, HIDDEN, FFN, seed=rank, tensor_id=3)

    def ring(raw, qtype, out_dim, in_dim):
        first = DeviceQuantWeight.upload(QuantWeight(raw, qtype, out_dim, in_dim), dev)
        copies = [first] + [DeviceQuantWeight(first.raw.clone(), qtype, out_dim, in_dim)
                            for _ in range(L - 1)]
        torch.cuda.synchronize()
        for w in copies:
            w.resident = True   # bytes complete before any GEMV is enqueued
        return copies

    gates, ups, downs = (ring(gate_h, Q4_K, FFN, HIDDEN), ring(up_h, Q4_K, FFN, HIDDEN),
                         ring(down_h, Q6_K, HIDDEN, FFN))
    xh_host = torch.from_numpy(synth.make_activation(B, HIDDEN, seed=0, tensor_id=10)).pin_memory()
    xf_host = torch.from_numpy(synth.make_activation(B, FFN, seed=0, tensor_id=11)).pin_memory()
    xh, xf = xh_host.to(dev), xf_host.to(dev)
    # shard outputs land in slot `rank` of a [world, B, rows] gather buffer
    y_gate = torch.empty(world, B, FFN, dtype=torch.float32, device=dev)
    y_up = torch.empty(world, B, FFN, dtype=torch.float32, device=dev)
    y_down = torch.empty(world, B, HIDDEN, dtype=torch.float32, device=dev)
    out_host = [torch.empty(B, n, dtype=torch.float32).pin_memory() for n in (FFN, FFN, HIDDEN)]

    def gather(buf):
        if world > 1:
            dist.all_gather_into_tensor(buf.view(-1), buf[rank].reshape(-1))

    # ffn_gate and ffn_up of a layer read the same x: one qmatvec_many launch per layer, as the
    # reference's CPU path issues them (qwen35_cpu.cr:1883); ffn_down is its own launch.
    gate_up = [GemvMany([gates[l], ups[l]], xh, [y_gate[rank], y_up[rank]]) for l in range(L)]

    def launch_q4():
        for l in range(L):
            if args.separate:
                gates[l].gemv(xh, out=y_gate[rank])
                ups[l].gemv(xh, out=y_up[rank])
            else:
                gate_up[l].run()

    def launch_q6():
        for l in range(L):
            downs[l].gemv(xf, out=y_down[rank])

    if args.no_graph:
        run_q4, run_q6 = launch_q4, launch_q6
    else:
        # The 3L launches of a step are captured once into two CUDA graphs (one per kernel kind,
        # so an event can sit between them) and replayed: the host cost of 96 Python->C calls per
        # step would otherwise bound a step made of 4-7 us kernels.
        launch_q4()
        launch_q6()
        torch.cuda.synchronize()
        g4, g6 = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g4):
            launch_q4()
        with torch.cuda.graph(g6):
            launch_q6()
        run_q4, run_q6 = g4.replay, g6.replay

    def step(marks=None):
        run_q4()
        if marks is not None:
            marks[1].record()
        run_q6()
        if marks is not None:
            marks[2].record()
        gather(y_gate)
        gather(y_up)
        gather(y_down)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    sync_all()
    marks = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        for k in range(args.steps):
            marks[k][0].record()
            step(marks[k])
            marks[k][3].record()
        sync_all()
    total_ms = marks[0][0].elapsed_time(marks[-1][3])
    q4_ms = sum(m[0].elapsed_time(m[1]) for m in marks)
    q6_ms = sum(m[1].elapsed_time(m[2]) for m in marks)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    step_bytes = L * (2 * Q4K_BYTES + Q6K_BYTES)
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # end to end through the resident path with host activations
    def e2e_step():
        xh.copy_(xh_host, non_blocking=True)
        xf.copy_(xf_host, non_blocking=True)
        step()
        out_host[0].copy_(y_gate[rank], non_blocking=True)
        out_host[1].copy_(y_up[rank], non_blocking=True)
        out_host[2].copy_(y_down[rank], non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(args.warmup):
        e2e_step()
    sync_all()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        e2e_step()
    e1.record()
    sync_all()
    e2e_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9

    if rank == 0:
        peak, peak_src = measured_peak()
        q4_per_launch = 1 if args.separate else 2     # GEMVs per Q4_K launch
        q4_launch_ms = q4_ms / (args.steps * 2 * L) * q4_per_launch
        q6_launch_ms = q6_ms / (args.steps * L)
        q4_alg = q4_per_launch * Q4K_BYTES + B * HIDDEN * 4 + q4_per_launch * B * FFN * 4
        q6_alg = algorithmic_bytes(Q6K_BYTES, FFN, HIDDEN, B)
        q4_ach = q4_alg / (q4_launch_ms * 1e-3) / 1e9
        q6_ach = q6_alg / (q6_launch_ms * 1e-3) / 1e9
        line = {
            "metric": "q4k_q6k_gemv_weight_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "ffn9b_b1", "layers": L, "batch": B,
                       "launch": "eager" if args.no_graph else "cuda graph replay",
                       "per_layer": "ffn_gate+ffn_up Q4_K 12288x4096, ffn_down Q6_K 4096x12288",
                       "weight_bytes_per_step_per_gpu": step_bytes,
                       "l2": f"{L} distinct weight sets ({step_bytes / 1e9:.2f} GB) >> 126 MB L2",
                       "parallelism": "single GPU" if world == 1 else
                       f"row-sharded x{world}, weak (per-GPU rows fixed), all-gather of outputs"},
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": B * (HIDDEN + FFN) * 4,
                    "d2h_bytes_per_step": B * (2 * FFN + HIDDEN) * 4},
            "gpu_launches": args.steps * (3 if args.separate else 2) * L,
            "roofline": {"bound": "hbm",
                         "kernel": "Q4_K GEMV 12288x4096 b1" if args.separate else
                         "Q4_K GEMV 2 x 12288x4096 b1 (ffn_gate + ffn_up, one launch)",
                         "achieved": q4_ach,
                         "peak": peak, "unit": "GB/s", "frac": q4_ach / peak,
                         "traffic": q4_per_launch * NCU_TRAFFIC_BYTES["q4k_12288x4096_b1"] if B == 1 else None,
                         "peak_source": f"of {peak_src}", "us_per_launch": q4_launch_ms * 1e3,
                         "algorithmic_bytes": q4_alg, "frac_of_nominal_8tbs": q4_ach / 8000.0},
            "roofline_q6k": {"bound": "hbm", "kernel": "Q6_K GEMV 4096x12288 b1",
                             "achieved": q6_ach, "peak": peak, "unit": "GB/s",
                             "frac": q6_ach / peak, "us_per_launch": q6_launch_ms * 1e3,
                             "traffic": NCU_TRAFFIC_BYTES["q6k_4096x12288_b1"] if B == 1 else None,
                             "algorithmic_bytes": q6_alg, "frac_of_nominal_8tbs": q6_ach / 8000.0},
            "clocks": clocks.summary(),
        }
        if world == 1 and not args.no_extras:
            try:
                peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
            except Exception:
                peaks = {}
            del gates, ups, downs
            torch.cuda.empty_cache()
            line["extras"] = measure_extras(dev, gate_h, down_h, peaks)
        if world == 1 and not args.no_cpu:
            from oracle import loader as oracle
            line["cpu_baseline"] = cpu_baseline(args.cpu_seconds, oracle.max_threads())
            line["cpu_baseline_1thread"] = cpu_baseline(min(args.cpu_seconds, 5.0), 1)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the prefill-GEMM and lm_head side measurements")
    ap.add_argument("--kernel-choice", type=int, default=0,
                    help="diagnostics: passed to cogni_qmm_set_kernel_choice before the run")
    ap.add_argument("--separate", action="store_true",
                    help="launch ffn_gate and ffn_up separately instead of one qmatvec_many launch")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of graph replay")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
