#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path: Q4_K / Q6_K decode GEMV at 9B shapes, batch 1.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L]

Workload ("ffn9b_b1"): the feed-forward projections of a 9B-shaped decoder, per layer
  ffn_gate Q4_K 12288x4096, ffn_up Q4_K 12288x4096, ffn_down Q6_K 4096x12288, batch 1,
on seeded synthetic GGUF superblocks (cogni_ml_b200.synth) that stand in for the model file the
reference measures on.  One step = one pass over L layers (2L launches: ffn_gate + ffn_up share x and
are one launch); the L layers are distinct device buffers totalling far more than L2, so every
launch streams its weights from HBM.

Printed JSON (one line on stdout, rank 0; the reference probes' key=value lines go to stderr):
  value     weight GB/s with inputs resident in HBM (CUDA events on the launching stream)
  e2e       the same pass with HOST activations: pinned H2D of the step's inputs, the GEMVs, D2H of
            the step's result, every step
  roofline  the kernel with the largest share of the step (Q6_K ffn_down) against the measured copy
            bandwidth; roofline_q4k the other one
  cpu_baseline  the CPU restatement of the reference's QuantMatmul timed on this host
  extras    the benchmark's other configurations (N = 1): every projection of the 9B layer at batch
            1 / 4 / 8 / 16, the 27B projections and lm_head, Q8_0, prefill GEMM, each beside the CPU
            port's time and, where the reference has a kernel for it, the reference's own PTX kernel
            on this GPU

N > 1 (weak scaling: per-GPU bytes fixed): every rank holds the row shard of a model N times wider.
Every projection's outputs are exchanged before the next projection starts, as a row-sharded decode
needs it: by default inside the GEMV launch (peer stores over NVLink plus per-rank flags,
cogni_qmm_gemv_many_exchange), with --exchange nccl by an all-gather after every launch.  What the
ranks compute is verified before it is timed (`sharded_check`): the gathered rows of every rank
against the CPU oracle and the vocabulary-sharded lm_head argmax of the 151936 x 5120 head.
`extras.sharded_27b` / `extras.prefill_sharded` are the strong-scaling configurations (fixed 27B
matrices split by rows, prefill with N-sharded weights plus all-gather).
"""
from __future__ import annotations

import argparse
import importlib.util
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
Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
TYPE_NAME = {8: "Q8_0", 12: "Q4_K", 13: "Q5_K", 14: "Q6_K", 20: "IQ4_NL"}
Q4K_BYTES = FFN * (HIDDEN // 256) * 144      # 28,311,552
Q6K_BYTES = HIDDEN * (FFN // 256) * 210      # 41,287,680
DTYPE = "f32 io / bfp15 x, s32 group sums, f32 accumulate"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each headline kernel, from one ncu
# capture of the 4-layer case (batch 1; the traffic of a launch does not depend on the layer count)
NCU_TRAFFIC_BYTES = {"q4k_2x12288x4096_b1": 2 * (28_356_608 + 65_536), "q6k_4096x12288_b1": 41_368_576 + 65_536}
TRAFFIC_SOURCE = "ncu, 4-layer case"


def log(line: str) -> None:
    """key=value lines in the style of the reference's probes (bin/cuda_q4k_gemv_probe.cr:272-289)."""
    print(line, file=sys.stderr, flush=True)


def host_threads() -> int:
    """Cores this process may run on; OMP_NUM_THREADS (torchrun sets it to 1) is not consulted."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def load_synth():
    """cogni_ml_b200/synth.py by path: numpy only, so the CPU legs never map the CUDA library."""
    spec = importlib.util.spec_from_file_location("_bench_synth", ROOT / "cogni_ml_b200" / "synth.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def algorithmic_bytes(weight_bytes: int, in_dim: int, out_dim: int, batch: int) -> int:
    """Weights once + activations in + outputs out, per GEMV launch."""
    return weight_bytes + batch * in_dim * 4 + batch * out_dim * 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return json.loads(p.read_text()), "measured"
        except Exception:
            pass
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


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


# ------------------------------------------------------------------------------ CPU legs
def cpu_baseline(seconds: float, threads: int):
    """Times the C restatement of QuantMatmul.matmul_add on one layer's three projections."""
    synth = load_synth()
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


def workload_config(layers: int, batch: int) -> dict:
    """The workload, identical for both arms (how an arm runs it is under `run`)."""
    step_bytes = layers * (2 * Q4K_BYTES + Q6K_BYTES)
    return {"workload": "ffn9b_b1", "layers": layers, "batch": batch,
            "per_layer": "ffn_gate+ffn_up Q4_K 12288x4096, ffn_down Q6_K 4096x12288",
            "weight_bytes_per_step_per_gpu": step_bytes,
            "l2": f"{layers} distinct weight sets ({step_bytes / 1e9:.2f} GB) >> 126 MB L2"}


def run_reference(args):
    """--impl reference: the reference's CPU QuantMatmul for the same workload.  The reference is
    Crystal and cannot be compiled in this image, so its line-for-line C restatement (oracle/) is
    what runs, on all the cores this process may use.  Each step is a bounded sample (whole passes
    over one layer's three projections); ms_per_step is the time a full step of `layers` layers
    takes at the sampled rate."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = host_threads()
    per_step = max(1.0, min(8.0, 120.0 / max(1, args.steps + args.warmup)))
    for _ in range(args.warmup):
        cpu_baseline(per_step / 4, threads)
    vals = [cpu_baseline(per_step, threads) for _ in range(args.steps)]
    value = float(np.mean([v["value"] for v in vals]))
    step_bytes = args.layers * (2 * Q4K_BYTES + Q6K_BYTES)
    base = dict(vals[-1], value=value)
    cfg = workload_config(args.layers, args.batch)
    print(json.dumps({
        "impl": "reference", "metric": "q4k_q6k_gemv_weight_gbs", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": step_bytes / value / 1e6, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": cfg,
        "run": {"launch": "cpu, bounded sample of whole layer passes per step", "threads": threads,
                "note": "reference CPU QuantMatmul restated in C (Crystal toolchain absent)"},
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------ GPU helpers
def timed(fn, reps, warm=3):
    import torch
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


_side_stream = None


def graphed(fn):
    """fn captured into a CUDA graph (after one eager run on a side stream; one side stream for
    the whole run: the engine keeps a workspace region per stream it has seen)."""
    import torch
    global _side_stream
    if _side_stream is None:
        _side_stream = torch.cuda.Stream()
    side = _side_stream
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        fn()
    return graph


def weight_ring(raw, qtype, out_dim, in_dim, dev, min_bytes=200e6, max_copies=16):
    """Distinct device copies of one weight, enough of them to exceed L2."""
    import torch

    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight
    n = int(max(2, min(max_copies, min_bytes // raw.nbytes + 1)))
    first = DeviceQuantWeight.upload(QuantWeight(raw, qtype, out_dim, in_dim), dev)
    ring = [first] + [DeviceQuantWeight(first.raw.clone(), qtype, out_dim, in_dim) for _ in range(n - 1)]
    torch.cuda.synchronize()
    for w in ring:
        w.resident = True
    return ring


def gemv_us(ring, x, batch):
    """us per GEMV launch over a ring of weight copies, replayed from a CUDA graph."""
    import torch
    y = torch.empty(batch, ring[0].out_dim, dtype=torch.float32, device=x.device)

    def go():
        for w in ring:
            w.gemv(x, out=y)
    g = graphed(go)
    reps = max(3, 600 // len(ring))
    return timed(g.replay, reps) * 1e3 / len(ring)


def reference_ptx_us(qtype, ring, x, batch, kind):
    """us per launch of the reference's own PTX GEMV (oracle/_ref cubins) on the same weights:
    `warp4` one token, `tbatch4` four tokens weight-stationary, `batched` grid over tokens.  A
    reported same-box baseline; None where the cubins are absent."""
    import torch
    try:
        from oracle import ref_kernels as ref
        if not ref.available():
            return None
    except Exception:
        return None
    out_dim, in_dim = ring[0].out_dim, ring[0].in_dim
    y = torch.empty(batch, out_dim, dtype=torch.float32, device=x.device)

    def go():
        for w in ring:
            if kind == "warp4":
                ref.gemv_warp4(qtype, w.raw.data_ptr(), x.data_ptr(), y.data_ptr(), in_dim, out_dim)
            elif kind == "tbatch4":
                for t in range(0, batch, 4):
                    ref.gemv_tbatch4(qtype, w.raw.data_ptr(), x.data_ptr() + 4 * t * in_dim,
                                     y.data_ptr() + 4 * t * out_dim, in_dim, out_dim)
            else:
                ref.gemv_batched(qtype, w.raw.data_ptr(), x.data_ptr(), y.data_ptr(), in_dim, out_dim, batch)
    torch.cuda.synchronize()
    for _ in range(2):
        go()
    ref.synchronize()
    # the reference launches on the null stream: time with events recorded on it
    null = torch.cuda.default_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = max(2, 100 // len(ring))
    with torch.cuda.stream(null):
        e0.record()
        for _ in range(reps):
            go()
        e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (reps * len(ring))


def config_rows(dev, peaks, cpu_threads):
    """One row per (projection, batch) of the benchmark's decode configurations: GPU us per launch
    (weights rotated through copies > L2), weight GB/s, the CPU port's time on the same bytes, and
    the reference's PTX kernel where it has one."""
    import torch

    from cogni_ml_b200 import synth
    from oracle import loader as oracle
    hbm = peaks["hbm_gbs"]
    shapes = [  # (config, name, type, out_dim, in_dim, batches)
        ("1", "q8_0_3584x1024", Q8_0, 3584, 1024, (1,)),
        ("3", "q_proj", Q4_K, 4096, 4096, (1, 4, 8, 16)),
        ("3", "k_proj", Q4_K, 1024, 4096, (1, 4, 8, 16)),
        ("3", "v_proj", Q4_K, 1024, 4096, (1, 4, 8, 16)),
        ("3", "o_proj", Q4_K, 4096, 4096, (1, 4, 8, 16)),
        ("2/3", "ffn_gate", Q4_K, 12288, 4096, (1, 4, 8, 16)),
        ("2/3", "ffn_down", Q6_K, 4096, 12288, (1, 4, 8, 16)),
        ("3", "q5k_variant", Q5_K, 4096, 4096, (1, 4, 8, 16)),
        ("5", "27b_ffn_gate", Q4_K, 17408, 5120, (1, 8)),
        ("5", "27b_ffn_down", Q6_K, 5120, 17408, (1, 8)),
    ]
    rows = []
    for cfg, name, qtype, out_dim, in_dim, batches in shapes:
        raw = synth.make_weight(qtype, out_dim, in_dim, seed=11, tensor_id=qtype)
        ring = weight_ring(raw, qtype, out_dim, in_dim, dev)
        for batch in batches:
            xh = synth.make_activation(batch, in_dim, seed=11, tensor_id=50 + batch)
            x = torch.from_numpy(xh).to(dev)
            us = gemv_us(ring, x, batch)
            t0 = time.perf_counter()
            oracle.matmul_add(xh, batch, in_dim, raw, qtype, out_dim, np.zeros(out_dim, np.float32),
                              threads=cpu_threads)
            cpu_ms = (time.perf_counter() - t0) * 1e3
            alg = algorithmic_bytes(raw.nbytes, in_dim, out_dim, batch)
            row = {"config": cfg, "name": name, "type": TYPE_NAME[qtype], "out_dim": out_dim,
                   "in_dim": in_dim, "batch": batch, "cuda_us": us, "weight_gbs": raw.nbytes / us / 1e3,
                   "hbm_frac_measured": alg / us / 1e3 / hbm, "hbm_frac_nominal": alg / us / 1e3 / 8000.0,
                   "cpu_ms": cpu_ms, "cpu_threads": cpu_threads}
            if name == "q8_0_3584x1024":
                row["note"] = "3.9 MB: L2- and launch-latency-bound, reported for parity not for roofline"
            if qtype != Q8_0 or batch == 1:
                kind = "warp4" if batch == 1 else "tbatch4"
                ref_us = reference_ptx_us(qtype, ring, x, batch, kind)
                if ref_us is not None:
                    row["reference_ptx_us"] = ref_us
                    row["reference_ptx_kernel"] = kind
            rows.append(row)
            log(f"config={cfg} tensor={name} type={TYPE_NAME[qtype]} out_dim={out_dim} in_dim={in_dim} "
                f"batch={batch} cuda_us={us:.2f} weight_gbs={raw.nbytes / us / 1e3:.0f} "
                f"hbm_frac_measured={row['hbm_frac_measured']:.3f} cpu_ms={cpu_ms:.2f} "
                f"cpu_threads={cpu_threads} nproc={os.cpu_count()} gpus=1"
                + (f" reference_ptx_us={row['reference_ptx_us']:.2f}" if "reference_ptx_us" in row else ""))
        del ring
        torch.cuda.empty_cache()
    return rows


def measure_extras(dev, gate_h, down_h, peaks, cpu_threads):
    """The path's other kernels at their benchmark shapes (reported beside the headline): prefill
    dequant-fused GEMM (TFLOP/s), the fused vocab-sized lm_head GEMV + top-1 (GB/s), the fused FFN
    block, the verifier's row batches."""
    import torch

    from cogni_ml_b200 import DeviceQuantWeight, GemvMany, QuantWeight, synth
    from oracle import loader as oracle

    out = {"prefill": [], "lm_head": None, "swiglu_down": None, "ffn_block_fused": None,
           "batched_ffn": None, "configs": None}
    tf_burst, tf_sust = peaks.get("bf16_tflops"), peaks.get("bf16_tflops_sustained")
    for qtype, raw, n, k in ((Q4_K, gate_h, FFN, HIDDEN), (Q6_K, down_h, HIDDEN, FFN)):
        dw = DeviceQuantWeight.upload(QuantWeight(raw, qtype, n, k), dev)
        # CPU time of the same GEMM, extrapolated from 4 token rows (the reference loops rows outermost)
        xs = synth.make_activation(4, k, seed=2, tensor_id=60)
        t0 = time.perf_counter()
        oracle.matmul_add(xs, 4, k, raw, qtype, n, np.zeros(n, np.float32), threads=cpu_threads)
        cpu_ms_per_row = (time.perf_counter() - t0) * 1e3 / 4
        for m in (512, 2048, 4096):
            x = torch.randn(m, k, device=dev).bfloat16()
            y = torch.empty(m, n, dtype=torch.float32, device=dev)
            ms = timed(lambda: dw.gemm(x, out=y), 10)
            tf = 2.0 * m * n * k / ms / 1e9
            out["prefill"].append({"type": TYPE_NAME[qtype], "M": m, "N": n, "K": k, "ms": ms, "tflops": tf,
                                   "frac_of_measured_burst": tf / tf_burst if tf_burst else None,
                                   "frac_of_measured_sustained": tf / tf_sust if tf_sust else None,
                                   "frac_of_nominal_2250": tf / 2250.0,
                                   "cpu_ms_extrapolated": cpu_ms_per_row * m, "cpu_threads": cpu_threads})
            log(f"config=4 prefill type={TYPE_NAME[qtype]} M={m} N={n} K={k} cuda_ms={ms:.3f} tflops={tf:.0f} "
                f"tc_frac_measured_burst={tf / tf_burst if tf_burst else 0:.3f} "
                f"cpu_ms_extrapolated={cpu_ms_per_row * m:.0f} cpu_threads={cpu_threads}")
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
        graph = graphed(fn)
        out["ffn_block_fused"][name] = timed(graph.replay, 20) * 1e3 / 4
        del graph
    del plain_calls
    del calls
    # the speculative verifier's row batches: one layer's ffn_gate + ffn_up (one launch) and ffn_down
    out["batched_ffn"] = []
    hbm = peaks["hbm_gbs"]
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
                                   "gate_up_frac_of_measured": 2 * gates[0].nbytes / us_gu / 1e3 / hbm,
                                   "down_q6k_us": us_dn, "down_gbs": downs[0].nbytes / us_dn / 1e3,
                                   "down_frac_of_measured": downs[0].nbytes / us_dn / 1e3 / hbm})
        del bcalls
    del downs, gates
    torch.cuda.empty_cache()
    out["configs"] = config_rows(dev, peaks, cpu_threads)
    vocab, hid = 151936, 5120
    head_h = synth.make_weight(Q6_K, vocab, hid, seed=7, tensor_id=9)
    head = DeviceQuantWeight.upload(QuantWeight(head_h, Q6_K, vocab, hid), dev)
    out["lm_head"] = []
    for batch in (1, 8):
        xhh = synth.make_activation(batch, hid, seed=7, tensor_id=12)
        xh = torch.from_numpy(xhh).to(dev)
        ms = timed(lambda: head.gemv_top1(xh), 20)
        nbytes = head.nbytes + batch * hid * 4 + 8 * batch
        t0 = time.perf_counter()
        logits = oracle.matmul_add(xhh, batch, hid, head_h, Q6_K, vocab, np.zeros(vocab, np.float32),
                                   threads=cpu_threads).reshape(batch, vocab)
        cpu_ms = (time.perf_counter() - t0) * 1e3
        idx, _ = head.gemv_top1(xh)
        same = all(int(idx[b]) == oracle.top1(logits[b])[0] for b in range(batch))
        row = {"kernel": f"Q6_K 151936x5120 GEMV + top-1, batch {batch}", "ms": ms,
               "achieved_gbs": nbytes / ms / 1e6, "algorithmic_bytes": nbytes,
               "frac_of_measured": nbytes / ms / 1e6 / hbm, "cpu_ms": cpu_ms, "cpu_threads": cpu_threads,
               "argmax_equals_cpu": same}
        if batch == 1:
            try:
                from oracle import ref_kernels as ref
                if ref.available():
                    width = (vocab + 3) // 4
                    pid = torch.zeros(width, dtype=torch.int32, device=dev)
                    pval = torch.zeros(width, dtype=torch.float32, device=dev)
                    tid = torch.zeros(1, dtype=torch.int32, device=dev)
                    tval = torch.zeros(1, dtype=torch.float32, device=dev)
                    torch.cuda.synchronize()

                    def ref_head():
                        ref.q6k_top1(head.raw.data_ptr(), xh.data_ptr(), pid.data_ptr(), pval.data_ptr(),
                                     tid.data_ptr(), tval.data_ptr(), hid, vocab)
                    ref_head()
                    ref.synchronize()
                    t0 = time.perf_counter()
                    for _ in range(5):
                        ref_head()
                    ref.synchronize()
                    row["reference_ptx_ms"] = (time.perf_counter() - t0) * 1e3 / 5
                    row["reference_ptx_argmax_equals_cpu"] = int(tid) == oracle.top1(logits[0])[0]
            except Exception as exc:  # the baseline leg must never take the bench down
                row["reference_ptx_error"] = str(exc)[:200]
        out["lm_head"].append(row)
        log(f"config=5 lm_head batch={batch} cuda_ms={ms:.4f} weight_gbs={head.nbytes / ms / 1e6:.0f} "
            f"hbm_frac_measured={row['frac_of_measured']:.3f} cpu_ms={cpu_ms:.1f} cpu_threads={cpu_threads} "
            f"argmax_equals_cpu={str(same).lower()}"
            + (f" reference_ptx_ms={row['reference_ptx_ms']:.3f}" if "reference_ptx_ms" in row else ""))
    return out


# ------------------------------------------------------------------------------ multi-GPU legs
def reduce_max(value: float, dev) -> float:
    import torch
    import torch.distributed as dist
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sharded_check(dev, world, rank, exchange, step_layer0, bufs, cpu_threads):
    """What the ranks compute, verified before it is timed.  (1) One layer's exchanged projections:
    every slot of the gather buffers on rank 0 against the CPU oracle on that rank's weights.
    (2) The 151936 x 5120 lm_head split by vocabulary rows: ShardedLmHead.top1 equal to the oracle's
    argmax over the concatenated shards, batch 1 and 8."""
    import torch
    import torch.distributed as dist

    from cogni_ml_b200 import QuantWeight, synth
    from cogni_ml_b200.sharded import ShardedLmHead
    from oracle import loader as oracle
    out = {}
    step_layer0()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    y_gate, y_up, y_down = (b.clone() for b in bufs)
    if rank == 0:
        worst = 0.0
        xh = synth.make_activation(1, HIDDEN, seed=0, tensor_id=10)
        xf = synth.make_activation(1, FFN, seed=0, tensor_id=11)
        for g in range(world):
            for tid, buf, qtype, n, k, x in ((1, y_gate, Q4_K, FFN, HIDDEN, xh), (2, y_up, Q4_K, FFN, HIDDEN, xh),
                                             (3, y_down, Q6_K, HIDDEN, FFN, xf)):
                raw = synth.make_weight(qtype, n, k, seed=g, tensor_id=tid)
                ref = oracle.matmul_add(x, 1, k, raw, qtype, n, np.zeros(n, np.float32), threads=cpu_threads)
                got = buf[g].cpu().numpy().ravel()
                worst = max(worst, float(np.abs(got - ref).max() / np.abs(ref).max()))
        out["gathered_rows_max_rel_err"] = worst
        out["gathered_rows_ok"] = worst <= 1e-3
    # vocabulary-sharded lm_head: rank g's shard is its own seeded tensor; the global head is their
    # concatenation (rank 0 regenerates every shard for the oracle)
    vocab, hid = 151936, 5120
    rows = vocab // world
    shard = synth.make_weight(Q6_K, rows, hid, seed=100 + rank, tensor_id=9)

    def local_factory(qw, r0, r1, device):
        from cogni_ml_b200 import DeviceQuantWeight
        dw = DeviceQuantWeight.upload(QuantWeight(shard, Q6_K, rows, hid), device)
        dw.row_begin = r0
        return dw

    head = ShardedLmHead(_HeadShape(rows * world, hid), dev, local_factory=local_factory)
    ok = True
    margins = []
    for batch in (1, 8):
        xhh = synth.make_activation(batch, hid, seed=7, tensor_id=12 + batch)
        idx, val = head.top1(torch.from_numpy(xhh).to(dev))
        torch.cuda.synchronize()
        if rank == 0:
            full = np.concatenate([synth.make_weight(Q6_K, rows, hid, seed=100 + g, tensor_id=9)
                                   for g in range(world)])
            logits = oracle.matmul_add(xhh, batch, hid, full, Q6_K, rows * world,
                                       np.zeros(rows * world, np.float32), threads=cpu_threads).reshape(batch, -1)
            for b in range(batch):
                ri, rv = oracle.top1(logits[b])
                ok = ok and int(idx[b]) == ri
                margins.append(float(rv) - float(np.partition(logits[b], -2)[-2]))
            del full
    if rank == 0:
        out["lm_head_sharded_argmax_equals_cpu"] = ok
        out["lm_head_min_top1_top2_margin"] = min(margins)
    dist.barrier()
    return out


class _HeadShape:
    """out_dim / in_dim / type of the sharded head for ShardedLmHead (the bytes live per rank)."""

    def __init__(self, out_dim, in_dim):
        self.out_dim, self.in_dim, self.type = out_dim, in_dim, Q6_K


def sharded_27b(dev, world, rank, exchange, peaks):
    """Config 5, strong scaling: the fixed 27B matrices split by rows over the ranks, batch 1 and 8.
    Per batch: kernel-only us of the shard GEMVs (no exchange); the decode chain ffn_gate + ffn_up
    (one launch) -> ffn_down with every launch exchanging its outputs inside the kernel and the
    next one reading the gathered (value, epoch) words; the same chain with an NCCL all-gather
    after each launch.  us per launch, max over ranks; aggregate weight GB/s of the whole box."""
    import torch
    import torch.distributed as dist

    from cogni_ml_b200 import CogniQmmError, GemvMany, synth
    from cogni_ml_b200.sharded import ExchangingGemv
    hid, ffn = 5120, 17408
    rows = []
    g_rows, d_rows = ffn // world, hid // world
    gate_raw = synth.make_weight(Q4_K, g_rows, hid, seed=rank, tensor_id=Q4_K)
    down_raw = synth.make_weight(Q6_K, d_rows, ffn, seed=rank, tensor_id=Q6_K)
    copies = int(max(2, min(24, 250e6 // (2 * gate_raw.nbytes + down_raw.nbytes) + 1)))
    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight
    g0 = DeviceQuantWeight.upload(QuantWeight(gate_raw, Q4_K, g_rows, hid), dev)
    d0 = DeviceQuantWeight.upload(QuantWeight(down_raw, Q6_K, d_rows, ffn), dev)
    gates = [g0] + [DeviceQuantWeight(g0.raw.clone(), Q4_K, g_rows, hid) for _ in range(copies - 1)]
    ups = [DeviceQuantWeight(g0.raw.clone(), Q4_K, g_rows, hid) for _ in range(copies)]
    downs = [d0] + [DeviceQuantWeight(d0.raw.clone(), Q6_K, d_rows, ffn) for _ in range(copies - 1)]
    torch.cuda.synchronize()
    for w in gates + ups + downs:
        w.resident = True
    layer_bytes = 2 * ffn * (hid // 256) * 144 + hid * (ffn // 256) * 210
    for batch in (1, 8):
        xh = torch.from_numpy(synth.make_activation(batch, hid, seed=1, tensor_id=70 + batch)).to(dev)
        xf = torch.from_numpy(synth.make_activation(batch, ffn, seed=1, tensor_id=80 + batch)).to(dev)
        yg = torch.empty(world, batch, g_rows, dtype=torch.float32, device=dev)
        yu = torch.empty_like(yg)
        yd = torch.empty(world, batch, d_rows, dtype=torch.float32, device=dev)
        plain_gu = [GemvMany([gates[i], ups[i]], xh, [yg[rank], yu[rank]]) for i in range(copies)]

        def kernel_only():
            for i in range(copies):
                plain_gu[i].run()
                downs[i].gemv(xf, out=yd[rank])
        us_kernel = timed(graphed(kernel_only).replay, 10) * 1e3 / (2 * copies)
        row = {"batch": batch, "layers_in_ring": copies,
               "per_layer": "ffn_gate+ffn_up Q4_K 17408x5120 (one launch), ffn_down Q6_K 5120x17408, rows / n_gpus per rank",
               "kernel_us_per_launch": reduce_max(us_kernel, dev) if world > 1 else us_kernel}
        best = row["kernel_us_per_launch"]
        if world > 1:
            bg = exchange.buffer(f"g27_{batch}", batch, ffn)
            bu = exchange.buffer(f"u27_{batch}", batch, ffn)
            bd = exchange.buffer(f"d27_{batch}", batch, hid)
            try:
                # the chain: gate/up read the gathered words of the previous down projection, down
                # reads the gathered words of gate (standing in for silu(gate) * up)
                fgu = [ExchangingGemv(exchange, [gates[i], ups[i]], bd, [bg, bu], True) for i in range(copies)]
                fdn = [ExchangingGemv(exchange, [downs[i]], bg, [bd], True) for i in range(copies)]
                ExchangingGemv(exchange, [downs[0]], xf, [bd], False).run()   # the first input of the chain

                def chain():
                    for i in range(copies):
                        fgu[i].run()
                        fdn[i].run()
                dist.barrier()
                us = timed(graphed(chain).replay, 10) * 1e3 / (2 * copies)
                row["chain_fused_exchange_us_per_launch"] = best = reduce_max(us, dev)
            except CogniQmmError as exc:   # same answer on every rank: the shape decides
                row["chain_fused_exchange_us_per_launch"] = None
                row["fused_exchange_note"] = f"not offered for this shape (status {exc.status})"

            def chain_nccl():
                for i in range(copies):
                    plain_gu[i].run()
                    dist.all_gather_into_tensor(yg.view(-1), yg[rank].reshape(-1))
                    dist.all_gather_into_tensor(yu.view(-1), yu[rank].reshape(-1))
                    downs[i].gemv(xf, out=yd[rank])
                    dist.all_gather_into_tensor(yd.view(-1), yd[rank].reshape(-1))
            dist.barrier()
            us = timed(chain_nccl, 5) * 1e3 / (2 * copies)
            row["chain_nccl_allgather_us_per_launch"] = reduce_max(us, dev)
            if row.get("chain_fused_exchange_us_per_launch") is None:
                best = row["chain_nccl_allgather_us_per_launch"]
        row["aggregate_weight_gbs"] = layer_bytes / (2 * best) / 1e3
        rows.append(row)
    return rows


def prefill_sharded(dev, world, rank, peaks):
    """Config 4 with N-sharded weights: each rank's GEMM over its [N / G] rows, then the all-gather
    of the [M, N / G] outputs (NCCL).  TFLOP/s aggregate, kernel only and with the all-gather."""
    import torch
    import torch.distributed as dist

    from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth
    rows = []
    for qtype, n, k in ((Q4_K, FFN, HIDDEN), (Q6_K, HIDDEN, FFN)):
        local = n // world
        raw = synth.make_weight(qtype, local, k, seed=rank, tensor_id=qtype)
        dw = DeviceQuantWeight.upload(QuantWeight(raw, qtype, local, k), dev)
        for m in (512, 2048, 4096):
            x = torch.randn(m, k, device=dev).bfloat16()
            gath = torch.empty(world, m, local, dtype=torch.float32, device=dev)
            ms_kernel = timed(lambda: dw.gemm(x, out=gath[rank]), 10)

            def with_gather():
                dw.gemm(x, out=gath[rank])
                if world > 1:
                    dist.all_gather_into_tensor(gath.view(-1), gath[rank].reshape(-1))
            if world > 1:
                dist.barrier()
            ms_total = timed(with_gather, 10)
            if world > 1:
                ms_kernel, ms_total = reduce_max(ms_kernel, dev), reduce_max(ms_total, dev)
            flops = 2.0 * m * n * k
            rows.append({"type": TYPE_NAME[qtype], "M": m, "N": n, "K": k, "n_gpus": world,
                         "kernel_ms": ms_kernel, "kernel_plus_allgather_ms": ms_total,
                         "tflops_kernel": flops / ms_kernel / 1e9, "tflops_with_allgather": flops / ms_total / 1e9})
        del dw
    return rows


# ------------------------------------------------------------------------------ the bench
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
    cpu_threads = host_threads()
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
    # shard outputs land in slot `rank` of a [world, B, rows] gather buffer: regions of the exchange
    # arena (peer-mapped) when the exchange is fused into the launches, plain tensors otherwise
    exchange = None
    fused = world > 1 and args.exchange == "fused" and B <= 8
    if world > 1:
        from cogni_ml_b200.sharded import ExchangingGemv, PeerExchange
        exchange = PeerExchange(64 << 20, dev)
    y_gate = torch.empty(world, B, FFN, dtype=torch.float32, device=dev)
    y_up = torch.empty(world, B, FFN, dtype=torch.float32, device=dev)
    y_down = torch.empty(world, B, HIDDEN, dtype=torch.float32, device=dev)
    if fused:   # gather buffers of (value, epoch) words, [B][world * rows]
        x_gate = exchange.buffer("y_gate", B, world * FFN)
        x_up = exchange.buffer("y_up", B, world * FFN)
        x_down = exchange.buffer("y_down", B, world * HIDDEN)
    out_host = [torch.empty(B, n, dtype=torch.float32).pin_memory() for n in (FFN, FFN, HIDDEN)]

    def gather(buf):
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

    # kernel-only graphs, one per kernel kind (an event sits between them): the N = 1 step, and at
    # N > 1 the source of the per-kernel roofline numbers
    if args.no_graph:
        run_q4, run_q6 = launch_q4, launch_q6
    else:
        run_q4, run_q6 = graphed(launch_q4).replay, graphed(launch_q6).replay

    if world == 1:
        def step(marks=None):
            run_q4()
            if marks is not None:
                marks[1].record()
            run_q6()
            if marks is not None:
                marks[2].record()
    elif fused:
        # every launch exchanges its outputs and waits for the exchange before it, layer by layer
        # (the activations stay the static xh / xf so that every rank streams the same bytes as at
        # N = 1; a consumer that reads the gathered words instead is timed in extras.sharded_27b)
        ex_gu = [ExchangingGemv(exchange, [gates[l], ups[l]], xh, [x_gate, x_up], False) for l in range(L)]
        ex_dn = [ExchangingGemv(exchange, [downs[l]], xf, [x_down], False) for l in range(L)]

        def launch_exchanging(layers=range(L)):
            for l in layers:
                ex_gu[l].run()
                ex_dn[l].run()
        run_x = launch_exchanging if args.no_graph else graphed(launch_exchanging).replay

        def step(marks=None):
            run_x()
    else:
        def step(marks=None):   # an all-gather after every projection launch (eager NCCL)
            for l in range(L):
                gate_up[l].run()
                if args.exchange == "nccl":
                    gather(y_gate)
                    gather(y_up)
                downs[l].gemv(xf, out=y_down[rank])
                if args.exchange == "nccl":
                    gather(y_down)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    check = None
    if world > 1 and not args.no_check:
        if fused:
            def layer0():
                launch_exchanging(range(1))
                torch.cuda.synchronize()
                dist.barrier()     # every rank's stores have landed: read the words' values
                for dst, src, n in ((y_gate, x_gate, FFN), (y_up, x_up, FFN), (y_down, x_down, HIDDEN)):
                    dst.copy_(src[..., 0].reshape(B, world, n).permute(1, 0, 2))
        else:
            def layer0():
                gate_up[0].run()
                downs[0].gemv(xf, out=y_down[rank])
                for b in (y_gate, y_up, y_down):
                    gather(b)
        check = sharded_check(dev, world, rank, exchange, layer0, (y_gate, y_up, y_down), cpu_threads)

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
    if world == 1:
        q4_ms = sum(m[0].elapsed_time(m[1]) for m in marks) / args.steps
        q6_ms = sum(m[1].elapsed_time(m[2]) for m in marks) / args.steps
    else:
        total_ms = reduce_max(total_ms, dev)
        q4_ms = timed(run_q4, 10)      # kernel-only, per kind, for the roofline objects
        q6_ms = timed(run_q6, 10)
    ms_per_step = total_ms / args.steps
    step_bytes = L * (2 * Q4K_BYTES + Q6K_BYTES)
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9

    # end to end with host activations
    def e2e_step():
        xh.copy_(xh_host, non_blocking=True)
        xf.copy_(xf_host, non_blocking=True)
        step()
        if fused:   # this rank's columns of the gathered words
            out_host[0].copy_(x_gate[:, rank * FFN:(rank + 1) * FFN, 0], non_blocking=True)
            out_host[1].copy_(x_up[:, rank * FFN:(rank + 1) * FFN, 0], non_blocking=True)
            out_host[2].copy_(x_down[:, rank * HIDDEN:(rank + 1) * HIDDEN, 0], non_blocking=True)
        else:
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
        e2e_ms = reduce_max(e2e_ms, dev)
    e2e_value = world * step_bytes / (e2e_ms / args.steps * 1e-3) / 1e9

    extras = None
    peaks, peak_src = measured_peaks()
    if world > 1 and not args.no_extras:
        del gates, ups, downs, gate_up
        if fused:
            del ex_gu, ex_dn
        torch.cuda.empty_cache()
        extras = {"sharded_27b": sharded_27b(dev, world, rank, exchange, peaks),
                  "prefill_sharded": prefill_sharded(dev, world, rank, peaks)}
    from cogni_ml_b200 import lib as _lib
    timeouts = _lib.cogni_qmm_wait_timeouts()

    if rank == 0:
        peak = peaks["hbm_gbs"]
        q4_per_launch = 1 if args.separate else 2     # GEMVs per Q4_K launch
        q4_launch_ms = q4_ms / (2 * L) * q4_per_launch
        q6_launch_ms = q6_ms / L
        q4_alg = q4_per_launch * Q4K_BYTES + B * HIDDEN * 4 + q4_per_launch * B * FFN * 4
        q6_alg = algorithmic_bytes(Q6K_BYTES, FFN, HIDDEN, B)
        q4_ach = q4_alg / (q4_launch_ms * 1e-3) / 1e9
        q6_ach = q6_alg / (q6_launch_ms * 1e-3) / 1e9
        if world == 1:
            par = "single GPU"
        else:
            how = {"fused": "exchanged inside every GEMV launch (peer stores + flags)",
                   "nccl": "NCCL all-gather after every projection", "none": "no exchange"}[
                       "fused" if fused else args.exchange]
            par = f"row-sharded x{world}, weak (per-GPU rows fixed), outputs {how}"
        roof_q4 = {"bound": "hbm",
                   "kernel": "Q4_K GEMV 12288x4096 b1" if args.separate else
                   "Q4_K GEMV 2 x 12288x4096 b1 (ffn_gate + ffn_up, one launch)",
                   "achieved": q4_ach, "peak": peak, "unit": "GB/s", "frac": q4_ach / peak,
                   "traffic": NCU_TRAFFIC_BYTES["q4k_2x12288x4096_b1"] // (2 // q4_per_launch) if B == 1 else None,
                   "traffic_source": TRAFFIC_SOURCE, "peak_source": f"of {peak_src}",
                   "us_per_launch": q4_launch_ms * 1e3, "algorithmic_bytes": q4_alg,
                   "share_of_step": q4_ms / (q4_ms + q6_ms), "frac_of_nominal_8tbs": q4_ach / 8000.0}
        roof_q6 = {"bound": "hbm", "kernel": "Q6_K GEMV 4096x12288 b1 (ffn_down)",
                   "achieved": q6_ach, "peak": peak, "unit": "GB/s", "frac": q6_ach / peak,
                   "traffic": NCU_TRAFFIC_BYTES["q6k_4096x12288_b1"] if B == 1 else None,
                   "traffic_source": TRAFFIC_SOURCE, "peak_source": f"of {peak_src}",
                   "us_per_launch": q6_launch_ms * 1e3, "algorithmic_bytes": q6_alg,
                   "share_of_step": q6_ms / (q4_ms + q6_ms), "frac_of_nominal_8tbs": q6_ach / 8000.0}
        dominant_q6 = q6_ms >= q4_ms
        line = {
            "metric": "q4k_q6k_gemv_weight_gbs", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic",
            "config": workload_config(L, B),
            "run": {"launch": "eager" if args.no_graph else "cuda graph replay", "parallelism": par},
            "e2e": {"value": e2e_value, "unit": "GB/s",
                    "h2d_bytes_per_step": B * (HIDDEN + FFN) * 4,
                    "d2h_bytes_per_step": B * (2 * FFN + HIDDEN) * 4},
            "gpu_launches": args.steps * (3 if args.separate else 2) * L,
            "roofline": roof_q6 if dominant_q6 else roof_q4,
            ("roofline_q4k" if dominant_q6 else "roofline_q6k"): roof_q4 if dominant_q6 else roof_q6,
            "clocks": clocks.summary(),
            "wait_timeouts": timeouts,
        }
        if check is not None:
            line["sharded_check"] = check
        if extras is not None:
            line["extras"] = extras
        if world == 1 and not args.no_extras:
            del gates, ups, downs, gate_up
            torch.cuda.empty_cache()
            line["extras"] = measure_extras(dev, gate_h, down_h, peaks, cpu_threads)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(args.cpu_seconds, cpu_threads)
            line["cpu_baseline_1thread"] = cpu_baseline(min(args.cpu_seconds, 5.0), 1)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_probe(args):
    """--probe type,out_dim,in_dim,batch[;...]: one GEMV shape at a time on one GPU, weights rotated
    through copies > L2; prints one key=value line per shape (the profiling summaries under
    profiles/ name this command).  With --no-graph the launches are eager, so that a profiler sees
    them one by one."""
    import torch

    from cogni_ml_b200 import lib, synth
    dev = torch.device("cuda", 0)
    peaks, _ = measured_peaks()
    if args.kernel_choice:
        lib.cogni_qmm_set_kernel_choice(args.kernel_choice)
    out = []
    for spec in args.probe.split(";"):
        qtype, out_dim, in_dim, batch = (int(v) for v in spec.split(","))
        raw = synth.make_weight(qtype, out_dim, in_dim, seed=1, tensor_id=qtype)
        ring = weight_ring(raw, qtype, out_dim, in_dim, dev)
        x = torch.from_numpy(synth.make_activation(batch, in_dim, seed=1)).to(dev)
        if args.no_graph:
            y = torch.empty(batch, out_dim, dtype=torch.float32, device=dev)

            def go():
                for w in ring:
                    w.gemv(x, out=y)
            us = timed(go, 3) * 1e3 / len(ring)
        else:
            us = gemv_us(ring, x, batch)
        alg = algorithmic_bytes(raw.nbytes, in_dim, out_dim, batch)
        row = {"type": TYPE_NAME[qtype], "out_dim": out_dim, "in_dim": in_dim, "batch": batch,
               "cuda_us": us, "weight_gbs": raw.nbytes / us / 1e3,
               "hbm_frac_measured": alg / us / 1e3 / peaks["hbm_gbs"], "copies": len(ring)}
        out.append(row)
        log(" ".join(f"{k}={v:.3f}" if isinstance(v, float) else f"{k}={v}" for k, v in row.items()))
        del ring
        torch.cuda.empty_cache()
    print(json.dumps({"probe": out, "wait_timeouts": lib.cogni_qmm_wait_timeouts()}))


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
                    help="skip the side measurements (other configurations, sharded 27B, prefill)")
    ap.add_argument("--no-check", action="store_true", help="N > 1: skip the sharded_check verification")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl", "none"],
                    help="N > 1: how every projection's outputs reach the other GPUs")
    ap.add_argument("--kernel-choice", type=int, default=0,
                    help="diagnostics: passed to cogni_qmm_set_kernel_choice before the run")
    ap.add_argument("--separate", action="store_true",
                    help="launch ffn_gate and ffn_up separately instead of one qmatvec_many launch")
    ap.add_argument("--no-graph", action="store_true", help="launch eagerly instead of graph replay")
    ap.add_argument("--probe", default="", help="type,out_dim,in_dim,batch[;...]: time single GEMV shapes instead of the step")
    args = ap.parse_args()
    if args.probe:
        run_probe(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
