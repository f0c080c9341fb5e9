"""The benchmark's configurations at their own shapes, through the C ABI against the CPU oracle.

  * prefill (chunked) GEMM: Q4_K 12288 x 4096 and Q6_K 4096 x 12288, M in {512, 2048, 4096}, the
    host's automatic tile / split choice.  8 evenly spaced token rows x all n against the CPU
    QuantMatmul (<= 2e-2 * |y|inf, the stated bf16-operand tolerance); all token rows x 64 output
    columns against the kernel's exact operand set (bf16 activations x bf16-rounded oracle weights
    in f64, <= 1e-4 * |y|inf).
  * 27B-scale decode: Q4_K 17408 x 5120 and Q6_K 5120 x 17408 at batch 1 and 8
    (<= 1e-3 * |y|inf), the Q6_K 151936 x 5120 lm_head at batch 1 and 8 with the fused top-1:
    argmax EQUAL to the oracle's (QuantMatmul, then max and first index, qwen35_cpu.cr:2045-2056);
    the oracle's top-1 / top-2 margin is printed beside the engine's max|err| on the logits so
    that a near-tie is visible.
  * adversarial activations for the tiled GEMV's block-floating-point step (activations are
    quantised to 15 bits per scale group before the integer MMAs): one 2**20 outlier in every
    scale group, groups that are tiny next to their neighbours, a dynamic range of 2**40 across a
    row.
"""
import numpy as np
import pytest
import torch

from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth

pytestmark = pytest.mark.gpu
Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.IQ4_NL


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).bfloat16().float().numpy()


_weights = {}


def weight(qtype, out_dim, in_dim, seed):
    key = (qtype, out_dim, in_dim, seed)
    if key not in _weights:
        _weights.clear()  # one big tensor at a time
        _weights[key] = synth.make_weight(qtype, out_dim, in_dim, seed=seed, tensor_id=qtype)
    return _weights[key]


@pytest.mark.parametrize("m", [512, 2048, 4096])
@pytest.mark.parametrize("qtype,n,k", [(Q4_K, 12288, 4096), (Q6_K, 4096, 12288)])
def test_prefill_gemm_at_benchmark_shapes(cuda, oracle, engine, qtype, n, k, m):
    w = weight(qtype, n, k, seed=4)
    x = bf16_round(synth.make_activation(m, k, seed=4 + m))
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, n, k), cuda)
    y = dw.gemm(torch.from_numpy(x).to(cuda).bfloat16()).cpu().numpy()
    assert y.shape == (m, n) and np.isfinite(y).all()
    # 8 evenly spaced token rows x all n against the CPU QuantMatmul
    rows = [int(r) for r in np.linspace(0, m - 1, 8)]
    full = np.stack([oracle.matmul_add(x[r], 1, k, w, qtype, n, np.zeros(n, np.float32),
                                       threads=oracle.max_threads()) for r in rows])
    err = np.abs(y[rows] - full).max() / np.abs(full).max()
    # all token rows x 64 evenly spaced output columns against the kernel's exact operand set
    cols = np.linspace(0, n - 1, 64).astype(np.int64)
    rb = len(w) // n
    wq = np.stack([bf16_round(oracle.dequantize(qtype, w[c * rb:(c + 1) * rb], k)) for c in cols])
    ref = x.astype(np.float64) @ wq.astype(np.float64).T
    err_tight = np.abs(y[:, cols] - ref).max() / np.abs(ref).max()
    print(f"prefill type={qtype} M={m} N={n} K={k} rel_err_vs_cpu_quantmatmul={err:.3e} "
          f"rel_err_vs_bf16_operands={err_tight:.3e}")
    assert err <= 2e-2
    assert err_tight <= 1e-4
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("batch", [1, 8])
@pytest.mark.parametrize("qtype,out_dim,in_dim", [(Q4_K, 17408, 5120), (Q6_K, 5120, 17408)])
def test_27b_projections(cuda, oracle, engine, qtype, out_dim, in_dim, batch):
    w = weight(qtype, out_dim, in_dim, seed=5)
    x = synth.make_activation(batch, in_dim, seed=50 + batch)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    y = torch.full((batch, out_dim), float("nan"), dtype=torch.float32, device=cuda)
    dw.gemv(torch.from_numpy(x).to(cuda), out=y)
    y = y.cpu().numpy()
    ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                            threads=oracle.max_threads()).reshape(batch, out_dim)
    err = np.abs(y - ref).max() / np.abs(ref).max()
    print(f"27b type={qtype} {out_dim}x{in_dim} batch={batch} rel_err={err:.3e}")
    assert np.isfinite(y).all() and err <= 1e-3
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("batch", [1, 8])
def test_27b_lm_head_top1_equals_the_cpu_argmax(cuda, oracle, engine, batch):
    vocab, hid = 151936, 5120
    w = weight(Q6_K, vocab, hid, seed=7)
    x = synth.make_activation(batch, hid, seed=70 + batch)
    dw = DeviceQuantWeight.upload(QuantWeight(w, Q6_K, vocab, hid), cuda)
    xd = torch.from_numpy(x).to(cuda)
    idx, val = dw.gemv_top1(xd)
    logits_gpu = dw.gemv(xd).cpu().numpy()
    logits = oracle.matmul_add(x, batch, hid, w, Q6_K, vocab, np.zeros(vocab, np.float32),
                               threads=oracle.max_threads()).reshape(batch, vocab)
    max_err = float(np.abs(logits_gpu - logits).max())
    for b in range(batch):
        ri, rv = oracle.top1(logits[b])
        second = float(np.partition(logits[b], -2)[-2])
        print(f"lm_head batch={batch} row={b} oracle_top1={ri} engine_top1={int(idx[b])} "
              f"value={float(rv):.6e} margin_top1_top2={float(rv) - second:.3e} "
              f"engine_max_abs_err_on_logits={max_err:.3e}")
        assert int(idx[b]) == ri, "fused lm_head argmax differs from the CPU reference"
        assert abs(float(val[b]) - float(rv)) <= 1e-3 * abs(float(rv))
    assert max_err <= 1e-3 * np.abs(logits).max()
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


def adversarial(kind, batch, in_dim, seed):
    x = synth.make_activation(batch, in_dim, seed=seed).copy()
    rng = np.random.default_rng(seed)
    if kind == "outlier_per_group":       # one 2**20 outlier in every 16-element group
        pos = np.arange(0, in_dim, 16) + rng.integers(0, 16, in_dim // 16)
        x[:, pos] *= np.float32(2.0 ** 20)
    elif kind == "tiny_groups":           # every other 32-element group 2**-20 of its neighbours
        g = (np.arange(in_dim) // 32) % 2 == 1
        x[:, g] *= np.float32(2.0 ** -20)
    elif kind == "wide_range":            # magnitudes sweep 2**-20 .. 2**20 along the row
        x *= np.exp2(np.linspace(-20, 20, in_dim)).astype(np.float32)
    elif kind == "zeros_and_one":         # all zero but one element per row
        x[:] = 0
        x[np.arange(batch), rng.integers(0, in_dim, batch)] = 3.0
    return x


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL])
@pytest.mark.parametrize("kind", ["outlier_per_group", "tiny_groups", "wide_range", "zeros_and_one"])
@pytest.mark.parametrize("batch", [1, 4, 8])
def test_adversarial_activations(cuda, oracle, engine, qtype, kind, batch):
    out_dim, in_dim = 512, 4096
    w = synth.make_weight(qtype, out_dim, in_dim, seed=9, tensor_id=qtype)
    x = adversarial(kind, batch, in_dim, seed=90 + batch)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    y = dw.gemv(torch.from_numpy(x).to(cuda)).cpu().numpy()
    ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                            threads=oracle.max_threads()).reshape(batch, out_dim)
    for b in range(batch):  # per row of x: the rows' magnitudes differ by design
        err = np.abs(y[b] - ref[b]).max() / np.abs(ref[b]).max()
        assert err <= 1e-3, f"type {qtype} {kind} batch row {b}: rel err {err:.3e}"
    assert engine.lib.cogni_qmm_wait_timeouts() == 0
