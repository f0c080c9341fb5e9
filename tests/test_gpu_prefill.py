"""Prefill GEMM (dequant-fused, bf16 operands on the tensor cores) against the CPU oracle.

Two references per case:
  * tight: the oracle's f32 dequantised weights rounded to bf16, times the bf16 activations, in
    f64 — the kernel's exact operand set, so only fp32 accumulation order differs
    (tolerance 1e-4 * |y|inf);
  * the stated acceptance: the CPU QuantMatmul on the same bf16 activations without rounding the
    weights, on a row subset, relative error <= 2e-2 * |y|inf.
"""
import numpy as np
import pytest
import torch

from cogni_ml_b200 import DeviceQuantWeight, QuantWeight, synth

pytestmark = pytest.mark.gpu
Q4_K, Q5_K, Q6_K, Q8_0, IQ4_NL = synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.Q8_0, synth.IQ4_NL


def bf16_round(a: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(a, np.float32)).bfloat16().float().numpy()


def run_case(cuda, oracle, qtype, m, n, k, seed, out_dtype=torch.float32):
    w = synth.make_weight(qtype, n, k, seed=seed, tensor_id=qtype)
    x = bf16_round(synth.make_activation(m, k, seed=seed))
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, n, k), cuda)
    xd = torch.from_numpy(x).to(cuda).bfloat16()
    y = dw.gemm(xd, out_dtype=out_dtype).float().cpu().numpy()
    wq = bf16_round(oracle.dequantize(qtype, w, n * k)).reshape(n, k).astype(np.float64)
    ref = x.astype(np.float64) @ wq.T
    return w, x, y, ref


@pytest.mark.parametrize("qtype", [Q4_K, Q5_K, Q6_K, Q8_0, IQ4_NL])
@pytest.mark.parametrize("m,n,k", [(128, 128, 256), (256, 256, 512), (200, 200, 768), (1, 37, 256),
                                   (300, 1000, 1024)])
def test_gemm_matches_bf16_operand_reference(cuda, oracle, engine, qtype, m, n, k):
    w, x, y, ref = run_case(cuda, oracle, qtype, m, n, k, seed=3)
    assert y.shape == (m, n) and not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("tile", [128, 256, 512])
@pytest.mark.parametrize("qtype,m,n,k", [(Q4_K, 700, 300, 512), (Q6_K, 513, 128, 1024),
                                         (Q5_K, 1100, 260, 256), (Q4_K, 40, 128, 2048),
                                         (Q8_0, 530, 300, 768), (IQ4_NL, 260, 200, 512)])
def test_gemm_every_token_tile_width(cuda, oracle, engine, tile, qtype, m, n, k):
    """The token-tile width (128 / 256 / 512 tokens per CTA) is normally chosen from the shape;
    here each width is forced, with token counts that leave ragged and empty tile halves."""
    engine.lib.cogni_qmm_set_kernel_choice({128: 49, 256: 50, 512: 51}[tile])
    try:
        w, x, y, ref = run_case(cuda, oracle, qtype, m, n, k, seed=13)
    finally:
        engine.lib.cogni_qmm_set_kernel_choice(48)
    assert not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("tile", [128, 256, 512])
@pytest.mark.parametrize("qtype,m,n,k", [(Q6_K, 200, 200, 2048), (Q6_K, 300, 1000, 6144),
                                         (Q6_K, 64, 37, 4096), (Q4_K, 300, 1000, 1280),
                                         (Q5_K, 130, 129, 768), (Q4_K, 600, 50, 256),
                                         (IQ4_NL, 270, 300, 1024)])
def test_gemm_staged_superblocks(cuda, oracle, engine, tile, qtype, m, n, k):
    """Rows that are multiples of 16 bytes (Q4_K / Q5_K always, Q6_K when in_dim is a multiple of
    2048) are fetched by TMA into shared memory and expanded from there; rows beyond out_dim are
    zero-filled boxes.  The result must equal the direct-read path bit for bit (same expansion,
    same MMA order; without a split along K, whose four-way form adds the partial tiles in an
    order that depends on the number of dequant warps, which differs between the two paths)."""
    engine.lib.cogni_qmm_set_kernel_choice({128: 49, 256: 50, 512: 51}[tile])
    engine.lib.cogni_qmm_set_kernel_choice(53)
    try:
        w, x, y, ref = run_case(cuda, oracle, qtype, m, n, k, seed=19)
        engine.lib.cogni_qmm_set_kernel_choice(56)
        _, _, y_direct, _ = run_case(cuda, oracle, qtype, m, n, k, seed=19)
    finally:
        engine.lib.cogni_qmm_set_kernel_choice(55)
        engine.lib.cogni_qmm_set_kernel_choice(52)
        engine.lib.cogni_qmm_set_kernel_choice(48)
    assert not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert np.array_equal(y, y_direct)
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("qtype,m,n,k", [(Q4_K, 512, 512, 1024), (Q5_K, 700, 384, 2048),
                                         (Q4_K, 1300, 260, 4352), (Q5_K, 37, 132, 512),
                                         (Q4_K, 2048, 1280, 4096)])
def test_gemm_cta_pairs_match_single_ctas(cuda, oracle, engine, qtype, m, n, k):
    """512-token tiles of Q4_K / Q5_K run on clusters of two CTAs (tcgen05 cta_group::2: each CTA
    dequantises 128 of the 256 weight rows and loads 128 of every 256 tokens).  The accumulation
    order is the one-CTA kernel's, so the outputs must be equal bit for bit, launch after launch;
    the shapes leave a pair whose second CTA has no valid row, ragged token boxes and a K that is
    no multiple of the ring depths."""
    w = synth.make_weight(qtype, n, k, seed=29, tensor_id=qtype)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, n, k), cuda)
    x = bf16_round(synth.make_activation(m, k, seed=29))
    xd = torch.from_numpy(x).to(cuda).bfloat16()
    lib = engine.lib
    lib.cogni_qmm_set_kernel_choice(51)   # 512-token tiles
    lib.cogni_qmm_set_kernel_choice(53)   # no split along K: the pair kernel takes whole rows
    try:
        lib.cogni_qmm_set_kernel_choice(58)
        single = dw.gemm(xd).clone()
        lib.cogni_qmm_set_kernel_choice(57)
        for _ in range(20):
            assert torch.equal(dw.gemm(xd), single)
    finally:
        lib.cogni_qmm_set_kernel_choice(57)
        lib.cogni_qmm_set_kernel_choice(52)
        lib.cogni_qmm_set_kernel_choice(48)
    rb = len(w) // n
    wq = np.stack([bf16_round(oracle.dequantize(qtype, w[c * rb:(c + 1) * rb], k)) for c in range(n)])
    ref = x.astype(np.float64) @ wq.astype(np.float64).T
    y = single.float().cpu().numpy()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("qtype,m,n,k", [(Q4_K, 300, 260, 4352), (Q6_K, 100, 132, 2048)])
def test_gemm_last_row_tile_is_reproducible(cuda, engine, qtype, m, n, k):
    """A last row tile with four valid rows, launched many times: every launch must give the same
    bits.  (TMA boxes that reached beyond the last row of the matrix gave stale bytes in the rows
    inside about once in twenty launches; the boxes are kept inside the matrix since.)"""
    w = synth.make_weight(qtype, n, k, seed=23, tensor_id=qtype)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, n, k), cuda)
    xd = torch.from_numpy(bf16_round(synth.make_activation(m, k, seed=23))).to(cuda).bfloat16()
    engine.lib.cogni_qmm_set_kernel_choice(53)  # whole K per CTA: staged and direct reads then agree bit for bit
    try:
        engine.lib.cogni_qmm_set_kernel_choice(56)
        try:
            direct = dw.gemm(xd).clone()
        finally:
            engine.lib.cogni_qmm_set_kernel_choice(55)
        for _ in range(100):
            assert torch.equal(dw.gemm(xd), direct)
    finally:
        engine.lib.cogni_qmm_set_kernel_choice(52)
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("tile", [128, 256, 512])
@pytest.mark.parametrize("qtype,m,n,k", [(Q6_K, 513, 128, 4096), (Q4_K, 300, 260, 4352),
                                         (Q5_K, 64, 128, 8192), (Q8_0, 200, 130, 4096)])
def test_gemm_split_along_k(cuda, oracle, engine, tile, qtype, m, n, k):
    """Two CTAs per tile, half of K each, partial tiles added onto a zeroed y (chosen by the host
    when there are few row tiles for the SMs; forced here).  k = 4352 gives unequal halves."""
    engine.lib.cogni_qmm_set_kernel_choice({128: 49, 256: 50, 512: 51}[tile])
    engine.lib.cogni_qmm_set_kernel_choice(54)
    try:
        w, x, y, ref = run_case(cuda, oracle, qtype, m, n, k, seed=17)
        _, _, y2, _ = run_case(cuda, oracle, qtype, m, n, k, seed=17)
    finally:
        engine.lib.cogni_qmm_set_kernel_choice(48)
        engine.lib.cogni_qmm_set_kernel_choice(52)
    assert not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert np.array_equal(y, y2), "two addends commute: the split result must be reproducible"
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("qtype,m,n,k", [(Q6_K, 513, 128, 4096), (Q4_K, 300, 260, 4352),
                                         (Q8_0, 530, 300, 4096), (Q5_K, 1000, 384, 8192),
                                         (Q6_K, 512, 1024, 12288), (IQ4_NL, 77, 200, 6144)])
def test_gemm_four_ordered_splits(cuda, oracle, engine, qtype, m, n, k):
    """Four CTAs per tile, a quarter of K each.  Four float addends do not commute, so the kernel
    fixes the order: the tile's columns form four groups, split z adds its part of group
    (z + t) mod 4 at step t, and a turn counter per (tile, group) admits the steps in order.  Every
    launch must therefore give the same bits; y is not zeroed (the first part of a group is
    stored), so the output buffer starts as NaN here.  k = 4352 gives unequal quarters."""
    w = synth.make_weight(qtype, n, k, seed=31, tensor_id=qtype)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, n, k), cuda)
    x = bf16_round(synth.make_activation(m, k, seed=31))
    xd = torch.from_numpy(x).to(cuda).bfloat16()
    lib = engine.lib
    lib.cogni_qmm_set_kernel_choice(59)
    try:
        first = dw.gemm(xd).clone()
        for _ in range(20):
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device=cuda)
            assert torch.equal(dw.gemm(xd, out=out), first), "the order of the additions is fixed"
    finally:
        lib.cogni_qmm_set_kernel_choice(52)
    rb = len(w) // n
    wq = np.stack([bf16_round(oracle.dequantize(qtype, w[c * rb:(c + 1) * rb], k)) for c in range(n)])
    ref = x.astype(np.float64) @ wq.astype(np.float64).T
    y = first.cpu().numpy()
    assert not np.isnan(y).any()
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    assert lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("qtype,n,k", [(Q4_K, 1024, 4096), (Q6_K, 512, 12288), (Q8_0, 512, 4096),
                                       (IQ4_NL, 256, 2048)])
def test_gemm_within_stated_tolerance_of_cpu_quant_matmul(cuda, oracle, qtype, n, k):
    m = 512
    w, x, y, ref = run_case(cuda, oracle, qtype, m, n, k, seed=5)
    assert np.abs(y - ref).max() <= 1e-4 * np.abs(ref).max()
    rows = [0, 1, 255, 256, 511]                              # row subset through the CPU QuantMatmul
    full = np.stack([oracle.matmul_add(x[r], 1, k, w, qtype, n, np.zeros(n, np.float32),
                                       threads=oracle.max_threads()) for r in rows])
    assert np.abs(y[rows] - full).max() <= 2e-2 * np.abs(full).max()


def test_gemm_bf16_output(cuda, oracle):
    w, x, y, ref = run_case(cuda, oracle, Q4_K, 256, 256, 512, seed=7, out_dtype=torch.bfloat16)
    assert np.abs(y - ref).max() <= 1e-2 * np.abs(ref).max()    # bf16 rounding of the result
