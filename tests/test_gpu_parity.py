"""GPU parity: the CUDA path through the C ABI against the CPU oracle on the same seeded inputs.

Tolerances (stated by the benchmark's acceptance rule):
  * dequantised weights: bit-exact against the CPU dequantiser;
  * GEMV outputs: max|err| <= 1e-3 * max|y_ref| (fp32 accumulation on the GPU, f64 in the oracle);
    the reference's own CUDA probes use cos >= 0.99999 and max_diff <= 1e-3
    (bin/cuda_q4k_gemv_probe.cr:269-289), also checked here;
  * fused lm_head argmax index: exact.
"""
import numpy as np
import pytest
import torch

from cogni_ml_b200 import (DeviceQuantWeight, Projection, QuantMatmul, QuantProjectionRunner,
                           QuantWeight, synth)

pytestmark = pytest.mark.gpu

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = synth.Q8_0, synth.Q4_K, synth.Q5_K, synth.Q6_K, synth.IQ4_NL
ALL_TYPES = [Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL]
REL_TOL = 1e-3


@pytest.fixture(autouse=True, params=["auto", "rowwarp"])
def kernel_choice(request, engine):
    """Every case runs twice: automatic kernel selection (the tiled tensor-core GEMV where the
    shape allows it) and the general row-per-warp kernel forced."""
    engine.lib.cogni_qmm_set_kernel_choice(1 if request.param == "rowwarp" else 0)
    yield request.param
    engine.lib.cogni_qmm_set_kernel_choice(0)
    assert engine.lib.cogni_qmm_wait_timeouts() == 0, "a bounded device-side wait expired"


def cosine(a, b):
    a = a.astype(np.float64).ravel()
    b = b.astype(np.float64).ravel()
    return float(a @ b / (np.linalg.norm(a) * np.linalg.norm(b)))


def assert_close(y, ref, what=""):
    err = float(np.abs(y.astype(np.float64) - ref.astype(np.float64)).max())
    mag = float(np.abs(ref).max())
    assert err <= REL_TOL * mag, f"{what}: max|err| {err:.3e} > 1e-3 * |y|inf {mag:.3e}"
    assert cosine(y, ref) >= 0.99999, what


def run_gemv(cuda, qtype, out_dim, in_dim, batch, seed, addend=None):
    w = synth.make_weight(qtype, out_dim, in_dim, seed=seed, tensor_id=qtype)
    x = synth.make_activation(batch, in_dim, seed=seed)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    y = torch.full((batch, out_dim), float("nan"), dtype=torch.float32, device=cuda)
    kw = {}
    if addend == "bias":
        kw["bias"] = torch.from_numpy(np.linspace(-2, 2, out_dim, dtype=np.float32)).to(cuda)
    elif addend == "residual":
        kw["residual"] = torch.from_numpy(synth.make_activation(batch, out_dim, seed, 77)).to(cuda)
    dw.gemv(torch.from_numpy(x).to(cuda), out=y, **kw)
    return w, x, y.cpu().numpy(), {k: v.cpu().numpy() for k, v in kw.items()}


@pytest.mark.parametrize("qtype", ALL_TYPES)
def test_dequantize_bit_exact(cuda, oracle, qtype):
    out_dim, in_dim = 61, 1024
    w = synth.make_weight(qtype, out_dim, in_dim, seed=11, tensor_id=qtype)
    ref = oracle.dequantize(qtype, w, out_dim * in_dim)
    got = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda).dequantize()
    got = got.cpu().numpy().ravel()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("qtype", ALL_TYPES)
def test_dequantize_subnormal_and_extreme_scales(cuda, oracle, qtype):
    """Half scales that are subnormal, zero, negative and the largest finite value."""
    in_dim = synth.BLOCK_ELEMS[qtype] * 8
    w = synth.make_weight(qtype, 1, in_dim, seed=5, tensor_id=qtype).copy()
    bb = synth.BLOCK_BYTES[qtype]
    d_off = 208 if qtype == Q6_K else 0
    for i, h in enumerate([0x0001, 0x03FF, 0x0000, 0x8000, 0x8001, 0x7BFF, 0xFBFF, 0x0400]):
        w[i * bb + d_off] = h & 0xFF
        w[i * bb + d_off + 1] = h >> 8
    ref = oracle.dequantize(qtype, w, in_dim)
    got = DeviceQuantWeight.upload(QuantWeight(w, qtype, 1, in_dim), cuda).dequantize()
    assert np.array_equal(got.cpu().numpy().ravel().view(np.uint32), ref.view(np.uint32))


def _f16_le(h):
    return [h & 0xFF, h >> 8]


def test_iq4_nl_reference_golden_vectors_on_the_device(cuda, oracle):
    """The reference's own known-answer spec for IQ4_NL (spec/iq4_nl_dequant_spec.cr:34-106) run
    through the device: the full-block dequant is exact, and the fused matmul with the bias as the
    accumulator start agrees with the spec's bulk-dequant reference (f32 accumulation here against
    f64 there, so to 1e-6 relative instead of bit for bit)."""
    kvalues = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113], np.float32)
    raw = np.array(_f16_le(0x3C00) + [j | ((15 - j) << 4) for j in range(16)], np.uint8)
    got = DeviceQuantWeight.upload(QuantWeight(raw, IQ4_NL, 1, 32), cuda).dequantize().cpu().numpy().ravel()
    assert np.array_equal(got[:16], kvalues) and np.array_equal(got[16:], kvalues[::-1])
    # spec :73-106: two rows of weights, two rows of activations, bias [0.25, -0.75]
    in_dim, out_dim, rows = 32, 2, 2
    raw2 = _f16_le(0x3C00) + [j | ((15 - j) << 4) for j in range(16)]
    raw2 += _f16_le(0x3800) + [(15 - j) | (j << 4) for j in range(16)]
    raw2 = np.array(raw2, np.uint8)
    x = np.array([(((i * 17) % 23) - 11) for i in range(rows * in_dim)], np.float32) / np.float32(7.0)
    bias = np.array([0.25, -0.75], np.float32)
    y = QuantMatmul.matmul_add(x, rows, in_dim, raw2, IQ4_NL, out_dim, bias)
    dense = got_dense = oracle.dequantize(IQ4_NL, raw2, in_dim * out_dim).reshape(out_dim, in_dim)
    ref = bias[None, :].astype(np.float64) + x.reshape(rows, in_dim).astype(np.float64) @ dense.astype(np.float64).T
    assert np.abs(y.reshape(rows, out_dim) - ref).max() <= 1e-6 * np.abs(ref).max()
    assert np.array_equal(oracle.matmul_add(x, rows, in_dim, raw2, IQ4_NL, out_dim, bias),
                          ref.astype(np.float32).ravel())


def test_config0_q8_0_gemv_batch1(cuda, oracle):
    """Q8_0 3584 x 1024, batch 1: the reference's CPU-runnable case."""
    w, x, y, _ = run_gemv(cuda, Q8_0, 3584, 1024, 1, seed=0)
    ref = oracle.matmul_add(x, 1, 1024, w, Q8_0, 3584, np.zeros(3584, np.float32))
    assert_close(y.ravel(), ref, "Q8_0 3584x1024")
    # the reference's Q8_0 probe threshold (bin/cuda_q8_gemv_probe.cr:390)
    assert cosine(y, ref) >= 0.999999 and np.abs(y.ravel() - ref).max() <= 1e-4


@pytest.mark.parametrize("qtype,out_dim,in_dim", [(Q4_K, 12288, 4096), (Q6_K, 4096, 12288)])
def test_config1_9b_ffn_gemv_batch1(cuda, oracle, qtype, out_dim, in_dim):
    w, x, y, _ = run_gemv(cuda, qtype, out_dim, in_dim, 1, seed=1)
    ref = oracle.matmul_add(x, 1, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                            threads=oracle.max_threads())
    assert_close(y.ravel(), ref, f"type {qtype} {out_dim}x{in_dim}")


@pytest.mark.parametrize("qtype,in_dim", [(Q4_K, 2048), (Q5_K, 1024), (Q6_K, 8192), (Q6_K, 1024),
                                          (Q4_K, 256), (Q8_0, 2048), (Q8_0, 768)])
@pytest.mark.parametrize("batch", [1, 2])
def test_many_tiles_per_cta(cuda, oracle, qtype, in_dim, batch):
    """Tall weights: every persistent CTA walks ten or more row tiles, so the stage ring and the
    tile buffers of the tiled kernel wrap several times, with several stages per tile (Q6_K at
    8192 columns) and with tiles much smaller than a stage (256 and 1024 columns)."""
    sms = torch.cuda.get_device_properties(cuda).multi_processor_count
    out_dim = sms * 16 * 10 + 21
    w, x, y, _ = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=9)
    ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                            threads=oracle.max_threads())
    assert not np.isnan(y).any()
    assert_close(y.ravel(), ref, f"type {qtype} {out_dim}x{in_dim} batch {batch}")


@pytest.mark.parametrize("qtype,out_dim,in_dim,batch", [
    (Q6_K, 100, 12288, 2), (Q6_K, 333, 12288, 5), (Q4_K, 80, 16384, 8), (Q5_K, 48, 8192, 11),
    (Q8_0, 70, 12288, 4), (Q6_K, 40, 16384, 1),
])
def test_long_rows_in_column_ranges(cuda, oracle, qtype, out_dim, in_dim, batch):
    """Rows whose activations do not fit into shared memory at this batch run as several launches
    over column ranges that add onto y; the residual goes in with the first."""
    w, x, y, add = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=52, addend="residual")
    ref = np.stack([oracle.matmul_add(x[b], 1, in_dim, w, qtype, out_dim, add["residual"][b])
                    for b in range(batch)])
    assert_close(y, ref.reshape(batch, out_dim), f"type {qtype} {out_dim}x{in_dim} batch {batch}")


@pytest.mark.parametrize("qtype,out_dim,in_dim,batch", [
    (Q6_K, 4096, 12288, 1),   # the 9B ffn_down shape: fused path
    (Q4_K, 512, 2048, 2), (Q8_0, 300, 1024, 1), (Q5_K, 257, 768, 2),
    (Q6_K, 128, 1024, 5),     # batch 5: the 8-row instance of the kernel
    (Q4_K, 192, 2048, 11),    # a pass of 8 rows and a pass of 3
    (IQ4_NL, 128, 1024, 3), (IQ4_NL, 300, 2048, 1),
    (Q8_0, 64, 96, 1),        # in_dim not a multiple of 256: scratch path as well
])
def test_gemv_swiglu_fused_down_projection(cuda, oracle, qtype, out_dim, in_dim, batch):
    """y = residual + W (silu(gate) * up) (qwen35_cpu.cr:1716-1718) against the CPU restatement:
    SwiGLU product in f32, then QuantMatmul with the residual as the accumulator start."""
    w = synth.make_weight(qtype, out_dim, in_dim, seed=31, tensor_id=qtype)
    gate = synth.make_activation(batch, in_dim, seed=31, tensor_id=5) * np.float32(2.0)
    up = synth.make_activation(batch, in_dim, seed=31, tensor_id=6)
    res = synth.make_activation(batch, out_dim, seed=31, tensor_id=7)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    y = dw.gemv_swiglu(torch.from_numpy(gate).to(cuda), torch.from_numpy(up).to(cuda),
                       residual=torch.from_numpy(res).to(cuda)).cpu().numpy()
    comb = oracle.swiglu(gate, up).reshape(batch, in_dim)
    ref = np.stack([oracle.matmul_add(comb[b], 1, in_dim, w, qtype, out_dim, res[b],
                                      threads=oracle.max_threads()) for b in range(batch)])
    assert_close(y, ref, f"swiglu type {qtype} {out_dim}x{in_dim} batch {batch}")


def test_gemv_swiglu_needs_scratch_for_unfused_shapes(cuda, engine):
    # in_dim that is no multiple of 256 has no fused kernel: the product needs the caller's scratch
    w = synth.make_weight(Q8_0, 64, 96, seed=3)
    dw = DeviceQuantWeight.upload(QuantWeight(w, Q8_0, 64, 96), cuda)
    g = torch.zeros(5, 96, device=cuda)
    y = torch.empty(5, 64, device=cuda)
    st = engine.lib.cogni_qmm_gemv_swiglu(Q8_0, dw.raw.data_ptr(), g.data_ptr(), g.data_ptr(), None, 0,
                                          y.data_ptr(), None, 96, 64, 5, 0, None)
    assert st == 1004  # COGNI_QMM_ERR_SCRATCH


@pytest.mark.parametrize("qtype", ALL_TYPES)
def test_embedding_lookup_bit_exact_and_range_check(cuda, oracle, qtype):
    """Rows of a quantized [vocab, n_embd] table by device-resident token ids, bit-identical to the
    CPU dequantiser on the row slice (Qwen35CPU#embedding_lookup, qwen35_cpu.cr:3305-3332)."""
    vocab, n_embd = 1000, 1024
    w = synth.make_weight(qtype, vocab, n_embd, seed=17, tensor_id=qtype)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, vocab, n_embd), cuda)
    ids = np.array([0, 999, 17, 17, 512, 3], dtype=np.int32)
    got = dw.embedding_lookup(torch.from_numpy(ids).to(cuda)).cpu().numpy()
    rb = len(w) // vocab
    for t, tid in enumerate(ids):
        ref = oracle.dequantize(qtype, w[tid * rb:(tid + 1) * rb], n_embd)
        assert np.array_equal(got[t].view(np.uint32), ref.view(np.uint32)), (t, tid)
    with pytest.raises(IndexError):
        dw.embedding_lookup(torch.tensor([5, vocab], dtype=torch.int32, device=cuda))
    with pytest.raises(IndexError):
        dw.embedding_lookup(torch.tensor([-1], dtype=torch.int32, device=cuda))
    # without the check an id outside the table yields zeros, the others are unaffected
    out = dw.embedding_lookup(torch.tensor([vocab + 7, 3], dtype=torch.int32, device=cuda),
                              check_range=False).cpu().numpy()
    assert not out[0].any() and np.array_equal(out[1], got[5])


def test_top1_feeds_embedding_lookup_on_device(cuda, oracle):
    """argmax -> next-token embedding without leaving the device: the int32 index the fused lm_head
    writes is the token id the gather reads."""
    vocab, hid = 4096, 1024
    w = synth.make_weight(Q6_K, vocab, hid, seed=23, tensor_id=3)
    dw = DeviceQuantWeight.upload(QuantWeight(w, Q6_K, vocab, hid), cuda)
    x = synth.make_activation(1, hid, seed=23)
    idx, _val = dw.gemv_top1(torch.from_numpy(x).to(cuda))
    emb = dw.embedding_lookup(idx).cpu().numpy()
    logits = oracle.matmul_add(x, 1, hid, w, Q6_K, vocab, np.zeros(vocab, np.float32),
                               threads=oracle.max_threads())
    tid, _ = oracle.top1(logits)
    rb = len(w) // vocab
    ref = oracle.dequantize(Q6_K, w[tid * rb:(tid + 1) * rb], hid)
    assert int(idx.item()) == tid and np.array_equal(emb[0].view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("qtype,in_dim,out_dims,batch", [
    (Q4_K, 4096, [12288, 12288], 1),        # post_attention_norm -> ffn_gate + ffn_up (9B shapes)
    (Q4_K, 1024, [512, 96, 32, 32], 2),     # attn_norm -> qkv / gate / alpha / beta
    (Q6_K, 2048, [300], 1), (Q8_0, 1024, [257, 64], 2), (Q5_K, 768, [128], 1),
    (Q4_K, 512, [64, 64], 4),               # batch 4: the 4-row instance of the kernel
    (Q6_K, 1024, [96, 40], 7),
    (IQ4_NL, 512, [64, 64], 2), (IQ4_NL, 1024, [100, 36], 6),
])
def test_gemv_many_rmsnorm_fused_prologue(cuda, oracle, qtype, in_dim, out_dims, batch):
    """y_j = W_j (RMSNorm(x) * w_norm) for matrices sharing x (qwen35_cpu.cr:484-490, 1793, 1883)
    against the CPU restatement: rms_norm rows, then QuantMatmul per matrix."""
    from cogni_ml_b200 import gemv_many
    x = synth.make_activation(batch, in_dim, seed=41, tensor_id=1) * np.float32(3.0)
    wn = (1.0 + 0.1 * synth.make_activation(1, in_dim, seed=41, tensor_id=2)).ravel()
    raws = [synth.make_weight(qtype, n, in_dim, seed=41 + j, tensor_id=qtype) for j, n in enumerate(out_dims)]
    dws = [DeviceQuantWeight.upload(QuantWeight(r, qtype, n, in_dim), cuda) for r, n in zip(raws, out_dims)]
    ys = gemv_many(dws, torch.from_numpy(x).to(cuda), norm_weight=torch.from_numpy(wn).to(cuda), eps=1e-6)
    xn = oracle.rmsnorm(x, wn, 1e-6)
    for r, n, y in zip(raws, out_dims, ys):
        ref = oracle.matmul_add(xn, batch, in_dim, r, qtype, n, np.zeros(n, np.float32),
                                threads=oracle.max_threads()).reshape(batch, n)
        assert_close(y.cpu().numpy(), ref, f"rmsnorm + gemv type {qtype} {n}x{in_dim} batch {batch}")


LAYER = [("q_proj", Q4_K, 4096, 4096), ("k_proj", Q4_K, 1024, 4096), ("v_proj", Q4_K, 1024, 4096),
         ("o_proj", Q4_K, 4096, 4096), ("ffn_gate", Q4_K, 12288, 4096),
         ("ffn_down", Q6_K, 4096, 12288), ("q5k_variant", Q5_K, 4096, 4096)]


@pytest.mark.parametrize("batch", [1, 4, 8, 16])
def test_config2_layer_projections_row_batched(cuda, oracle, batch):
    """One 9B-shaped layer's projections at batch 1/4/8/16 (the speculative-verifier rows)."""
    for i, (name, qtype, out_dim, in_dim) in enumerate(LAYER):
        w, x, y, _ = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=20 + i)
        ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim,
                                np.zeros(out_dim, np.float32), threads=oracle.max_threads())
        assert not np.isnan(y).any(), name
        assert_close(y.ravel(), ref, f"{name} batch {batch}")


@pytest.mark.parametrize("qtype", ALL_TYPES)
@pytest.mark.parametrize("batch", [1, 2, 3, 5, 7, 16, 19])
def test_ragged_shapes(cuda, oracle, qtype, batch):
    """out_dim that is no multiple of any tile, the smallest legal in_dim, odd batches."""
    be = synth.BLOCK_ELEMS[qtype]
    for out_dim, in_dim in [(1, be), (37, 256), (130, 768), (257, 1280)]:
        w, x, y, _ = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=31)
        ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32))
        assert not np.isnan(y).any()
        assert_close(y.ravel(), ref, f"type {qtype} {out_dim}x{in_dim} b{batch}")


@pytest.mark.parametrize("qtype", ALL_TYPES)
@pytest.mark.parametrize("addend", ["bias", "residual"])
def test_bias_and_residual(cuda, oracle, qtype, addend):
    out_dim, in_dim, batch = 300, 1024, 4
    w, x, y, add = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=41, addend=addend)
    if addend == "bias":
        ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, add["bias"])
    else:  # the reference passes a residual as the bias of a one-row call
        ref = np.concatenate([oracle.matmul_add(x[b], 1, in_dim, w, qtype, out_dim,
                                                add["residual"][b]) for b in range(batch)])
    assert_close(y.ravel(), ref, f"{addend} type {qtype}")


@pytest.mark.parametrize("qtype", ALL_TYPES)
def test_matmul_add_host_surface(cuda, oracle, qtype):
    """QuantMatmul.matmul_add with host arrays, as spec/q4k_matmul_spec.cr:62-88 drives it."""
    rows, in_dim, out_dim = 2, 4096, 96
    w = synth.make_weight(qtype, out_dim, in_dim, seed=51, tensor_id=qtype)
    i = np.arange(rows * in_dim, dtype=np.uint64)
    x = (((i * 2654435761) % (1 << 32)) % 2000).astype(np.int64) - 1000
    x = (x / np.float32(1000.0)).astype(np.float32)
    bias = ((np.arange(out_dim) % 10) / np.float32(100.0)).astype(np.float32)
    mine = QuantMatmul.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias)
    ref = oracle.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias)
    assert_close(mine, ref, f"matmul_add type {qtype}")


@pytest.mark.parametrize("qtype", [Q4_K, Q5_K, Q6_K, Q8_0])
@pytest.mark.parametrize("batch", [1, 2, 5])
def test_gemv_many_shares_x_across_weights(cuda, oracle, qtype, batch):
    """qmatvec_many: several matrices (ragged row counts, more than one launch's worth), one x."""
    from cogni_ml_b200 import gemv_many
    in_dim = 1024
    out_dims = [33, 256, 16, 1000] + [48] * 31          # 35 matrices > 32 per launch
    x = synth.make_activation(batch, in_dim, seed=43)
    xd = torch.from_numpy(x).to(cuda)
    raws = [synth.make_weight(qtype, n, in_dim, seed=43, tensor_id=100 + j) for j, n in enumerate(out_dims)]
    dws = [DeviceQuantWeight.upload(QuantWeight(r, qtype, n, in_dim), cuda) for r, n in zip(raws, out_dims)]
    outs = [torch.full((batch, n), float("nan"), device=cuda) for n in out_dims]
    gemv_many(dws, xd, outs)
    for j, n in enumerate(out_dims):
        ref = oracle.matmul_add(x, batch, in_dim, raws[j], qtype, n, np.zeros(n, np.float32))
        assert_close(outs[j].cpu().numpy().ravel(), ref, f"matrix {j}")


def test_matmul_add_rejects_unknown_type(cuda):
    with pytest.raises(RuntimeError, match="unsupported tensor type"):
        QuantMatmul.matmul_add(np.zeros(32, np.float32), 1, 32, np.zeros(64, np.uint8), 2, 1,
                               np.zeros(1, np.float32))


@pytest.mark.parametrize("qtype", ALL_TYPES)
@pytest.mark.parametrize("batch", [1, 3, 4, 8, 11, 16])
def test_lm_head_top1(cuda, oracle, qtype, batch):
    out_dim, in_dim, base = 5000, 1024, 7000
    w = synth.make_weight(qtype, out_dim, in_dim, seed=61, tensor_id=qtype)
    x = synth.make_activation(batch, in_dim, seed=61)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    dw.row_begin = base
    xd = torch.from_numpy(x).to(cuda)
    for _ in range(2):  # twice: the scratch buffer must come back ready for reuse
        idx, val, key = dw.gemv_top1(xd, want_keys=True)
        logits = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim,
                                   np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
        for b in range(batch):
            ri, rv = oracle.top1(logits[b])
            assert int(idx[b]) == ri + base
            assert abs(float(val[b]) - rv) <= REL_TOL * np.abs(logits[b]).max()
        from cogni_ml_b200 import unpack_top1_keys
        i2, v2 = unpack_top1_keys(key)
        assert torch.equal(i2, idx) and torch.equal(v2, val)


@pytest.mark.parametrize("qtype", ALL_TYPES)
@pytest.mark.parametrize("batch", [1, 2, 5])
def test_lm_head_top2_and_margin(cuda, oracle, qtype, batch):
    """Best and runner-up per row (the verifier's margin), against a sort of the oracle's logits;
    twice, because the scratch buffer must come back ready for reuse."""
    out_dim, in_dim, base = 5003, 1024, 100
    w = synth.make_weight(qtype, out_dim, in_dim, seed=63, tensor_id=qtype)
    x = synth.make_activation(batch, in_dim, seed=63)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    dw.row_begin = base
    xd = torch.from_numpy(x).to(cuda)
    logits = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim,
                               np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
    for _ in range(2):
        idx, val, key = dw.gemv_top2(xd, want_keys=True)
        for b in range(batch):
            order = np.argsort(-logits[b], kind="stable")[:2]      # stable: lower index first on ties
            scale = np.abs(logits[b]).max()
            gap12 = logits[b][order[0]] - logits[b][order[1]]
            third = np.sort(logits[b])[-3]
            if gap12 > 4 * REL_TOL * scale and logits[b][order[1]] - third > 4 * REL_TOL * scale:
                assert [int(idx[b, 0]) - base, int(idx[b, 1]) - base] == list(order)
            assert abs(float(val[b, 0]) - logits[b][order[0]]) <= REL_TOL * scale
            assert abs(float(val[b, 1]) - logits[b][order[1]]) <= REL_TOL * scale
            assert float(val[b, 0]) >= float(val[b, 1])
        assert (key[:, 0] > key[:, 1]).all()
    # the first column is what the fused top-1 returns
    i1, v1 = dw.gemv_top1(xd)
    assert torch.equal(i1, idx[:, 0].contiguous()) or batch > 2   # batch > 2 takes another GEMV kernel


def test_lm_head_top2_tie_takes_the_two_lowest_indices(cuda):
    in_dim, out_dim = 256, 300
    row = synth.make_weight(Q6_K, 1, in_dim, seed=71)
    w = np.tile(row, out_dim)
    x = synth.make_activation(1, in_dim, seed=71)
    dw = DeviceQuantWeight.upload(QuantWeight(w, Q6_K, out_dim, in_dim), cuda)
    idx, val = dw.gemv_top2(torch.from_numpy(x).to(cuda))
    assert idx[0].tolist() == [0, 1] and float(val[0, 0]) == float(val[0, 1])


@pytest.mark.parametrize("qtype,batch", [(Q6_K, 1), (Q4_K, 2), (Q8_0, 1), (Q6_K, 5), (Q4_K, 8),
                                         (Q5_K, 12), (Q8_0, 3)])
def test_lm_head_top1_with_fused_output_norm(cuda, oracle, qtype, batch):
    """output_norm -> lm_head -> argmax per row in one call (rmsnorm_project_top1_rows,
    qwen35_metal.cr:9187) against rms_norm rows + QuantMatmul + argmax on the CPU."""
    out_dim, in_dim = 4000, 1024
    w = synth.make_weight(qtype, out_dim, in_dim, seed=65, tensor_id=qtype)
    x = synth.make_activation(batch, in_dim, seed=65) * np.float32(4.0)
    wn = (1.0 + 0.2 * synth.make_activation(1, in_dim, seed=65, tensor_id=9)).ravel()
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    idx, val = dw.gemv_top1(torch.from_numpy(x).to(cuda), norm_weight=torch.from_numpy(wn).to(cuda))
    xn = oracle.rmsnorm(x, wn, 1e-6)
    logits = oracle.matmul_add(xn, batch, in_dim, w, qtype, out_dim,
                               np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
    for b in range(batch):
        ri, rv = oracle.top1(logits[b])
        assert int(idx[b]) == ri and abs(float(val[b]) - rv) <= REL_TOL * np.abs(logits[b]).max()


def test_lm_head_top1_tie_takes_lowest_index(cuda):
    """Identical rows give identical logits: the lowest row index must win."""
    in_dim, out_dim = 256, 300
    row = synth.make_weight(Q6_K, 1, in_dim, seed=71)
    w = np.tile(row, out_dim)
    x = synth.make_activation(1, in_dim, seed=71)
    dw = DeviceQuantWeight.upload(QuantWeight(w, Q6_K, out_dim, in_dim), cuda)
    idx, _ = dw.gemv_top1(torch.from_numpy(x).to(cuda))
    assert int(idx[0]) == 0


def test_runner_lifecycle_matches_oracle(cuda, oracle):
    tokens, hidden, ffn = 4, 1024, 1536
    gate = QuantWeight(synth.make_weight(Q4_K, ffn, hidden, 81, 1), Q4_K, ffn, hidden)
    down = QuantWeight(synth.make_weight(Q6_K, hidden, ffn, 81, 2), Q6_K, hidden, ffn)
    xs = synth.make_activation(tokens, hidden, 81, 3)
    hs = synth.make_activation(tokens, ffn, 81, 4)
    runner = QuantProjectionRunner.from_weights(
        [Projection("ffn_gate", gate, "x"), Projection("ffn_down", down, "h", residual="x")],
        tokens, {"x": xs, "h": hs}, cuda)
    runner.upload_weights()
    runner.reset_sequence()
    runner.active_tokens = 3
    assert runner.run_repeated(2) == 6
    out = runner.read_outputs()
    ref_gate = oracle.matmul_add(xs, 3, hidden, gate.raw, Q4_K, ffn, np.zeros(ffn, np.float32))
    assert_close(out["ffn_gate"].ravel(), ref_gate, "runner gate")
    for t in range(3):
        ref = oracle.matmul_add(hs[t], 1, ffn, down.raw, Q6_K, hidden, xs[t])
        assert_close(out["ffn_down"][t], ref, "runner down+residual")
    runner.close()
    runner.close()  # idempotent, as every close in the reference's driver binding


@pytest.mark.parametrize("qtype,in_dim,slabs", [
    (Q4_K, 4096, 2), (Q4_K, 4096, 4), (Q5_K, 2048, 2), (Q6_K, 12288, 4), (Q6_K, 12288, 3),
    (Q6_K, 5120, 5), (Q8_0, 2048, 2), (IQ4_NL, 2048, 2), (Q6_K, 3072, 3),
])
@pytest.mark.parametrize("batch", [1, 2, 4, 8])
def test_gemv_k_slabs(cuda, oracle, engine, kernel_choice, qtype, in_dim, slabs, batch):
    """The tiled GEMV with the K dimension of every row tile split over `slabs` CTAs whose partial
    sums meet in the workspace: same results as whole rows per CTA, bit-identical from launch to
    launch (the slabs are summed in slab order whoever arrives last), residual added once, ragged
    last tile, and the fused top-1 on the completed rows."""
    if kernel_choice == "rowwarp":
        pytest.skip("slabs exist only in the tiled kernel")
    out_dim = 16 * 37 + 5
    engine.lib.cogni_qmm_set_kernel_choice(60 + slabs)
    try:
        w, x, y, add = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=61, addend="residual")
        dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
        xd = torch.from_numpy(x).to(cuda)
        res = torch.from_numpy(add["residual"]).to(cuda)
        again = [dw.gemv(xd, residual=res).cpu().numpy() for _ in range(3)]
        idx, val = dw.gemv_top1(xd)
    finally:
        engine.lib.cogni_qmm_set_kernel_choice(60)
    ref = np.stack([oracle.matmul_add(x[b], 1, in_dim, w, qtype, out_dim, add["residual"][b],
                                      threads=oracle.max_threads()) for b in range(batch)])
    assert not np.isnan(y).any()
    assert_close(y, ref, f"slabs {slabs} type {qtype} {out_dim}x{in_dim} batch {batch}")
    for a in again:
        assert np.array_equal(a.view(np.uint32), y.view(np.uint32)), "slab sums depend on arrival order"
    logits = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32),
                               threads=oracle.max_threads()).reshape(batch, out_dim)
    for b in range(batch):
        assert int(idx[b]) == oracle.top1(logits[b])[0]


@pytest.mark.parametrize("qtype", [Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL])
@pytest.mark.parametrize("in_dim", [32768, 32768 + 256])
@pytest.mark.parametrize("batch", [1, 8])
def test_gemv_longest_rows(cuda, oracle, engine, kernel_choice, qtype, in_dim, batch):
    """Rows of 32768 columns are the longest the tiled kernel takes (128 work items per row tile);
    one superblock more goes to the row-per-warp kernel.  Either way the call must succeed and
    agree with the oracle, with the residual added once."""
    out_dim = 16 * 5 + 3
    w, x, y, add = run_gemv(cuda, qtype, out_dim, in_dim, batch, seed=71, addend="residual")
    ref = np.stack([oracle.matmul_add(x[b], 1, in_dim, w, qtype, out_dim, add["residual"][b],
                                      threads=oracle.max_threads()) for b in range(batch)])
    assert not np.isnan(y).any()
    assert_close(y, ref, f"type {qtype} {out_dim}x{in_dim} batch {batch}")
    assert engine.lib.cogni_qmm_wait_timeouts() == 0


@pytest.mark.parametrize("qtype,batch,out_dim", [(IQ4_NL, 1, 2000), (IQ4_NL, 2, 5000), (IQ4_NL, 1, 300),
                                                 (Q4_K, 3, 4000), (Q6_K, 5, 2500), (Q8_0, 1, 1000)])
def test_fused_top1_stays_inside_an_exactly_sized_scratch(cuda, engine, oracle, kernel_choice, qtype, batch, out_dim):
    """The fused top-1 instances run 4 or 8 batch rows per launch whatever the batch; only the
    caller's `batch` rows have slots in the scratch.  A sentinel-filled guard region right behind a
    scratch buffer of exactly cogni_qmm_gemv_top1_scratch_bytes() must come back untouched."""
    in_dim = 1024
    w = synth.make_weight(qtype, out_dim, in_dim, seed=71, tensor_id=qtype)
    x = synth.make_activation(batch, in_dim, seed=71)
    dw = DeviceQuantWeight.upload(QuantWeight(w, qtype, out_dim, in_dim), cuda)
    need = engine.lib.cogni_qmm_gemv_top1_scratch_bytes(out_dim, batch)
    guard = 64 * 1024
    buf = torch.zeros(need + guard, dtype=torch.uint8, device=cuda)
    buf[need:] = 0xA5
    xd = torch.from_numpy(x).to(cuda)
    idx = torch.empty(batch, dtype=torch.int32, device=cuda)
    val = torch.empty(batch, dtype=torch.float32, device=cuda)
    for _ in range(2):
        st = engine.lib.cogni_qmm_gemv_top1(qtype, dw.raw.data_ptr(), xd.data_ptr(), in_dim, out_dim, batch, 0,
                                            buf.data_ptr(), need, idx.data_ptr(), val.data_ptr(), None, None)
        assert st == 0
    torch.cuda.synchronize()
    assert bool((buf[need:] == 0xA5).all()), "the kernel wrote behind the caller's scratch buffer"
    logits = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32)).reshape(batch, out_dim)
    for b in range(batch):
        assert int(idx[b]) == oracle.top1(logits[b])[0]


def test_expired_wait_is_counted_reported_and_reset(cuda, engine, oracle):
    """A bounded device-side wait that runs out: the kernel returns, cogni_qmm_wait_timeouts()
    reads 1, the host-buffer entry point reports COGNI_QMM_ERR_TIMEOUT instead of handing back a
    result, and after cogni_qmm_reset_wait_timeouts() launches are valid again.  The wait is made
    to run out by a one-warp kernel that waits 2 ms on a barrier nothing arrives at."""
    lib = engine.lib
    assert lib.cogni_qmm_wait_timeouts() == 0
    out_dim, in_dim = 256, 1024
    w = synth.make_weight(Q4_K, out_dim, in_dim, seed=81, tensor_id=Q4_K)
    x = synth.make_activation(1, in_dim, seed=81)
    ref = oracle.matmul_add(x, 1, in_dim, w, Q4_K, out_dim, np.zeros(out_dim, np.float32))
    try:
        assert lib.cogni_qmm_diag_expire_wait(2000, None) == 0
        torch.cuda.synchronize()
        assert lib.cogni_qmm_wait_timeouts() == 1
        y = np.zeros(out_dim, np.float32)
        st = lib.cogni_qmm_matmul_add_host(x.ctypes.data, 1, in_dim, w.ctypes.data, w.nbytes, Q4_K, out_dim,
                                           None, y.ctypes.data)
        assert st == 1007 and b"wait expired" in lib.cogni_qmm_status_string(st)
    finally:
        assert lib.cogni_qmm_reset_wait_timeouts() == 0
    assert lib.cogni_qmm_wait_timeouts() == 0
    y = QuantMatmul.matmul_add(x, 1, in_dim, w, Q4_K, out_dim, np.zeros(out_dim, np.float32))
    assert_close(y.ravel(), ref, "after the reset")
