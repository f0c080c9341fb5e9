"""CPU oracle against every pin available without the reference toolchain.

  * the reference's own synthetic known-answer spec (spec/iq4_nl_dequant_spec.cr:34-106), which
    pins fp16_to_f32, the nibble order and the bias-seeded f64 accumulator shared by all types;
  * hand-derivable known-answer blocks per type (tests/golden/known_answer_blocks.json);
  * a second, independently written numpy restatement (bit-exact dequantisation, identical fused
    matmul after rounding to f32);
  * the reference's relational specs on synthetic tensors: fused matmul vs bulk dequant + dense
    f64 matmul (spec/q4k_matmul_spec.cr:62-88: cos >= 0.9999999, max|d|/max|ref| <= 1e-5).
"""
import json
from pathlib import Path

import numpy as np
import pytest

from cogni_ml_b200 import synth
from oracle import oracle_np

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 8, 12, 13, 14, 20
TYPES = [Q8_0, Q4_K, Q5_K, Q6_K]
IQ4_NL_KVALUES = np.array([-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113],
                          dtype=np.float32)


def f16_le(v):
    return [v & 0xFF, (v >> 8) & 0xFF]


def test_fp16_to_f32_all_65536_values(oracle):
    """dequant.cr:257-283 against numpy's IEEE conversion; NaNs compared by class."""
    h = np.arange(65536, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.fp16_to_f32(int(v)) for v in h], dtype=np.float32)
    nan = np.isnan(ref)
    assert np.array_equal(np.isnan(got), nan)
    assert np.array_equal(got[~nan].view(np.uint32), ref[~nan].view(np.uint32))
    assert oracle.fp16_to_f32(0x0001) == np.float32(2.0 ** -24)       # smallest subnormal
    assert oracle.fp16_to_f32(0x8000).view(np.uint32) == 0x80000000   # -0.0 keeps its sign


def test_get_scale_min_k4_inverts_the_packing(oracle):
    rng = np.random.default_rng(0)
    sc = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    mn = rng.integers(0, 64, size=(50, 8), dtype=np.uint8)
    packed = synth.pack_scales_k4(sc, mn)
    for i in range(50):
        for j in range(8):
            assert oracle.get_scale_min_k4(j, packed[i]) == (float(sc[i, j]), float(mn[i, j]))


def test_iq4_nl_full_block_matches_reference_spec(oracle):
    """spec/iq4_nl_dequant_spec.cr:35-51."""
    raw = f16_le(0x3C00) + [j | ((15 - j) << 4) for j in range(16)]
    out = oracle.dequantize(IQ4_NL, np.array(raw, np.uint8), 32)
    assert np.array_equal(out[:16], IQ4_NL_KVALUES)
    assert np.array_equal(out[16:], IQ4_NL_KVALUES[::-1])


def test_iq4_nl_partial_tail_block_matches_reference_spec(oracle):
    """spec/iq4_nl_dequant_spec.cr:53-69."""
    raw = f16_le(0x3C00) + [j | ((15 - j) << 4) for j in range(16)]
    raw += f16_le(0xB800) + [0x08] * 16
    out = oracle.dequantize(IQ4_NL, np.array(raw, np.uint8), 40)
    assert out.size == 40
    assert (out[0], out[15], out[16], out[31]) == (-127.0, 113.0, 113.0, -127.0)
    assert np.array_equal(out[32:40], np.full(8, -0.5, np.float32))


def test_iq4_nl_fused_matmul_equals_bulk_dequant_matmul(oracle):
    """spec/iq4_nl_dequant_spec.cr:73-106: exact equality, bias as the accumulator start."""
    in_dim, out_dim, rows = 32, 2, 2
    raw = f16_le(0x3C00) + [j | ((15 - j) << 4) for j in range(16)]
    raw += f16_le(0x3800) + [(15 - j) | (j << 4) for j in range(16)]
    raw = np.array(raw, np.uint8)
    x = np.array([(((i * 17) % 23) - 11) for i in range(rows * in_dim)], np.float32) / np.float32(7.0)
    bias = np.array([0.25, -0.75], np.float32)
    mine = oracle.matmul_add(x, rows, in_dim, raw, IQ4_NL, out_dim, bias)
    dense = oracle.dequantize(IQ4_NL, raw, in_dim * out_dim)
    ref = np.zeros(rows * out_dim, np.float32)
    for r in range(rows):
        for o in range(out_dim):
            s = float(bias[o])
            for j in range(in_dim):
                s += float(x[r * in_dim + j]) * float(dense[o * in_dim + j])
            ref[r * out_dim + o] = np.float32(s)
    assert np.array_equal(mine, ref)


def test_known_answer_blocks(oracle):
    cases = json.loads((Path(__file__).parent / "golden" / "known_answer_blocks.json").read_text())
    assert sorted(c["type"] for c in cases) == TYPES
    for c in cases:
        raw = np.array(c["raw"], np.uint8)
        exp = np.array(c["expected"], np.float32)
        got = oracle.dequantize(c["type"], raw, c["n"])
        assert np.array_equal(got.view(np.uint32), exp.view(np.uint32)), f"type {c['type']}"
        assert np.array_equal(oracle_np.dequantize(c["type"], raw, c["n"]).view(np.uint32),
                              exp.view(np.uint32))
        # fused matmul against one-hot activations reproduces each weight, plus the bias
        n = c["n"]
        for j in (0, 1, 17, n // 2, n - 1):
            x = np.zeros(n, np.float32)
            x[j] = 1.0
            y = oracle.matmul_add(x, 1, n, raw, c["type"], 1, np.array([3.0], np.float32))
            assert y[0] == np.float32(3.0 + float(exp[j]))


@pytest.mark.parametrize("qtype", TYPES)
def test_c_oracle_agrees_with_numpy_restatement(oracle, qtype):
    out_dim, in_dim, rows = 23, 1024, 3
    w = synth.make_weight(qtype, out_dim, in_dim, seed=5, tensor_id=qtype)
    a = oracle.dequantize(qtype, w, out_dim * in_dim)
    b = oracle_np.dequantize(qtype, w, out_dim * in_dim)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))
    x = synth.make_activation(rows, in_dim, seed=5)
    bias = np.linspace(-1, 1, out_dim).astype(np.float32)
    y1 = oracle.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias)
    y2 = oracle_np.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias)
    assert np.abs(y1 - y2).max() <= 2e-7 * np.abs(y1).max()
    assert np.array_equal(y1, oracle.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias, threads=4))


@pytest.mark.parametrize("qtype", TYPES)
def test_fused_matmul_vs_bulk_dequant_relational_spec(oracle, qtype):
    """spec/q4k_matmul_spec.cr:62-88 on a synthetic 4096-column tensor, for every type."""
    rows, in_dim, out_dim = 2, 4096, 64
    w = synth.make_weight(qtype, out_dim, in_dim, seed=9, tensor_id=qtype)
    i = np.arange(rows * in_dim, dtype=np.uint64)
    x = ((((i * 2654435761) % (1 << 32)) % 2000).astype(np.int64) - 1000) / np.float32(1000.0)
    x = x.astype(np.float32)
    bias = ((np.arange(out_dim) % 10) / np.float32(100.0)).astype(np.float32)
    mine = oracle.matmul_add(x, rows, in_dim, w, qtype, out_dim, bias)
    dense = oracle.dequantize(qtype, w, out_dim * in_dim).reshape(out_dim, in_dim).astype(np.float64)
    ref = (bias.astype(np.float64)[None, :] + x.reshape(rows, in_dim).astype(np.float64) @ dense.T)
    ref = ref.astype(np.float32).ravel()
    cos = float(mine.astype(np.float64) @ ref.astype(np.float64) /
                (np.linalg.norm(mine.astype(np.float64)) * np.linalg.norm(ref.astype(np.float64))))
    assert cos >= 0.9999999
    assert np.abs(mine - ref).max() / np.abs(ref).max() <= 1e-5


def test_range_variant_touches_only_its_rows(oracle):
    w = synth.make_weight(Q4_K, 40, 512, seed=2)
    x = synth.make_activation(1, 512, seed=2)
    z = np.zeros(40, np.float32)
    full = oracle.matmul_add(x, 1, 512, w, Q4_K, 40, z)
    part = oracle.matmul_add(x, 1, 512, w, Q4_K, 40, z, o_begin=10, o_end=25)
    assert np.array_equal(part[10:25], full[10:25])
    assert not part[:10].any() and not part[25:].any()


def test_unsupported_type_raises(oracle):
    with pytest.raises(ValueError, match="Unsupported quant type"):
        oracle.matmul_add(np.zeros(32, np.float32), 1, 32, np.zeros(64, np.uint8), 2, 1,
                          np.zeros(1, np.float32))
    with pytest.raises(ValueError, match="Unsupported dequantization type"):
        oracle.dequantize(2, np.zeros(64, np.uint8), 32)


def test_top1_highest_value_lowest_index(oracle):
    """qwen35_cpu.cr:2052-2055: max, then the first index holding it."""
    assert oracle.top1(np.array([1.0, 5.0, 5.0, -2.0], np.float32)) == (1, np.float32(5.0))
    assert oracle.top1(np.array([-3.0, -3.0], np.float32)) == (0, np.float32(-3.0))
    assert oracle.top1(np.array([0.0, -0.0, 0.0], np.float32))[0] == 0


def test_swiglu_restatements_agree_and_known_values():
    """silu(v) = v / (1 + exp(-v)) (qwen35_cpu.cr:517-519): silu(0) = 0, silu(v) -> v for large v,
    silu(-v) = -v * (1 - sigmoid(v)); C and numpy restatements agree to the last bit or ulp."""
    from oracle import loader, oracle_np
    g = np.array([0.0, 1.0, -1.0, 20.0, -20.0, 0.5, 88.0, -88.0], dtype=np.float32)
    u = np.array([3.0, 2.0, 2.0, 1.0, 1.0, -4.0, 1.0, 1.0], dtype=np.float32)
    c = loader.swiglu(g, u)
    n = oracle_np.swiglu(g, u)
    assert c[0] == 0.0 and abs(c[1] - 2.0 * 0.7310586) < 1e-6 and abs(c[2] + 2.0 * 0.26894143) < 1e-6
    assert abs(c[3] - 20.0) < 1e-5 and abs(c[4]) < 1e-6 and c[6] == 88.0 and abs(c[7]) < 1e-30
    assert np.allclose(c, n, rtol=3e-7, atol=1e-30)
    rng = np.random.default_rng(0)
    g = (rng.standard_normal(4096) * 4).astype(np.float32)
    u = rng.standard_normal(4096).astype(np.float32)
    assert np.allclose(loader.swiglu(g, u), oracle_np.swiglu(g, u), rtol=3e-7, atol=1e-12)


def test_rmsnorm_restatements_agree_and_known_values():
    """rms_norm (qwen35_cpu.cr:484-490): a row of equal values v normalises to w * v / sqrt(v^2 + eps);
    the C and numpy restatements agree bit for bit."""
    from oracle import loader, oracle_np
    w = np.array([1.0, 2.0, -1.0, 0.5], dtype=np.float32)
    x = np.array([[2.0, 2.0, 2.0, 2.0], [0.0, 0.0, 0.0, 0.0], [3.0, -4.0, 0.0, 0.0]], dtype=np.float32)
    c = loader.rmsnorm(x, w, 1e-6)
    inv0 = np.float32(1.0 / np.sqrt(4.0 + 1e-6))
    assert np.array_equal(c[0], (np.float32(2.0) * inv0) * w) and not c[1].any()
    inv2 = np.float32(1.0 / np.sqrt(25.0 / 4.0 + np.float64(np.float32(1e-6))))
    assert np.array_equal(c[2], (x[2] * inv2) * w)
    rng = np.random.default_rng(1)
    x = (rng.standard_normal((5, 1536)) * 7).astype(np.float32)
    w = rng.standard_normal(1536).astype(np.float32)
    assert np.array_equal(loader.rmsnorm(x, w, 1e-6), oracle_np.rmsnorm(x, w, 1e-6))
