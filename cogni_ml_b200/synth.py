"""Seeded synthetic GGUF tensors with the shapes, block layouts and value distributions of the
benchmark configurations (they stand in for the Qwen3.5-9B / 27B model tensors the reference
measures on, which are not redistributable test inputs).

Everything is generated with numpy's counter-based Philox generator keyed by
(seed, tensor_id), so any process regenerates identical bytes.

Per block (offsets as in src/ml/gguf/dequant.cr):
  Q8_0  d = half(|N(0,0.02)|/127), 32 quants uniform int8 in [-127,127]
  Q4_K  d = half(|N(0,0.01)|), dmin = half(|N(0,0.01)|), 8 (scale,min) pairs uniform [0,63]
        packed the way get_scale_min_k4 unpacks them, 128 B uniform nibbles
  Q5_K  as Q4_K plus a uniform 32 B fifth-bit plane
  Q6_K  128 B ql + 64 B qh uniform, 16 int8 scales uniform [-64,63], d = half(|N(0,0.001)|)
  IQ4_NL d = half(|N(0,0.02)|/127), 16 B uniform nibbles (indices into the 16-level table)
Activations are f32 N(0,1).
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 8, 12, 13, 14, 20
BLOCK_BYTES = {Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210, IQ4_NL: 18}
BLOCK_ELEMS = {Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256, IQ4_NL: 32}
TYPE_NAMES = {Q8_0: "Q8_0", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K", IQ4_NL: "IQ4_NL"}


def row_bytes(qtype: int, in_dim: int) -> int:
    if in_dim % BLOCK_ELEMS[qtype]:
        raise ValueError(f"in_dim {in_dim} is not a multiple of the {TYPE_NAMES[qtype]} block")
    return in_dim // BLOCK_ELEMS[qtype] * BLOCK_BYTES[qtype]


def tensor_bytes(qtype: int, out_dim: int, in_dim: int) -> int:
    return out_dim * row_bytes(qtype, in_dim)


def _rng(seed: int, tensor_id: int) -> np.random.Generator:
    return np.random.Generator(np.random.Philox(key=[np.uint64(seed), np.uint64(tensor_id)]))


def pack_scales_k4(sc: np.ndarray, mn: np.ndarray) -> np.ndarray:
    """Inverse of get_scale_min_k4 (dequant.cr:240-249): sc, mn uint8 [n, 8] in [0,63] -> [n, 12]."""
    sc = sc.astype(np.uint8)
    mn = mn.astype(np.uint8)
    out = np.zeros((sc.shape[0], 12), dtype=np.uint8)
    out[:, 0:4] = (sc[:, 0:4] & 63) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 63) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def _half_bytes(values: np.ndarray) -> np.ndarray:
    return values.astype(np.float16).view(np.uint8).reshape(-1, 2)


def _blocks(qtype: int, nb: int, rng: np.random.Generator) -> np.ndarray:
    out = np.empty((nb, BLOCK_BYTES[qtype]), dtype=np.uint8)
    if qtype == Q8_0:
        out[:, 0:2] = _half_bytes(np.abs(rng.normal(0.0, 0.02, nb)) / 127.0)
        out[:, 2:34] = rng.integers(-127, 128, size=(nb, 32), dtype=np.int8).view(np.uint8)
    elif qtype == IQ4_NL:
        out[:, 0:2] = _half_bytes(np.abs(rng.normal(0.0, 0.02, nb)) / 127.0)
        out[:, 2:18] = rng.integers(0, 256, size=(nb, 16), dtype=np.uint8)
    elif qtype in (Q4_K, Q5_K):
        out[:, 0:2] = _half_bytes(np.abs(rng.normal(0.0, 0.01, nb)))
        out[:, 2:4] = _half_bytes(np.abs(rng.normal(0.0, 0.01, nb)))
        sc = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
        mn = rng.integers(0, 64, size=(nb, 8), dtype=np.uint8)
        out[:, 4:16] = pack_scales_k4(sc, mn)
        out[:, 16:] = rng.integers(0, 256, size=(nb, BLOCK_BYTES[qtype] - 16), dtype=np.uint8)
    elif qtype == Q6_K:
        out[:, 0:192] = rng.integers(0, 256, size=(nb, 192), dtype=np.uint8)
        out[:, 192:208] = rng.integers(-64, 64, size=(nb, 16), dtype=np.int8).view(np.uint8)
        out[:, 208:210] = _half_bytes(np.abs(rng.normal(0.0, 0.001, nb)))
    else:
        raise ValueError(f"unsupported tensor type {qtype}")
    return out


def make_weight(qtype: int, out_dim: int, in_dim: int, seed: int = 0, tensor_id: int = 0,
                rows_per_chunk: int = 4096) -> np.ndarray:
    """Raw GGUF bytes of an [out_dim, in_dim] weight, flat uint8 array (row-major rows of blocks)."""
    bpr = in_dim // BLOCK_ELEMS[qtype]
    rb = row_bytes(qtype, in_dim)
    rng = _rng(seed, tensor_id)
    out = np.empty(out_dim * rb, dtype=np.uint8)
    for r0 in range(0, out_dim, rows_per_chunk):
        r1 = min(out_dim, r0 + rows_per_chunk)
        out[r0 * rb:r1 * rb] = _blocks(qtype, (r1 - r0) * bpr, rng).reshape(-1)
    return out


def make_activation(batch: int, in_dim: int, seed: int = 0, tensor_id: int = 1000) -> np.ndarray:
    """f32 N(0,1) activations [batch, in_dim]."""
    return _rng(seed, tensor_id).standard_normal((batch, in_dim), dtype=np.float32)
