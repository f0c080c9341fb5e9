"""Second, independent restatement of the reference's CPU arithmetic in vectorised numpy.
TEST INFRASTRUCTURE ONLY: it cross-checks the C oracle (two implementations written
separately from the same reference lines must agree), it is never on the product path.

Bulk dequantisation is all-f32 (src/ml/gguf/dequant.cr); weight values for the fused matmul
are f64 (src/ml/gguf/quant_matmul.cr).  `weights64` returns the f64 weight matrix the fused
matmul multiplies by, so `bias + x @ W.T` in f64 is the reference result up to summation order.
"""
from __future__ import annotations

import numpy as np

Q8_0, Q4_K, Q5_K, Q6_K = 8, 12, 13, 14
_BB = {Q8_0: 34, Q4_K: 144, Q5_K: 176, Q6_K: 210}
_BE = {Q8_0: 32, Q4_K: 256, Q5_K: 256, Q6_K: 256}


def _half(col: np.ndarray, ft) -> np.ndarray:
    """little-endian f16 bytes [n, 2] -> ft (numpy's conversion is exact, subnormals included)."""
    return np.ascontiguousarray(col).view(np.float16).reshape(-1).astype(ft)


def _scale_min_k4(s: np.ndarray):
    """dequant.cr:240-249 for all j at once: s uint8 [n, 12] -> (sc, m) int [n, 8]."""
    s = s.astype(np.int32)
    sc = np.empty((s.shape[0], 8), dtype=np.int32)
    m = np.empty_like(sc)
    sc[:, :4] = s[:, 0:4] & 63
    m[:, :4] = s[:, 4:8] & 63
    sc[:, 4:] = (s[:, 8:12] & 0x0F) | ((s[:, 0:4] >> 6) << 4)
    m[:, 4:] = (s[:, 8:12] >> 4) | ((s[:, 4:8] >> 6) << 4)
    return sc, m


def _quants(qtype: int, blk: np.ndarray) -> np.ndarray:
    """Integer quants in element order, int32 [n, block_elems] (Q6_K already minus 32)."""
    n = blk.shape[0]
    if qtype == Q8_0:
        return blk[:, 2:34].view(np.int8).astype(np.int32)
    if qtype in (Q4_K, Q5_K):
        ql = blk[:, 16:144] if qtype == Q4_K else blk[:, 48:176]
        ql = ql.reshape(n, 4, 32).astype(np.int32)
        lo, hi = ql & 0x0F, ql >> 4
        if qtype == Q5_K:
            qh = blk[:, 16:48].astype(np.int32)[:, None, :]          # [n, 1, 32]
            pair = np.arange(4, dtype=np.int32)[None, :, None]       # [1, 4, 1]
            lo = lo + (((qh >> (2 * pair)) & 1) << 4)
            hi = hi + (((qh >> (2 * pair + 1)) & 1) << 4)
        return np.stack([lo, hi], axis=2).reshape(n, 256)           # pair, (lo|hi), l
    if qtype == Q6_K:
        ql = blk[:, 0:128].reshape(n, 2, 64).astype(np.int32)
        qh = blk[:, 128:192].reshape(n, 2, 32).astype(np.int32)
        a, b = ql[:, :, :32], ql[:, :, 32:]
        q1 = (a & 0xF) | (((qh >> 0) & 3) << 4)
        q2 = (b & 0xF) | (((qh >> 2) & 3) << 4)
        q3 = (a >> 4) | (((qh >> 4) & 3) << 4)
        q4 = (b >> 4) | (((qh >> 6) & 3) << 4)
        return (np.stack([q1, q2, q3, q4], axis=2) - 32).reshape(n, 256)
    raise ValueError(qtype)


def _weights(qtype: int, raw: np.ndarray, n: int, ft) -> np.ndarray:
    blk = np.ascontiguousarray(raw, dtype=np.uint8)[: n // _BE[qtype] * _BB[qtype]]
    blk = blk.reshape(-1, _BB[qtype])
    q = _quants(qtype, blk).astype(ft)
    if qtype == Q8_0:
        w = _half(blk[:, 0:2], ft)[:, None] * q
    elif qtype in (Q4_K, Q5_K):
        d, dmin = _half(blk[:, 0:2], ft), _half(blk[:, 2:4], ft)
        sc, m = _scale_min_k4(blk[:, 4:16])
        d1 = (d[:, None] * sc.astype(ft)).astype(ft)                 # [n, 8]
        m1 = (dmin[:, None] * m.astype(ft)).astype(ft)
        w = (np.repeat(d1, 32, axis=1) * q).astype(ft) - np.repeat(m1, 32, axis=1)
    else:  # Q6_K: scale index 8*half + l//16 + 2*k for output l + 32k of each 128-half
        d = _half(blk[:, 208:210], ft)
        sc = blk[:, 192:208].view(np.int8).astype(ft)                # [n, 16]
        ds = (d[:, None] * sc).astype(ft)
        w = (np.repeat(ds, 16, axis=1) * q).astype(ft)
    return w.astype(ft).reshape(-1)


def dequantize(qtype: int, raw: np.ndarray, n: int) -> np.ndarray:
    """Dequant.dequantize in f32 (dequant.cr:53-236)."""
    return _weights(qtype, raw, n, np.float32)


def weights64(qtype: int, raw: np.ndarray, out_dim: int, in_dim: int) -> np.ndarray:
    return _weights(qtype, raw, out_dim * in_dim, np.float64).reshape(out_dim, in_dim)


def matmul_add(x, rows, in_dim, w_raw, w_type, out_dim, bias) -> np.ndarray:
    """quant_matmul.cr:20-36 up to f64 summation order."""
    w = weights64(w_type, w_raw, out_dim, in_dim)
    x = np.asarray(x, dtype=np.float32).reshape(rows, in_dim).astype(np.float64)
    y = np.asarray(bias, dtype=np.float32).astype(np.float64)[None, :out_dim] + x @ w.T
    return y.astype(np.float32).reshape(-1)


def swiglu(gate, up) -> np.ndarray:
    """silu(gate) * up in f32, silu(v) = v / (1 + exp(-v)) (qwen35_cpu.cr:512-519, 1716-1717)."""
    g = np.asarray(gate, dtype=np.float32)
    u = np.asarray(up, dtype=np.float32)
    s = g / (np.float32(1.0) + np.exp(-g, dtype=np.float32))
    return (s * u).astype(np.float32)


def rmsnorm(x, w, eps=1.0e-6) -> np.ndarray:
    """x * inv_rms * w per row, sum of squares in f64 (qwen35_cpu.cr:484-490)."""
    w = np.asarray(w, dtype=np.float32).reshape(-1)
    x = np.asarray(x, dtype=np.float32).reshape(-1, w.size)
    ss = (x.astype(np.float64) ** 2).sum(axis=1)
    inv = (1.0 / np.sqrt(ss / x.shape[1] + np.float64(np.float32(eps)))).astype(np.float32)
    return ((x * inv[:, None]).astype(np.float32) * w[None, :]).astype(np.float32)
