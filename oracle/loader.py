"""ctypes access to the C oracle (oracle/qmm_oracle.c).  TEST INFRASTRUCTURE ONLY.

Builds libqmm_oracle.so with gcc on first use.  Only tests, the smoke check and the
CPU-baseline legs of the benchmark import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "libqmm_oracle.so"

Q8_0, Q4_K, Q5_K, Q6_K, IQ4_NL = 8, 12, 13, 14, 20


def build(force: bool = False) -> Path:
    src = [HERE / "qmm_oracle.c", HERE / "qmm_oracle.h"]
    if force or not LIB.exists() or max(p.stat().st_mtime for p in src) > LIB.stat().st_mtime:
        env = {k: v for k, v in os.environ.items() if k not in ("CC", "CXX")}
        subprocess.run(["make", "-C", str(HERE), "-B", "libqmm_oracle.so"], check=True, env=env,
                       capture_output=True)
    return LIB


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(str(LIB))
        vp, i, i64 = C.c_void_p, C.c_int, C.c_int64
        L.qmm_oracle_block_bytes.argtypes = [i]
        L.qmm_oracle_block_elements.argtypes = [i]
        L.qmm_oracle_row_bytes.restype = i64
        L.qmm_oracle_row_bytes.argtypes = [i, i]
        L.qmm_oracle_fp16_to_f32.restype = C.c_float
        L.qmm_oracle_fp16_to_f32.argtypes = [C.c_uint16]
        L.qmm_oracle_get_scale_min_k4.argtypes = [i, vp, vp, vp]
        L.qmm_oracle_dequantize.argtypes = [i, vp, i64, vp]
        L.qmm_oracle_matmul_add.argtypes = [i, vp, i, i, vp, i, vp, vp]
        L.qmm_oracle_matmul_add_mt.argtypes = [i, vp, i, i, vp, i, vp, vp, i]
        L.qmm_oracle_matmul_add_range.argtypes = [i, vp, i, i, vp, i, vp, vp, i, i, i]
        L.qmm_oracle_top1.argtypes = [vp, i64, vp, vp]
        _lib = L
    return _lib


def row_bytes(qtype: int, in_dim: int) -> int:
    return lib().qmm_oracle_row_bytes(qtype, in_dim)


def fp16_to_f32(h: int) -> np.float32:
    return np.float32(lib().qmm_oracle_fp16_to_f32(h))


def get_scale_min_k4(j: int, scales: np.ndarray):
    s = np.ascontiguousarray(scales, dtype=np.uint8)
    sc, m = C.c_float(), C.c_float()
    lib().qmm_oracle_get_scale_min_k4(j, s.ctypes.data, C.byref(sc), C.byref(m))
    return sc.value, m.value


def dequantize(qtype: int, raw: np.ndarray, n: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8)
    out = np.zeros(n, dtype=np.float32)
    if lib().qmm_oracle_dequantize(qtype, raw.ctypes.data, n, out.ctypes.data) != 0:
        raise ValueError(f"Unsupported dequantization type: {qtype}")
    return out


def matmul_add(x, rows: int, in_dim: int, w_raw, w_type: int, out_dim: int, bias,
               threads: int = 1, o_begin: int = 0, o_end: int | None = None) -> np.ndarray:
    """QuantMatmul.matmul_add; with o_begin/o_end only that row range of W is evaluated
    (other outputs stay 0)."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
    w = np.ascontiguousarray(w_raw, dtype=np.uint8).reshape(-1)
    b = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
    assert x.size >= rows * in_dim and b.size >= out_dim
    assert w.size >= out_dim * row_bytes(w_type, in_dim)
    y = np.zeros(rows * out_dim, dtype=np.float32)
    o_end = out_dim if o_end is None else o_end
    rc = lib().qmm_oracle_matmul_add_range(w_type, x.ctypes.data, rows, in_dim, w.ctypes.data,
                                           out_dim, b.ctypes.data, y.ctypes.data, o_begin, o_end,
                                           threads)
    if rc != 0:
        raise ValueError(f"Unsupported quant type for fused matmul: {w_type}")
    return y


def top1(logits: np.ndarray):
    v = np.ascontiguousarray(logits, dtype=np.float32).reshape(-1)
    idx, val = C.c_int32(), C.c_float()
    lib().qmm_oracle_top1(v.ctypes.data, v.size, C.byref(idx), C.byref(val))
    return idx.value, np.float32(val.value)


def swiglu(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    """silu(gate) * up in f32 (qwen35_cpu.cr:512-519, 1716-1717)."""
    g = np.ascontiguousarray(gate, dtype=np.float32).reshape(-1)
    u = np.ascontiguousarray(up, dtype=np.float32).reshape(-1)
    out = np.empty_like(g)
    L = lib()
    L.qmm_oracle_swiglu.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]
    L.qmm_oracle_swiglu.restype = None
    L.qmm_oracle_swiglu(g.ctypes.data, u.ctypes.data, g.size, out.ctypes.data)
    return out


def rmsnorm(x: np.ndarray, w: np.ndarray, eps: float = 1.0e-6) -> np.ndarray:
    """Rows of x normalised as Qwen35CPU#rms_norm does (qwen35_cpu.cr:484-490)."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, w.size)
    out = np.empty_like(x)
    L = lib()
    L.qmm_oracle_rmsnorm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_float, C.c_void_p]
    L.qmm_oracle_rmsnorm.restype = None
    L.qmm_oracle_rmsnorm(x.ctypes.data, x.shape[0], x.shape[1], w.ctypes.data, eps, out.ctypes.data)
    return out


def max_threads() -> int:
    return lib().qmm_oracle_max_threads()
