"""Host-side mirror of the reference's quantized-matmul call surface, running on the CUDA engine.

Names and argument meaning follow the reference so that parity tests read like its own specs:

  TensorType                       src/ml/gguf/reader.cr:36-96
  QuantWeight                      src/ml/gguf/compute.cr:20-45  (raw bytes + type + dims)
  QuantMatmul.matmul_add           src/ml/gguf/quant_matmul.cr:20-36 (host arrays in, host array out)
  DeviceQuantWeight                the resident form: raw GGUF bytes uploaded verbatim once
                                   (as QwenRecurrentLayerRunner#upload_weights does,
                                   src/ml/cuda/qwen_recurrent_layer_runner.cr:570-587), then
                                   gemv / gemv_top1 / gemm / dequantize on device buffers.

Every compute call goes through the C ABI in include/cogni_qmm.h.  torch is used only to own
device memory and streams.  There is no CPU path here: without the shared library the import
fails, without a GPU the calls raise.
"""
from __future__ import annotations

import enum
import warnings
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import check, lib


class TensorType(enum.IntEnum):
    """ggml tensor types handled by this engine (ids as in reader.cr:36-50)."""

    Q8_0 = 8
    Q4_K = 12
    Q5_K = 13
    Q6_K = 14
    IQ4_NL = 20  # dequantize, embedding lookup and the general GEMV; no tiled kernel

    @property
    def block_bytes(self) -> int:
        return lib.cogni_qmm_block_bytes(int(self))

    @property
    def block_elements(self) -> int:
        return lib.cogni_qmm_block_elements(int(self))


def row_bytes(w_type: int, in_dim: int) -> int:
    rb = lib.cogni_qmm_row_bytes(int(w_type), in_dim)
    if rb < 0:
        raise ValueError(f"unsupported tensor type {w_type} or in_dim {in_dim} not a block multiple")
    return rb


@dataclass
class QuantWeight:
    """Raw bytes + type + dims, as ML::GGUF::QuantWeight (compute.cr:20-45)."""

    raw: np.ndarray  # flat uint8, out_dim rows of in_dim/block_elements blocks
    type: int
    out_dim: int
    in_dim: int
    route_tag: Optional[str] = None

    def __post_init__(self):
        self.raw = np.ascontiguousarray(self.raw, dtype=np.uint8).reshape(-1)
        need = row_bytes(self.type, self.in_dim) * self.out_dim
        if self.raw.size < need:
            raise ValueError(f"raw holds {self.raw.size} bytes, {need} needed")


def _stream_ptr(stream: Optional[torch.cuda.Stream]) -> int:
    return (stream or torch.cuda.current_stream()).cuda_stream


def _require_cuda() -> None:
    if not torch.cuda.is_available():
        raise RuntimeError("cogni_ml_b200 needs a CUDA device (sm_100a); there is no CPU fallback")


class QuantMatmul:
    """Drop-in for ML::GGUF::QuantMatmul (quant_matmul.cr:13-36)."""

    @staticmethod
    def matmul_add(x, rows: int, in_dim: int, w_raw, w_type: int, out_dim: int, bias) -> np.ndarray:
        """result[r, o] = bias[o] + sum_j x[r, j] * dequant(W[o, j]); host arrays in and out.

        Unsupported types raise, as the reference does ("Unsupported quant type for fused matmul").
        """
        _require_cuda()
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1)
        w = np.ascontiguousarray(w_raw, dtype=np.uint8).reshape(-1)
        b = np.ascontiguousarray(bias, dtype=np.float32).reshape(-1)
        if x.size < rows * in_dim or b.size < out_dim:
            raise ValueError("x or bias shorter than rows*in_dim / out_dim")
        y = np.empty(rows * out_dim, dtype=np.float32)
        check(lib.cogni_qmm_matmul_add_host(x.ctypes.data, rows, in_dim, w.ctypes.data, w.size,
                                            int(w_type), out_dim, b.ctypes.data, y.ctypes.data),
              "cogni_qmm_matmul_add_host")
        return y


class DeviceQuantWeight:
    """A quantized weight resident in HBM: the verbatim GGUF bytes of rows [row_begin, row_end)."""

    def __init__(self, raw_dev: torch.Tensor, w_type: int, out_dim: int, in_dim: int,
                 row_begin: int = 0):
        self.raw = raw_dev
        self.type = int(w_type)
        self.out_dim = out_dim      # rows held by THIS buffer
        self.in_dim = in_dim
        self.row_begin = row_begin  # global index of the first row (vocab/row sharding)
        # True once the bytes are known to be complete on the device: gemv may then overlap its
        # weight fetch with the tail of the preceding kernel (cogni_qmm_gemv_resident)
        self.resident = False
        self._top1_scratch: Optional[torch.Tensor] = None

    @classmethod
    def upload(cls, qw: QuantWeight, device="cuda", row_begin: int = 0,
               row_end: Optional[int] = None) -> "DeviceQuantWeight":
        """Copies rows [row_begin, row_end) of the raw tensor to the device, unmodified."""
        _require_cuda()
        row_end = qw.out_dim if row_end is None else row_end
        rb = row_bytes(qw.type, qw.in_dim)
        with warnings.catch_warnings():
            # a read-only mmap slice is fine here: the tensor is only ever the source of a copy
            warnings.filterwarnings("ignore", message="The given NumPy array is not writable")
            host = torch.from_numpy(qw.raw[row_begin * rb:row_end * rb])
        dev = torch.empty(host.numel(), dtype=torch.uint8, device=device)
        dev.copy_(host)
        torch.cuda.current_stream(dev.device).synchronize()
        out = cls(dev, qw.type, row_end - row_begin, qw.in_dim, row_begin)
        out.resident = True
        return out

    @property
    def nbytes(self) -> int:
        return self.raw.numel()

    def dequantize(self, stream=None) -> torch.Tensor:
        """f32 [out_dim, in_dim], bit-identical to Dequant.dequantize on the CPU."""
        out = torch.empty(self.out_dim, self.in_dim, dtype=torch.float32, device=self.raw.device)
        check(lib.cogni_qmm_dequantize(self.type, self.raw.data_ptr(), self.out_dim * self.in_dim,
                                       out.data_ptr(), _stream_ptr(stream)), "cogni_qmm_dequantize")
        return out

    def gemv(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
             bias: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
             stream=None) -> torch.Tensor:
        """y[b, :] = (bias | residual[b, :]) + W @ x[b, :], x f32 [batch, in_dim] on the device."""
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[-1] != self.in_dim:
            raise ValueError("x must be contiguous f32 [batch, in_dim]")
        batch = x.numel() // self.in_dim
        if out is None:
            out = torch.empty(batch, self.out_dim, dtype=torch.float32, device=x.device)
        if bias is not None and residual is not None:
            raise ValueError("pass bias or residual, not both")
        addend, stride = (bias, 0) if bias is not None else (residual, self.out_dim)
        fn = lib.cogni_qmm_gemv_resident if self.resident else lib.cogni_qmm_gemv
        check(fn(self.type, self.raw.data_ptr(), x.data_ptr(),
                 addend.data_ptr() if addend is not None else None, stride,
                 out.data_ptr(), self.in_dim, self.out_dim, batch, _stream_ptr(stream)),
              "cogni_qmm_gemv")
        return out

    def gemv_top2(self, x: torch.Tensor, stream=None, want_keys: bool = False):
        """The two best rows per batch row: (index int32 [batch, 2], value f32 [batch, 2][, key
        int64 [batch, 2]]); column 0 is the argmax with the reference's tie rule, column 1 the
        runner-up (the verifier's margin is value[:, 0] - value[:, 1])."""
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[-1] != self.in_dim:
            raise ValueError("x must be contiguous f32 [batch, in_dim]")
        batch = x.numel() // self.in_dim
        need = lib.cogni_qmm_gemv_top2_scratch_bytes(self.out_dim, batch)
        scratch = getattr(self, "_top2_scratch", None)
        if scratch is None or scratch.numel() < need:
            scratch = self._top2_scratch = torch.zeros(need, dtype=torch.uint8, device=self.raw.device)
        idx = torch.empty(batch, 2, dtype=torch.int32, device=x.device)
        val = torch.empty(batch, 2, dtype=torch.float32, device=x.device)
        key = torch.empty(batch, 2, dtype=torch.int64, device=x.device) if want_keys else None
        check(lib.cogni_qmm_gemv_top2(self.type, self.raw.data_ptr(), x.data_ptr(), self.in_dim,
                                      self.out_dim, batch, self.row_begin, scratch.data_ptr(),
                                      scratch.numel(), idx.data_ptr(), val.data_ptr(),
                                      key.data_ptr() if key is not None else None,
                                      1 if self.resident else 0, _stream_ptr(stream)),
              "cogni_qmm_gemv_top2")
        return (idx, val, key) if want_keys else (idx, val)

    def embedding_lookup(self, token_ids: torch.Tensor, out: Optional[torch.Tensor] = None,
                         check_range: bool = True, stream=None) -> torch.Tensor:
        """Rows `token_ids` (int32 on the device) of this [vocab, n_embd] table as f32, bit-identical
        to the CPU dequantiser (Qwen35CPU#embedding_lookup, qwen35_cpu.cr:3305-3332).  With
        check_range an id outside the table raises like the reference (this synchronises)."""
        if token_ids.dtype != torch.int32 or not token_ids.is_contiguous():
            raise ValueError("token_ids must be a contiguous int32 tensor")
        n = token_ids.numel()
        if out is None:
            out = torch.empty(n, self.in_dim, dtype=torch.float32, device=token_ids.device)
        status = torch.zeros(1, dtype=torch.int32, device=token_ids.device) if check_range else None
        check(lib.cogni_qmm_embedding_lookup(self.type, self.raw.data_ptr(), self.out_dim, self.in_dim,
                                             token_ids.data_ptr(), n, out.data_ptr(),
                                             status.data_ptr() if status is not None else None,
                                             _stream_ptr(stream)), "cogni_qmm_embedding_lookup")
        if status is not None:
            bad = int(status.item())
            if bad:
                raise IndexError(f"embedding: token_id {int(token_ids.view(-1)[bad - 1])} out of range")
        return out

    def gemv_swiglu(self, gate: torch.Tensor, up: torch.Tensor, out: Optional[torch.Tensor] = None,
                    residual: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
        """y[b, :] = residual[b, :] + W @ (silu(gate[b, :]) * up[b, :]): the FFN down projection with
        the SwiGLU product fused in (qwen35_cpu.cr:1716-1718).  gate, up f32 [batch, in_dim]."""
        for t in (gate, up):
            if t.dtype != torch.float32 or not t.is_contiguous() or t.shape[-1] != self.in_dim:
                raise ValueError("gate and up must be contiguous f32 [batch, in_dim]")
        batch = gate.numel() // self.in_dim
        if out is None:
            out = torch.empty(batch, self.out_dim, dtype=torch.float32, device=gate.device)
        # shapes the fused kernel does not take (and the diagnostic row-per-warp mode) need room
        # for the product; the buffer is kept with the weight
        scratch = getattr(self, "_swiglu_scratch", None)
        if scratch is None or scratch.numel() < gate.numel() or scratch.device != gate.device:
            scratch = self._swiglu_scratch = torch.empty(gate.numel(), dtype=torch.float32,
                                                         device=gate.device)
        check(lib.cogni_qmm_gemv_swiglu(self.type, self.raw.data_ptr(), gate.data_ptr(), up.data_ptr(),
                                        residual.data_ptr() if residual is not None else None,
                                        self.out_dim if residual is not None else 0, out.data_ptr(),
                                        scratch.data_ptr(),
                                        self.in_dim, self.out_dim, batch, 1 if self.resident else 0,
                                        _stream_ptr(stream)), "cogni_qmm_gemv_swiglu")
        return out

    def top1_scratch(self, batch: int) -> torch.Tensor:
        need = lib.cogni_qmm_gemv_top1_scratch_bytes(self.out_dim, batch)
        if self._top1_scratch is None or self._top1_scratch.numel() < need:
            self._top1_scratch = torch.zeros(need, dtype=torch.uint8, device=self.raw.device)
        return self._top1_scratch

    def gemv_top1(self, x: torch.Tensor, stream=None, want_keys: bool = False,
                  norm_weight: Optional[torch.Tensor] = None, eps: float = 1.0e-6):
        """Fused lm_head: returns (index int32 [batch], value f32 [batch][, key int64 [batch]]).

        Indices are global: row_begin is added on the device.  With norm_weight (f32 [in_dim]) the
        rows are RMS-normalised inside the launch first (output_norm -> lm_head -> argmax)."""
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[-1] != self.in_dim:
            raise ValueError("x must be contiguous f32 [batch, in_dim]")
        batch = x.numel() // self.in_dim
        scratch = self.top1_scratch(batch)
        idx = torch.empty(batch, dtype=torch.int32, device=x.device)
        val = torch.empty(batch, dtype=torch.float32, device=x.device)
        key = torch.empty(batch, dtype=torch.int64, device=x.device) if want_keys else None
        if norm_weight is not None:
            xs = torch.empty_like(x)   # for shapes the fused kernel does not take
            check(lib.cogni_qmm_gemv_top1_rmsnorm(self.type, self.raw.data_ptr(), x.data_ptr(),
                                                  norm_weight.data_ptr(), float(eps), self.in_dim,
                                                  self.out_dim, batch, self.row_begin,
                                                  scratch.data_ptr(), scratch.numel(), xs.data_ptr(),
                                                  idx.data_ptr(), val.data_ptr(),
                                                  key.data_ptr() if key is not None else None,
                                                  1 if self.resident else 0, _stream_ptr(stream)),
                  "cogni_qmm_gemv_top1_rmsnorm")
            return (idx, val, key) if want_keys else (idx, val)
        check(lib.cogni_qmm_gemv_top1(self.type, self.raw.data_ptr(), x.data_ptr(), self.in_dim,
                                      self.out_dim, batch, self.row_begin, scratch.data_ptr(),
                                      scratch.numel(), idx.data_ptr(), val.data_ptr(),
                                      key.data_ptr() if key is not None else None,
                                      _stream_ptr(stream)), "cogni_qmm_gemv_top1")
        return (idx, val, key) if want_keys else (idx, val)

    def gemm(self, x_bf16: torch.Tensor, out_dtype=torch.float32, out: Optional[torch.Tensor] = None,
             stream=None) -> torch.Tensor:
        """Prefill: y[m, n] = sum_k x[m, k] * bf16(dequant(W[n, k])), x bf16 [M, in_dim]."""
        if x_bf16.dtype != torch.bfloat16 or not x_bf16.is_contiguous() or \
                x_bf16.shape[-1] != self.in_dim:
            raise ValueError("x must be contiguous bf16 [M, in_dim]")
        m = x_bf16.numel() // self.in_dim
        if out is None:
            out = torch.empty(m, self.out_dim, dtype=out_dtype, device=x_bf16.device)
        code = {torch.float32: 0, torch.bfloat16: 1}[out.dtype]
        check(lib.cogni_qmm_gemm_bf16(self.type, self.raw.data_ptr(), x_bf16.data_ptr(),
                                      out.data_ptr(), code, m, self.out_dim, self.in_dim,
                                      _stream_ptr(stream)), "cogni_qmm_gemm_bf16")
        return out


class GemvMany:
    """A prepared qmatvec_many call: several resident weights of one type and in_dim against one
    x (src/ml/gguf/qwen35_cpu.cr:1419-1490).  The pointer tables are built once; `run` issues one
    launch."""

    def __init__(self, weights, x: torch.Tensor, outs, residuals=None, norm_weight=None,
                 eps: float = 1.0e-6):
        """norm_weight (f32 [in_dim] on the device): the matrices see RMSNorm(x) * norm_weight,
        normalised inside the launch (Qwen35CPU#rms_norm, qwen35_cpu.cr:484-490)."""
        import ctypes as C
        self.norm_weight, self.eps, self._scratch = norm_weight, float(eps), None
        if norm_weight is not None:
            if norm_weight.dtype != torch.float32 or norm_weight.numel() != weights[0].in_dim:
                raise ValueError("norm_weight must be f32 [in_dim]")
            # room for the normalised x, for shapes the fused kernel does not take
            self._scratch = torch.empty_like(x)
        if not weights or len({(w.type, w.in_dim) for w in weights}) != 1:
            raise ValueError("weights must share type and in_dim")
        self.weights, self.x, self.outs = list(weights), x, list(outs)
        n = len(self.weights)
        w0 = self.weights[0]
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[-1] != w0.in_dim:
            raise ValueError("x must be contiguous f32 [batch, in_dim]")
        self.batch = x.numel() // w0.in_dim
        self._w = (C.c_void_p * n)(*[w.raw.data_ptr() for w in self.weights])
        self._y = (C.c_void_p * n)(*[o.data_ptr() for o in self.outs])
        self._n = (C.c_int * n)(*[w.out_dim for w in self.weights])
        self._add = None
        self._stride = 0
        if residuals is not None:
            self.residuals = list(residuals)
            self._add = (C.c_void_p * n)(*[r.data_ptr() if r is not None else None
                                           for r in self.residuals])
            self._stride = -1   # per matrix: out_dim; checked below
            if len({w.out_dim for w in self.weights}) != 1:
                raise ValueError("residuals need equal out_dim across the weights")
            self._stride = self.weights[0].out_dim
        self._resident = int(all(w.resident for w in self.weights))

    def run(self, stream=None):
        w0 = self.weights[0]
        if self.norm_weight is not None:
            check(lib.cogni_qmm_gemv_many_rmsnorm(w0.type, len(self.weights), self._w,
                                                  self.x.data_ptr(), self.norm_weight.data_ptr(),
                                                  self.eps, self._add, self._stride, self._y,
                                                  self._n, self._scratch.data_ptr(), w0.in_dim,
                                                  self.batch, self._resident, _stream_ptr(stream)),
                  "cogni_qmm_gemv_many_rmsnorm")
            return self.outs
        check(lib.cogni_qmm_gemv_many(w0.type, len(self.weights), self._w, self.x.data_ptr(),
                                      self._add, self._stride, self._y, self._n, w0.in_dim,
                                      self.batch, self._resident, _stream_ptr(stream)),
              "cogni_qmm_gemv_many")
        return self.outs


def gemv_many(weights, x: torch.Tensor, outs=None, stream=None, norm_weight=None, eps: float = 1.0e-6):
    """y_j = W_j @ x (or W_j @ (RMSNorm(x) * norm_weight)) for several weights sharing x, in one
    launch."""
    batch = x.numel() // weights[0].in_dim
    if outs is None:
        outs = [torch.empty(batch, w.out_dim, dtype=torch.float32, device=x.device) for w in weights]
    return GemvMany(weights, x, outs, norm_weight=norm_weight, eps=eps).run(stream)


def unpack_top1_keys(keys: torch.Tensor):
    """(index int32, value f32) from int64 keys, e.g. after a MAX all-reduce across vocab shards."""
    batch = keys.numel()
    idx = torch.empty(batch, dtype=torch.int32, device=keys.device)
    val = torch.empty(batch, dtype=torch.float32, device=keys.device)
    check(lib.cogni_qmm_top1_unpack_keys(keys.data_ptr(), batch, idx.data_ptr(), val.data_ptr(),
                                         _stream_ptr(None)), "cogni_qmm_top1_unpack_keys")
    return idx, val
