"""Name -> weight maps for a Qwen3.5-shaped GGUF model on the device, with the reference's checks.

  GGUFTensor            what the reference's reader hands out per tensor: name, ggml type, dims
                        ([in_dim, out_dim], GGUF order) and the raw bytes, a slice of the mmap
                        (src/ml/gguf/reader.cr:119-127, 169-194)
  load_qw               tensor -> QuantWeight with the reference's conventions
                        (Qwen35Weights#load_qw, src/ml/gguf/qwen35_weights.cr:201-212)
  RecurrentLayerWeights the quantized projections of one recurrent layer with the type and shape
                        validation of QwenRecurrentLayerRunner::Weights.load
                        (src/ml/cuda/qwen_recurrent_layer_runner.cr:51-118), same error texts
  Qwen35DeviceWeights   every quantized projection of the model uploaded once (raw bytes verbatim,
                        optionally this rank's row shard), looked up by tensor name; keeps the
                        object that backs the host bytes alive and releases everything in an
                        idempotent, mutex-guarded close() (qwen35_weights.cr:80-90, 147-160;
                        spec/qwen35_weights_lifecycle_spec.cr:31-41)

The GGUF container itself (header, key/values, tensor directory) is parsed by the host runtime;
this module starts at the tensor directory it produces.
"""
from __future__ import annotations

import threading
from dataclasses import dataclass
from typing import Callable, Dict, Mapping, Optional, Sequence

import numpy as np

from .quant_matmul import QuantWeight, TensorType


@dataclass
class GGUFTensor:
    name: str
    type: int
    dims: Sequence[int]        # GGUF order: dims[0] = in_dim, dims[1] = out_dim (rows)
    raw: np.ndarray            # flat uint8 view of the tensor's bytes


def load_qw(tensors: Mapping[str, GGUFTensor], name: str, prefix: str = "qwen35") -> QuantWeight:
    info = tensors.get(name)
    if info is None:
        raise KeyError(f"qwen35_weights: missing tensor {name!r}")
    in_dim = int(info.dims[0])
    out_dim = int(info.dims[1]) if len(info.dims) >= 2 else 1
    return QuantWeight(info.raw, int(info.type), out_dim, in_dim, f"{prefix}:{name}")


# quantized projections of a recurrent (DeltaNet) layer, in the reference's field order
RECURRENT_PROJECTIONS = ("attn_qkv", "attn_gate", "ssm_alpha", "ssm_beta", "ssm_out", "ffn_gate",
                         "ffn_up", "ffn_down")
FULL_ATTN_PROJECTIONS = ("attn_q", "attn_k", "attn_v", "attn_output", "ffn_gate", "ffn_up", "ffn_down")


@dataclass
class RecurrentLayerWeights:
    """QwenRecurrentLayerRunner::Weights, the part that belongs to the quantized matmul path."""

    hidden: int
    ffn_dim: int
    out_dim: int
    qkv_dim: int
    inner_dim: int
    h_v: int
    weights: Dict[str, QuantWeight]
    ffn_down_type: int

    @classmethod
    def load(cls, tensors: Mapping[str, GGUFTensor], layer: int) -> "RecurrentLayerWeights":
        h_k, h_v, s = 16, 32, 128
        q_dim, v_dim = h_k * s, h_v * s
        qkv_dim, inner_dim = 2 * q_dim + v_dim, v_dim
        prefix = f"blk.{layer}"

        def need(suffix):
            info = tensors.get(f"{prefix}.{suffix}")
            if info is None:
                raise ValueError(f"missing {prefix}.{suffix}")
            return info

        qkv, gate = need("attn_qkv.weight"), need("attn_gate.weight")
        alpha, beta = need("ssm_alpha.weight"), need("ssm_beta.weight")
        out = need("ssm_out.weight")
        ffn_gate, ffn_up, ffn_down = need("ffn_gate.weight"), need("ffn_up.weight"), need("ffn_down.weight")
        T = TensorType
        if qkv.type != T.Q5_K:
            raise ValueError("expected Q5_K attn_qkv")
        if not (gate.type == T.Q4_K and alpha.type == T.Q4_K and beta.type == T.Q4_K):
            raise ValueError("expected Q4_K gate/alpha/beta")
        if out.type != T.Q4_K:
            raise ValueError("expected Q4_K ssm_out")
        if not (ffn_gate.type == T.Q4_K and ffn_up.type == T.Q4_K and ffn_down.type in (T.Q4_K, T.Q6_K)):
            raise ValueError("expected Q4_K ffn gate/up and Q4_K/Q6_K ffn down")
        hidden, ffn_dim = int(qkv.dims[0]), int(ffn_gate.dims[1])
        if int(qkv.dims[1]) != qkv_dim:
            raise ValueError("attn_qkv shape mismatch")
        if not (int(gate.dims[0]) == hidden and int(gate.dims[1]) == inner_dim):
            raise ValueError("attn_gate shape mismatch")
        if not (int(alpha.dims[0]) == hidden and int(alpha.dims[1]) == h_v and
                int(beta.dims[0]) == hidden and int(beta.dims[1]) == h_v):
            raise ValueError("ssm_alpha/beta shape mismatch")
        if int(out.dims[0]) != inner_dim:
            raise ValueError("ssm_out input mismatch")
        if not (int(ffn_gate.dims[0]) == hidden and int(ffn_up.dims[0]) == hidden and
                int(ffn_up.dims[1]) == ffn_dim and int(ffn_down.dims[0]) == ffn_dim and
                int(ffn_down.dims[1]) == hidden):
            raise ValueError("ffn shape mismatch")
        weights = {name: load_qw(tensors, f"{prefix}.{name}.weight") for name in RECURRENT_PROJECTIONS}
        return cls(hidden, ffn_dim, int(out.dims[1]), qkv_dim, inner_dim, h_v, weights, int(ffn_down.type))


class Qwen35DeviceWeights:
    """Every quantized projection of the model resident on the device, by tensor name.

    `backing` is whatever keeps the host bytes valid (the reference keeps its GGUFFile, i.e. the
    mmap, as a field for the same reason); it is closed -- if it has a close() -- after the device
    buffers are dropped.  close() may be called any number of times, from any number of threads."""

    def __init__(self, tensors: Mapping[str, GGUFTensor], device, names: Optional[Sequence[str]] = None,
                 backing=None, rank: int = 0, world: int = 1,
                 upload: Optional[Callable] = None):
        from .quant_matmul import DeviceQuantWeight
        from .sharded import shard_rows
        self._lock = threading.Lock()
        self._closed = False
        self._backing = backing
        self.device = device
        self.rank, self.world = rank, world
        self._weights: Dict[str, object] = {}
        if names is None:
            names = [n for n, t in tensors.items() if len(t.dims) >= 2 and int(t.type) in
                     (TensorType.Q8_0, TensorType.Q4_K, TensorType.Q5_K, TensorType.Q6_K, TensorType.IQ4_NL)]
        up = upload or (lambda qw, r0, r1: DeviceQuantWeight.upload(qw, device, r0, r1))
        for name in names:
            qw = load_qw(tensors, name)
            r0, r1 = shard_rows(qw.out_dim, rank, world) if world > 1 else (0, qw.out_dim)
            self._weights[name] = up(qw, r0, r1)

    def __getitem__(self, name: str):
        with self._lock:
            if self._closed:
                raise RuntimeError("weights are closed")
            try:
                return self._weights[name]
            except KeyError:
                raise KeyError(f"qwen35_weights: missing tensor {name!r}") from None

    def __contains__(self, name: str) -> bool:
        return name in self._weights

    def layer(self, il: int, projections: Sequence[str] = RECURRENT_PROJECTIONS) -> Dict[str, object]:
        return {p: self[f"blk.{il}.{p}.weight"] for p in projections if f"blk.{il}.{p}.weight" in self}

    @property
    def closed(self) -> bool:
        return self._closed

    def close(self) -> None:
        with self._lock:
            if self._closed:
                return
            self._weights.clear()          # drops the device buffers
            backing, self._backing = self._backing, None
            if backing is not None and hasattr(backing, "close"):
                backing.close()
            self._closed = True
