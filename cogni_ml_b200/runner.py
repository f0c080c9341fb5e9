"""Resident upload / run / read-back lifecycle for quantized projections.

ResidentSequenceRunner mirrors ML::CUDA::ResidentSequenceRunner (src/ml/cuda/driver.cr:288-342)
name for name: a facade over five callables with an `active_tokens` prefix and the same
argument errors.

QuantProjectionRunner is the part of QwenRecurrentLayerRunner that belongs to the quantized
matmul path (src/ml/cuda/qwen_recurrent_layer_runner.cr:164-176, 473-488, 570-595, 1381-1386):
raw GGUF bytes uploaded once and kept resident, token rows staged through pinned host memory,
one weight-stationary GEMV per projection for all active tokens, outputs read back on demand.
The recurrent (DeltaNet) core of that runner is not part of this engine.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

import numpy as np
import torch

from .quant_matmul import DeviceQuantWeight, QuantWeight


class ResidentSequenceRunner:
    """driver.cr:288-342."""

    def __init__(self, tokens: int, upload_weights: Callable[[], None],
                 reset_sequence: Callable[[], None], run_token: Callable[[int], None],
                 read_outputs: Optional[Callable[[], None]] = None,
                 run_sequence_override: Optional[Callable[[int], None]] = None):
        if not tokens > 0:
            raise ValueError("tokens must be positive")
        self.tokens = tokens
        self._upload_weights = upload_weights
        self._reset_sequence = reset_sequence
        self._run_token = run_token
        self._read_outputs = read_outputs
        self._run_sequence_override = run_sequence_override
        self._active_tokens = tokens

    @property
    def active_tokens(self) -> int:
        return self._active_tokens

    @active_tokens.setter
    def active_tokens(self, value: int) -> None:
        if not value > 0:
            raise ValueError("active_tokens must be positive")
        if not value <= self.tokens:
            raise ValueError("active_tokens must be <= tokens")
        self._active_tokens = value

    def reset_active_tokens(self) -> None:
        self._active_tokens = self.tokens

    def upload_weights(self) -> None:
        self._upload_weights()

    def reset_sequence(self) -> None:
        self._reset_sequence()

    def run_sequence(self) -> None:
        if self._run_sequence_override is not None:
            self._run_sequence_override(self._active_tokens)
        else:
            for tok in range(self._active_tokens):
                self._run_token(tok)

    def run_repeated(self, reps: int) -> int:
        if not reps > 0:
            raise ValueError("reps must be positive")
        for _ in range(reps):
            self.run_sequence()
        return reps * self._active_tokens

    def read_outputs(self) -> None:
        if self._read_outputs is not None:
            self._read_outputs()


@dataclass
class Projection:
    """One quantized matmul of the layer: output `name` = W @ input buffer `source`."""

    name: str
    weight: QuantWeight
    source: str
    residual: Optional[str] = None  # name of an input buffer added to the result ("*_gemv_add_*")


class QuantProjectionRunner:
    """Resident runner for a set of quantized projections over `tokens` rows.

    from_weights -> upload_weights -> reset_sequence -> run_sequence / run_repeated ->
    read_outputs -> close, in the order the reference's runners use.
    """

    def __init__(self, projections: List[Projection], tokens: int, inputs: Dict[str, np.ndarray],
                 device="cuda"):
        if not torch.cuda.is_available():
            raise RuntimeError("QuantProjectionRunner needs a CUDA device; there is no CPU fallback")
        self.device = torch.device(device)
        self.projections = projections
        self.tokens = tokens
        self._closed = False
        self._weights: Dict[str, DeviceQuantWeight] = {}
        self._host_in: Dict[str, torch.Tensor] = {}
        self._dev_in: Dict[str, torch.Tensor] = {}
        self._dev_out: Dict[str, torch.Tensor] = {}
        self._host_out: Dict[str, torch.Tensor] = {}
        self._external: Dict[str, torch.Tensor] = {}
        for name, arr in inputs.items():
            arr = np.ascontiguousarray(arr, dtype=np.float32)
            if arr.ndim != 2 or arr.shape[0] != tokens:
                raise ValueError(f"input {name} must be [tokens, dim]")
            pinned = torch.empty(arr.shape, dtype=torch.float32).pin_memory()
            pinned.copy_(torch.from_numpy(arr))
            self._host_in[name] = pinned
            self._dev_in[name] = torch.empty(arr.shape, dtype=torch.float32, device=self.device)
        for p in projections:
            if p.source not in inputs or (p.residual and p.residual not in inputs):
                raise ValueError(f"projection {p.name} reads an unknown buffer")
            if inputs[p.source].shape[1] != p.weight.in_dim:
                raise ValueError(f"projection {p.name}: input width != in_dim")
            self._dev_out[p.name] = torch.empty(tokens, p.weight.out_dim, dtype=torch.float32,
                                                device=self.device)
            self._host_out[p.name] = torch.empty(tokens, p.weight.out_dim,
                                                 dtype=torch.float32).pin_memory()
        self._facade = ResidentSequenceRunner(tokens, self._do_upload, self._do_reset,
                                              self._run_token, self._do_read, self._run_tokens)

    @classmethod
    def from_weights(cls, projections: List[Projection], tokens: int,
                     inputs: Dict[str, np.ndarray], device="cuda") -> "QuantProjectionRunner":
        return cls(projections, tokens, inputs, device)

    # -- lifecycle, same names as the reference ------------------------------------------
    @property
    def active_tokens(self) -> int:
        return self._facade.active_tokens

    @active_tokens.setter
    def active_tokens(self, value: int) -> None:
        self._facade.active_tokens = value

    def upload_weights(self) -> None:
        self._facade.upload_weights()

    def reset_sequence(self) -> None:
        self._facade.reset_sequence()

    def run_sequence(self) -> None:
        self._facade.run_sequence()

    def run_repeated(self, reps: int) -> int:
        return self._facade.run_repeated(reps)

    def read_outputs(self) -> Dict[str, np.ndarray]:
        self._facade.read_outputs()
        n = self.active_tokens
        return {k: v[:n].numpy() for k, v in self._host_out.items()}

    def use_device_sequence_input(self, name: str, buf: torch.Tensor) -> None:
        """Chain runners on the device: read input `name` from another runner's output buffer."""
        if buf.dtype != torch.float32 or tuple(buf.shape) != tuple(self._dev_in[name].shape):
            raise ValueError("device input must be f32 with the declared shape")
        self._external[name] = buf

    def output_device_ptr(self, name: str) -> torch.Tensor:
        return self._dev_out[name]

    def weight_bytes(self) -> int:
        return sum(w.nbytes for w in self._weights.values())

    def close(self) -> None:
        if self._closed:
            return
        self._weights.clear()
        self._dev_in.clear()
        self._dev_out.clear()
        self._external.clear()
        self._closed = True

    # -- implementation ------------------------------------------------------------------
    def _do_upload(self) -> None:
        for p in self.projections:
            self._weights[p.name] = DeviceQuantWeight.upload(p.weight, self.device)

    def _do_reset(self) -> None:
        """Stage the token rows: pinned host -> device (asynchronous on the current stream)."""
        for name, pinned in self._host_in.items():
            if name not in self._external:
                self._dev_in[name].copy_(pinned, non_blocking=True)

    def _input(self, name: str) -> torch.Tensor:
        return self._external.get(name, self._dev_in[name])

    def _run_tokens(self, active_tokens: int) -> None:
        if not self._weights:
            raise RuntimeError("upload_weights must run before run_sequence")
        for p in self.projections:
            x = self._input(p.source)[:active_tokens]
            res = self._input(p.residual)[:active_tokens] if p.residual else None
            self._weights[p.name].gemv(x, out=self._dev_out[p.name][:active_tokens], residual=res)

    def _run_token(self, tok: int) -> None:
        for p in self.projections:
            x = self._input(p.source)[tok:tok + 1]
            res = self._input(p.residual)[tok:tok + 1] if p.residual else None
            self._weights[p.name].gemv(x, out=self._dev_out[p.name][tok:tok + 1], residual=res)

    def _do_read(self) -> None:
        for name, dev in self._dev_out.items():
            self._host_out[name].copy_(dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()
