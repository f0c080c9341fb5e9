"""cogni_ml_b200 — B200-native quantized-matmul engine for GGUF weights (Q8_0 / Q4_K / Q5_K / Q6_K).

The product is the C-ABI shared library built from csrc/ (see include/cogni_qmm.h); this package
is the host-side mirror of the reference's call surface over that ABI.  Importing it loads the
library and fails if it has not been built (`python cogni_ml_b200/build.py`).
"""
from . import synth  # noqa: F401  (numpy only)
from ._lib import CogniQmmError, lib  # noqa: F401
from .quant_matmul import (DeviceQuantWeight, GemvMany, QuantMatmul, QuantWeight,  # noqa: F401
                           TensorType, gemv_many, row_bytes, unpack_top1_keys)
from .runner import Projection, QuantProjectionRunner, ResidentSequenceRunner  # noqa: F401
from .loader import WeightUploader, plan_chunks  # noqa: F401

__all__ = ["CogniQmmError", "DeviceQuantWeight", "GemvMany", "gemv_many", "Projection", "QuantMatmul", "QuantProjectionRunner",
           "QuantWeight", "ResidentSequenceRunner", "TensorType", "WeightUploader", "lib", "plan_chunks",
           "row_bytes", "synth", "unpack_top1_keys"]
