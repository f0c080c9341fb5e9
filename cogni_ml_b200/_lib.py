"""ctypes binding of libcogni_qmm.so — one Python function per symbol in include/cogni_qmm.h.

There is no fallback: if the shared library is missing or a symbol cannot be resolved the
import fails, and every compute call needs a CUDA device.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libcogni_qmm.so"

_vp, _i, _i64, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_size_t

# symbol -> (restype, argtypes); kept in the order of include/cogni_qmm.h, then include/cogni_qmm_diag.h
SIGNATURES = {
    "cogni_qmm_abi_version": (_i, []),
    "cogni_qmm_status_string": (C.c_char_p, [_i]),
    "cogni_qmm_wait_timeouts": (C.c_uint, []),
    "cogni_qmm_reset_wait_timeouts": (_i, []),
    "cogni_qmm_block_bytes": (_i, [_i]),
    "cogni_qmm_block_elements": (_i, [_i]),
    "cogni_qmm_row_bytes": (_i64, [_i, _i]),
    "cogni_qmm_tensor_bytes": (_i64, [_i, _i, _i]),
    "cogni_qmm_dequantize": (_i, [_i, _vp, _i64, _vp, _vp]),
    "cogni_qmm_gemv": (_i, [_i, _vp, _vp, _vp, _i64, _vp, _i, _i, _i, _vp]),
    "cogni_qmm_gemv_resident": (_i, [_i, _vp, _vp, _vp, _i64, _vp, _i, _i, _i, _vp]),
    "cogni_qmm_gemv_many": (_i, [_i, _i, _vp, _vp, _vp, _i64, _vp, _vp, _i, _i, _i, _vp]),
    "cogni_qmm_gemv_many_rmsnorm": (_i, [_i, _i, _vp, _vp, _vp, C.c_float, _vp, _i64, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "cogni_qmm_embedding_lookup": (_i, [_i, _vp, _i, _i, _vp, _i, _vp, _vp, _vp]),
    "cogni_qmm_gemv_swiglu": (_i, [_i, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i, _i, _i, _i, _vp]),
    "cogni_qmm_gemv_many_exchange": (_i, [_i, _i, _vp, _vp, _vp, _i64, _vp, _i64, _vp, _i, _i, _i, _vp, _i, _vp]),
    "cogni_qmm_exchange_unpack": (_i, [_vp, _i64, C.c_uint32, _vp, _vp]),
    "cogni_qmm_sharded_gemv_nccl": (_i, [_vp, _i, _i, _i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "cogni_qmm_sharded_top1_nccl": (_i, [_vp, _i, _i, _vp, _vp, _i, _i, _i, C.c_int32, _vp, _sz, _vp, _vp, _vp, _vp]),
    "cogni_qmm_enable_peer_access": (_i, [_i]),
    "cogni_qmm_gemv_top1_scratch_bytes": (_sz, [_i, _i]),
    "cogni_qmm_gemv_top1": (_i, [_i, _vp, _vp, _i, _i, _i, C.c_int32, _vp, _sz, _vp, _vp, _vp, _vp]),
    "cogni_qmm_gemv_top1_rmsnorm": (_i, [_i, _vp, _vp, _vp, C.c_float, _i, _i, _i, C.c_int32, _vp, _sz, _vp, _vp, _vp, _vp, _i, _vp]),
    "cogni_qmm_gemv_top2_scratch_bytes": (_sz, [_i, _i]),
    "cogni_qmm_gemv_top2": (_i, [_i, _vp, _vp, _i, _i, _i, C.c_int32, _vp, _sz, _vp, _vp, _vp, _i, _vp]),
    "cogni_qmm_gemv_top1_noalloc_max_scratch": (_sz, []),
    "cogni_qmm_gemv_top1_noalloc": (_i, [_i, _vp, _vp, _i, _i, _i, C.c_int32, _vp, _vp, _vp, _vp]),
    "cogni_qmm_top1_unpack_keys": (_i, [_vp, _i, _vp, _vp, _vp]),
    "cogni_qmm_gemm_bf16": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "cogni_qmm_matmul_add_host": (_i, [_vp, _i, _i, _vp, _i64, _i, _i, _vp, _vp]),
    # include/cogni_qmm_diag.h
    "cogni_qmm_set_kernel_choice": (_i, [_i]),
    "cogni_qmm_diag_expire_wait": (_i, [C.c_uint, _vp]),
}


class CogniQmmError(RuntimeError):
    """Raised for any non-zero status, like ML::CUDA.check! in the reference's driver binding."""

    def __init__(self, what: str, status: int, text: str):
        super().__init__(f"{what} failed with status {status} ({text})")
        self.status = status


def load() -> C.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python cogni_ml_b200/build.py` "
            "(there is no CPU or PyTorch fallback for this engine)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here means the header and the library disagree
        fn.restype = res
        fn.argtypes = args
    return lib


lib = load()


def check(status: int, what: str) -> None:
    if status != 0:
        raise CogniQmmError(what, status, lib.cogni_qmm_status_string(status).decode())
