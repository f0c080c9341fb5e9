"""The C-ABI library without a GPU: it loads, exports every symbol include/cogni_qmm.h and include/cogni_qmm_diag.h declare,
answers the geometry queries, names its statuses and rejects bad arguments before touching CUDA."""
import ctypes as C
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = (ROOT / "include" / "cogni_qmm.h").read_text() + (ROOT / "include" / "cogni_qmm_diag.h").read_text()


def declared_symbols():
    body = re.sub(r"/\*.*?\*/", "", HEADER, flags=re.S)
    return sorted(set(re.findall(r"\b(cogni_qmm_\w+)\s*\(", body)))


def test_library_exports_every_declared_symbol(engine):
    names = declared_symbols()
    assert len(names) >= 15
    raw = C.CDLL(str(ROOT / "cogni_ml_b200" / "libcogni_qmm.so"))
    for name in names:
        assert hasattr(raw, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header(engine):
    from cogni_ml_b200._lib import SIGNATURES
    assert sorted(SIGNATURES) == declared_symbols()


def test_abi_version_and_geometry(engine):
    lib = engine.lib
    assert lib.cogni_qmm_abi_version() == 1
    # TensorType#block_bytes / #block_elements (reader.cr:53-80)
    assert [lib.cogni_qmm_block_bytes(t) for t in (8, 12, 13, 14)] == [34, 144, 176, 210]
    assert [lib.cogni_qmm_block_elements(t) for t in (8, 12, 13, 14)] == [32, 256, 256, 256]
    assert lib.cogni_qmm_block_bytes(2) == -1
    # sizes quoted by the benchmark configurations
    assert lib.cogni_qmm_tensor_bytes(8, 3584, 1024) == 3_899_392
    assert lib.cogni_qmm_tensor_bytes(12, 12288, 4096) == 28_311_552
    assert lib.cogni_qmm_tensor_bytes(13, 4096, 4096) == 11_534_336
    assert lib.cogni_qmm_tensor_bytes(14, 4096, 12288) == 41_287_680
    assert lib.cogni_qmm_tensor_bytes(14, 151936, 5120) == 638_131_200
    assert lib.cogni_qmm_row_bytes(12, 100) == -1          # not a block multiple
    assert lib.cogni_qmm_row_bytes(99, 256) == -1


def test_geometry_agrees_with_oracle(engine, oracle):
    for t in (8, 12, 13, 14):
        for k in (256, 1024, 4096, 12288):
            assert engine.lib.cogni_qmm_row_bytes(t, k) == oracle.row_bytes(t, k)


def test_status_strings(engine):
    s = engine.lib.cogni_qmm_status_string
    assert s(0) == b"ok"
    assert b"unsupported tensor type" in s(1001)
    assert b"invalid argument" in s(1002)
    assert b"misaligned" in s(1003)
    assert b"scratch" in s(1004)
    assert s(123456) == b"unknown status"


def test_argument_errors_come_before_any_cuda_call(engine):
    lib = engine.lib
    # null pointers / bad sizes: ERR_ARG; unknown type: ERR_TYPE; odd pointer: ERR_ALIGN
    assert lib.cogni_qmm_gemv(12, None, None, None, 0, None, 4096, 16, 1, None) == 1002
    assert lib.cogni_qmm_gemv(2, 16, 16, None, 0, 16, 4096, 16, 1, None) == 1001
    assert lib.cogni_qmm_gemv(12, 16, 16, None, 0, 16, 100, 16, 1, None) == 1002
    assert lib.cogni_qmm_gemv(12, 24, 16, None, 0, 16, 256, 16, 1, None) == 1003
    assert lib.cogni_qmm_gemv(12, 16, 16, 16, 7, 16, 256, 16, 1, None) == 1002   # bad addend stride
    assert lib.cogni_qmm_gemv_resident(12, None, None, None, 0, None, 256, 1, 1, None) == 1002
    assert lib.cogni_qmm_dequantize(12, 16, 100, 16, None) == 1002
    assert lib.cogni_qmm_gemv_top1(14, 16, 16, 256, 8, 1, 0, 16, 1, 16, 16, None, None) == 1004
    assert lib.cogni_qmm_gemm_bf16(2, 16, 16, 16, 0, 1, 1, 256, None) == 1001     # Q4_0: not a type of this engine
    assert lib.cogni_qmm_gemm_bf16(12, 16, 16, 16, 0, 1, 1, 100, None) == 1002
    assert lib.cogni_qmm_set_kernel_choice(7) == 1002
    assert lib.cogni_qmm_set_kernel_choice(17) == 1002   # timing modes are not in the shipped build
    assert lib.cogni_qmm_diag_expire_wait(0, None) == 1002
    assert lib.cogni_qmm_gemv_top1_scratch_bytes(0, 1) == 0
    assert lib.cogni_qmm_gemv_top1_scratch_bytes(151936, 1) >= 8 + 8 * (151936 // 64)


def test_host_entry_point_rejects_bad_calls_without_a_gpu(engine):
    import numpy as np
    x = np.zeros(256, np.float32)
    w = np.zeros(144, np.uint8)
    y = np.zeros(1, np.float32)
    lib = engine.lib
    assert lib.cogni_qmm_matmul_add_host(x.ctypes.data, 1, 256, w.ctypes.data, 144, 2, 1,
                                         x.ctypes.data, y.ctypes.data) == 1001
    assert lib.cogni_qmm_matmul_add_host(x.ctypes.data, 1, 256, w.ctypes.data, 100, 12, 1,
                                         x.ctypes.data, y.ctypes.data) == 1002   # too few bytes


def test_no_cpu_fallback_in_the_product(engine):
    """Compute calls without a GPU must raise, never fall back."""
    import numpy as np
    import torch
    if torch.cuda.is_available():
        pytest.skip("only meaningful on a machine without a GPU")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        engine.QuantMatmul.matmul_add(np.zeros(256, np.float32), 1, 256, np.zeros(144, np.uint8),
                                      12, 1, np.zeros(1, np.float32))
    # nothing under the package imports the oracle
    for path in (ROOT / "cogni_ml_b200").rglob("*.py"):
        assert "oracle" not in path.read_text(), path
