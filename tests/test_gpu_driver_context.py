"""The library inside a Driver-API context of the host's own making.

The reference never touches the CUDA runtime: `Context.create` calls cuInit / cuDeviceGet /
cuCtxCreate_v2 (src/ml/cuda/driver.cr:70-83), buffers come from cuMemAlloc_v2 and copies are
cuMemcpyHtoD_v2 / cuMemcpyDtoH_v2 (driver.cr:96-110, 262-276).  libcogni_qmm.so uses the CUDA
runtime, which adopts whatever context is current on the calling thread; this test performs the
reference's exact call sequence through ctypes on libcuda in a fresh process (no torch, no primary
context) and runs the GEMV, the fused top-1 and the bulk dequantiser between the copies.
"""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

SCRIPT = textwrap.dedent('''
    import ctypes as C, sys
    import numpy as np
    sys.path.insert(0, %r)
    from oracle import loader as oracle
    import importlib.util
    spec = importlib.util.spec_from_file_location("synth", %r)
    synth = importlib.util.module_from_spec(spec); spec.loader.exec_module(synth)

    cu = C.CDLL("libcuda.so.1")
    def check(code, what):
        if code != 0:
            raise RuntimeError(f"{what} failed with CUDA error {code}")   # ML::CUDA.check!
    check(cu.cuInit(0), "cuInit")
    dev = C.c_int()
    check(cu.cuDeviceGet(C.byref(dev), 0), "cuDeviceGet")
    ctx = C.c_void_p()
    check(cu.cuCtxCreate_v2(C.byref(ctx), 0, dev), "cuCtxCreate")
    cu.cuMemAlloc_v2.argtypes = [C.POINTER(C.c_uint64), C.c_size_t]
    cu.cuMemcpyHtoD_v2.argtypes = [C.c_uint64, C.c_void_p, C.c_size_t]
    cu.cuMemcpyDtoH_v2.argtypes = [C.c_void_p, C.c_uint64, C.c_size_t]
    cu.cuMemFree_v2.argtypes = [C.c_uint64]
    cu.cuMemsetD8_v2.argtypes = [C.c_uint64, C.c_ubyte, C.c_size_t]
    def alloc(nbytes):
        p = C.c_uint64()
        check(cu.cuMemAlloc_v2(C.byref(p), nbytes), "cuMemAlloc")
        return p.value
    def htod(arr):
        p = alloc(arr.nbytes)
        check(cu.cuMemcpyHtoD_v2(p, arr.ctypes.data, arr.nbytes), "cuMemcpyHtoD")
        return p
    lib = C.CDLL(%r)
    vp, i, i64 = C.c_uint64, C.c_int, C.c_int64
    lib.cogni_qmm_gemv.argtypes = [i, vp, vp, vp, i64, vp, i, i, i, C.c_void_p]
    lib.cogni_qmm_gemv_top1.argtypes = [i, vp, vp, i, i, i, C.c_int32, vp, C.c_size_t, vp, vp, vp, C.c_void_p]
    lib.cogni_qmm_gemv_top1_scratch_bytes.restype = C.c_size_t
    lib.cogni_qmm_dequantize.argtypes = [i, vp, i64, vp, C.c_void_p]
    for qtype, out_dim, in_dim, batch in ((12, 4096, 4096, 1), (14, 1024, 2560, 4), (8, 512, 1024, 2)):
        w = synth.make_weight(qtype, out_dim, in_dim, seed=3, tensor_id=qtype)
        x = synth.make_activation(batch, in_dim, seed=3)
        d_w, d_x = htod(w), htod(x)
        d_y = alloc(batch * out_dim * 4)
        check(lib.cogni_qmm_gemv(qtype, d_w, d_x, 0, 0, d_y, in_dim, out_dim, batch, None), "cogni_qmm_gemv")
        check(cu.cuCtxSynchronize(), "cuCtxSynchronize")
        y = np.empty(batch * out_dim, np.float32)
        check(cu.cuMemcpyDtoH_v2(y.ctypes.data, d_y, y.nbytes), "cuMemcpyDtoH")
        ref = oracle.matmul_add(x, batch, in_dim, w, qtype, out_dim, np.zeros(out_dim, np.float32))
        assert np.abs(y - ref).max() <= 1e-3 * np.abs(ref).max(), (qtype, np.abs(y - ref).max())
        need = lib.cogni_qmm_gemv_top1_scratch_bytes(out_dim, batch)
        d_s = alloc(need)
        check(cu.cuMemsetD8_v2(d_s, 0, need), "cuMemsetD8")
        d_i, d_v = alloc(batch * 4), alloc(batch * 4)
        check(lib.cogni_qmm_gemv_top1(qtype, d_w, d_x, in_dim, out_dim, batch, 0, d_s, need, d_i, d_v, 0, None),
              "cogni_qmm_gemv_top1")
        idx = np.empty(batch, np.int32)
        check(cu.cuMemcpyDtoH_v2(idx.ctypes.data, d_i, idx.nbytes), "cuMemcpyDtoH")
        for b in range(batch):
            assert idx[b] == oracle.top1(ref.reshape(batch, out_dim)[b])[0]
        d_f = alloc(out_dim * in_dim * 4)
        check(lib.cogni_qmm_dequantize(qtype, d_w, out_dim * in_dim, d_f, None), "cogni_qmm_dequantize")
        deq = np.empty(out_dim * in_dim, np.float32)
        check(cu.cuMemcpyDtoH_v2(deq.ctypes.data, d_f, deq.nbytes), "cuMemcpyDtoH")
        assert np.array_equal(deq.view(np.uint32), oracle.dequantize(qtype, w, out_dim * in_dim).view(np.uint32))
        for p in (d_w, d_x, d_y, d_s, d_i, d_v, d_f):
            cu.cuMemFree_v2(p)
        print(f"type={qtype} out_dim={out_dim} in_dim={in_dim} batch={batch} ok=true")
    assert lib.cogni_qmm_wait_timeouts() == 0
    cu.cuCtxDestroy_v2.argtypes = [C.c_void_p]
    check(cu.cuCtxDestroy_v2(ctx), "cuCtxDestroy")
    print("driver_context_ok")
''')


def test_library_runs_in_a_cuctxcreate_context(cuda):
    script = SCRIPT % (str(ROOT), str(ROOT / "cogni_ml_b200" / "synth.py"),
                       str(ROOT / "cogni_ml_b200" / "libcogni_qmm.so"))
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stdout + proc.stderr
    assert "driver_context_ok" in proc.stdout
