"""Runs the reference's own CUDA GEMV kernels (the cubins oracle/make_ref.py assembles from the
reference's PTX) the way the reference's probes do.  TEST INFRASTRUCTURE ONLY: used by the GPU
tests that pin the CPU oracle to reference-authored code and by the benchmark's same-box
`reference_ptx` timings; never by the product path.

The call sequence is the probes' (bin/cuda_q4k_gemv_probe.cr:158-266): cuModuleLoadData ->
cuModuleGetFunction -> kernelParams as an array of pointers to the boxed values -> cuLaunchKernel
with grid = ceil(out_dim / 4), block = 128, no dynamic shared memory, the null stream.  Modules are
loaded into whatever context is current on the calling thread (the tests make torch's primary
context current first); device pointers are plain integers (CUdeviceptr).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

REF_DIR = Path(__file__).resolve().parent / "_ref"

_cuda = None


class RefKernelError(RuntimeError):
    pass


def _check(code: int, what: str) -> None:
    if code != 0:  # the reference's cuda! helper (bin/cuda_q8_gemv_probe.cr:232-234)
        raise RefKernelError(f"{what} failed with CUDA error {code}")


def driver() -> C.CDLL:
    global _cuda
    if _cuda is None:
        L = C.CDLL("libcuda.so.1")
        L.cuInit.argtypes = [C.c_uint]
        L.cuModuleLoadData.argtypes = [C.POINTER(C.c_void_p), C.c_void_p]
        L.cuModuleGetFunction.argtypes = [C.POINTER(C.c_void_p), C.c_void_p, C.c_char_p]
        L.cuModuleUnload.argtypes = [C.c_void_p]
        L.cuLaunchKernel.argtypes = [C.c_void_p] + [C.c_uint] * 6 + [C.c_uint, C.c_void_p,
                                                                    C.POINTER(C.c_void_p), C.c_void_p]
        _check(L.cuInit(0), "cuInit")
        _cuda = L
    return _cuda


def available() -> bool:
    return all((REF_DIR / f"{n}.cubin").exists() for n in
               ("q4k_gemv", "q5k_gemv", "q6k_gemv", "q8_0_gemv", "output_top"))


class Module:
    """One cubin of oracle/_ref/, loaded into the current context."""

    def __init__(self, name: str):
        path = REF_DIR / f"{name}.cubin"
        if not path.exists():
            raise RefKernelError(f"{path} is missing: run `python oracle/make_ref.py` where the "
                                 "reference checkout is available")
        self._image = path.read_bytes()
        self._mod = C.c_void_p()
        _check(driver().cuModuleLoadData(C.byref(self._mod), self._image), f"cuModuleLoadData({name})")
        self._fns = {}

    def function(self, entry: str) -> C.c_void_p:
        if entry not in self._fns:
            fn = C.c_void_p()
            _check(driver().cuModuleGetFunction(C.byref(fn), self._mod, entry.encode()),
                   f"cuModuleGetFunction({entry})")
            self._fns[entry] = fn
        return self._fns[entry]

    def launch(self, entry: str, grid: int, block: int, params: list) -> None:
        """params: ints for u64 pointers, ('u32', v) tuples for 32-bit scalars."""
        boxed = []
        for p in params:
            boxed.append(C.c_uint32(p[1]) if isinstance(p, tuple) else C.c_uint64(p))
        arr = (C.c_void_p * len(boxed))(*[C.cast(C.pointer(b), C.c_void_p) for b in boxed])
        _check(driver().cuLaunchKernel(self.function(entry), grid, 1, 1, block, 1, 1, 0, None, arr,
                                       None), f"cuLaunchKernel({entry})")

    def close(self) -> None:
        if self._mod:
            driver().cuModuleUnload(self._mod)
            self._mod = C.c_void_p()


# tensor type -> (cubin, entry-name stem)
_GEMV = {8: ("q8_0_gemv", "q8_0_gemv"), 12: ("q4k_gemv", "q4_k_gemv"), 13: ("q5k_gemv", "q5_k_gemv"),
         14: ("q6k_gemv", "q6_k_gemv")}
_modules: dict = {}


def module(name: str) -> Module:
    if name not in _modules:
        _modules[name] = Module(name)
    return _modules[name]


def u32(v: int):
    return ("u32", int(v))


def gemv_warp4(qtype: int, d_w: int, d_x: int, d_out: int, in_dim: int, out_dim: int) -> None:
    """`<type>_gemv_warp4_f32`: one token (q4k_gemv_probe.ptx:219, q5k:5, q6k:193, the Q8_0 probe's
    heredoc bin/cuda_q8_gemv_probe.cr:126)."""
    cubin, stem = _GEMV[qtype]
    module(cubin).launch(f"{stem}_warp4_f32", (out_dim + 3) // 4, 128,
                         [d_w, d_x, d_out, u32(in_dim), u32(out_dim)])


def gemv_add_warp4(qtype: int, d_w: int, d_x: int, d_residual: int, d_out: int, in_dim: int,
                   out_dim: int) -> None:
    """`<type>_gemv_add_warp4_f32`: y = residual + W x (q4k_gemv_probe.ptx:1362, q6k:398)."""
    cubin, stem = _GEMV[qtype]
    module(cubin).launch(f"{stem}_add_warp4_f32", (out_dim + 3) // 4, 128,
                         [d_w, d_x, d_residual, d_out, u32(in_dim), u32(out_dim)])


def gemv_tbatch4(qtype: int, d_w: int, d_x: int, d_out: int, in_dim: int, out_dim: int) -> None:
    """`<type>_gemv_warp4_f32_tbatch4`: four tokens, x [4][in_dim], out [4][out_dim]
    (q4k_gemv_probe.ptx:437, q5k:237, q6k:977)."""
    cubin, stem = _GEMV[qtype]
    module(cubin).launch(f"{stem}_warp4_f32_tbatch4", (out_dim + 3) // 4, 128,
                         [d_w, d_x, d_out, u32(in_dim), u32(out_dim)])


def gemv_batched(qtype: int, d_w: int, d_x: int, d_out: int, in_dim: int, out_dim: int,
                 tokens: int) -> None:
    """`<type>_gemv_warp4_f32_batched`: grid = tokens * ceil(out_dim / 4) (q4k_gemv_probe.ptx:1584)."""
    cubin, stem = _GEMV[qtype]
    module(cubin).launch(f"{stem}_warp4_f32_batched", tokens * ((out_dim + 3) // 4), 128,
                         [d_w, d_x, d_out, u32(in_dim), u32(out_dim)])


def q4k_dual_gemv(d_w_a: int, d_w_b: int, d_x: int, d_out_a: int, d_out_b: int, in_dim: int,
                  out_dim: int) -> None:
    """`q4_k_dual_gemv_warp4_f32`: two Q4_K matrices of out_dim rows against one x; rows
    [0, 2*out_dim) select a | b (q4k_dual_gemv_probe.ptx:5; launched over ceil(2*out_dim / 4) CTAs,
    src/ml/cuda/qwen_recurrent_layer_runner.cr:608)."""
    module("q4k_dual_gemv").launch("q4_k_dual_gemv_warp4_f32", (2 * out_dim + 3) // 4, 128,
                                   [d_w_a, d_w_b, d_x, d_out_a, d_out_b, u32(in_dim), u32(out_dim)])


def q6k_top1(d_w: int, d_x: int, d_partial_ids: int, d_partial_values: int, d_top_id: int,
             d_top_value: int, in_dim: int, out_dim: int) -> None:
    """The fused lm_head route of the reference's output-head runner
    (src/ml/cuda/qwen_output_head_runner.cr:940-942): q6_k_gemv_top1_partial_f32 over
    ceil(vocab / 4) CTAs, then output_top1_values_reduce_probe on one CTA of 256 threads."""
    width = (out_dim + 3) // 4
    module("q6k_gemv").launch("q6_k_gemv_top1_partial_f32", width, 128,
                              [d_w, d_x, d_partial_ids, d_partial_values, u32(in_dim), u32(out_dim)])
    module("output_top").launch("output_top1_values_reduce_probe", 1, 256,
                                [d_partial_ids, d_partial_values, d_top_id, d_top_value, u32(width)])


def synchronize() -> None:
    _check(driver().cuCtxSynchronize(), "cuCtxSynchronize")
