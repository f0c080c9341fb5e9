// Fused lm_head top-1 for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need the lm_head:
// a runtime that hands every byte of HBM to its own arena at start-up, a plugin that is only
// given input and output buffers by its host, or a binding whose memory handles cannot be
// created late.  cogni_qmm_gemv_top1 asks such a caller for a scratch buffer it has no way to
// provide.  This file gives the same computation with the scratch held inside the library, in a
// file-scope device array: nothing is allocated, by this code or on its behalf.
//
// The array lives in every GPU context that loads the library, from load until exit, whether or
// not the entry point is ever called.  Its size is the fixed maximum below.
#include "qmm_common.cuh"

namespace {

// 1 MiB: covers the top-1 scratch of a 262144-row vocabulary at batch 16 with room to spare.
constexpr size_t kStaticScratchBytes = 1u << 20;
static __device__ __align__(256) unsigned char g_top1_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not an address a kernel can
// use: the device address has to be asked for with the device current.  The lookup is a cheap host
// call, so it is made on every call rather than cached: a cached address would go stale when the
// host destroys and re-creates the device's context (cudaDeviceReset).
int static_scratch_for_current_device(void **out) {
  void *ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&ptr, g_top1_static_scratch);
  if (e != cudaSuccess) return (int)e;
  if (!ptr) return COGNI_QMM_ERR_ARG;
  *out = ptr;
  return COGNI_QMM_OK;
}

}  // namespace

extern "C" {

size_t cogni_qmm_gemv_top1_noalloc_max_scratch(void) { return kStaticScratchBytes; }

int cogni_qmm_gemv_top1_noalloc(int type, const void *d_w, const float *d_x, int in_dim,
                                int out_dim, int batch, int32_t index_base, int32_t *d_top_index,
                                float *d_top_value, int64_t *d_top_key, void *stream) {
  if (out_dim <= 0 || batch <= 0) return COGNI_QMM_ERR_ARG;
  const size_t need = cogni_qmm_gemv_top1_scratch_bytes(out_dim, batch);
  if (need == 0) return COGNI_QMM_ERR_ARG;
  if (need > kStaticScratchBytes) return COGNI_QMM_ERR_LIMIT;  // vocabulary x batch too large
  void *scratch = nullptr;
  int st = static_scratch_for_current_device(&scratch);
  if (st != COGNI_QMM_OK) return st;
  // every argument check of cogni_qmm_gemv_top1 first: a rejected call must not touch the array
  st = cogni::check_top1_args(type, d_w, d_x, in_dim, out_dim, batch, index_base, scratch,
                              kStaticScratchBytes, d_top_index, d_top_value);
  if (st != COGNI_QMM_OK) return st;
  // The array keeps whatever the previous call (or a call that failed half-way) left in it; the
  // ticket counters at its start are the only part the kernel needs at zero.
  cudaError_t e = cudaMemsetAsync(scratch, 0, ((size_t)batch * 4 + 7) & ~(size_t)7,
                                  static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return (int)e;
  return cogni_qmm_gemv_top1(type, d_w, d_x, in_dim, out_dim, batch, index_base, scratch,
                             kStaticScratchBytes, d_top_index, d_top_value, d_top_key, stream);
}

}  // extern "C"
