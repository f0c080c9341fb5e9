// extern "C" entry points of libcogni_qmm.so: argument checks, kernel selection, and the
// one-shot host-buffer form.  Declarations and per-function contracts: include/cogni_qmm.h
// (the product ABI) and include/cogni_qmm_diag.h (A/B switches for tests and measurements).
#include <cstdio>
#include <cstring>

#include "qmm_common.cuh"
#include "../../include/cogni_qmm_diag.h"

using namespace cogni;

namespace cogni { extern int g_force_rowwarp; }

namespace {

bool supported(int type) { return block_bytes(type) > 0; }

int check_gemv_args(int type, const void *w, const void *x, const void *y, int in_dim, int out_dim,
                    int batch) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (!w || !x || !y || in_dim <= 0 || out_dim <= 0 || batch <= 0) return COGNI_QMM_ERR_ARG;
  if (in_dim % block_elems(type) != 0) return COGNI_QMM_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 3) ||
      (reinterpret_cast<uintptr_t>(y) & 3))
    return COGNI_QMM_ERR_ALIGN;
  return COGNI_QMM_OK;
}

}  // namespace

namespace cogni {
// Everything cogni_qmm_gemv_top1 checks before it touches the device (shared with the entry point
// that keeps the scratch inside the library, which must not write to it for a call it rejects).
int check_top1_args(int type, const void *d_w, const float *d_x, int in_dim, int out_dim, int batch,
                    int32_t index_base, const void *d_scratch, size_t scratch_bytes,
                    const int32_t *d_top_index, const float *d_top_value) {
  int st = check_gemv_args(type, d_w, d_x, d_top_value, in_dim, out_dim, batch);
  if (st) return st;
  if (!d_top_index || !d_scratch || index_base < 0) return COGNI_QMM_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(d_scratch) & 7) return COGNI_QMM_ERR_ALIGN;
  if (scratch_bytes < top1_scratch_bytes(out_dim, batch)) return COGNI_QMM_ERR_SCRATCH;
  return COGNI_QMM_OK;
}
}  // namespace cogni

extern "C" {

int cogni_qmm_abi_version(void) { return COGNI_QMM_ABI_VERSION; }

const char *cogni_qmm_status_string(int status) {
  switch (status) {
    case COGNI_QMM_OK: return "ok";
    case COGNI_QMM_ERR_TYPE: return "unsupported tensor type";
    case COGNI_QMM_ERR_ARG: return "invalid argument";
    case COGNI_QMM_ERR_ALIGN: return "misaligned device pointer";
    case COGNI_QMM_ERR_SCRATCH: return "scratch buffer too small";
    case COGNI_QMM_ERR_DEVICE: return "device is not compute capability 10.x";
    case COGNI_QMM_ERR_LIMIT: return "size beyond the entry point's fixed maximum";
    case COGNI_QMM_ERR_NCCL_MISSING: return "libnccl.so.2 could not be loaded";
    case COGNI_QMM_ERR_TIMEOUT: return "a bounded device-side wait expired: results invalid until cogni_qmm_reset_wait_timeouts()";
    default: break;
  }
  if (status > 0 && status < 1000) return cudaGetErrorString(static_cast<cudaError_t>(status));
  if (status > COGNI_QMM_ERR_NCCL_BASE && status < COGNI_QMM_ERR_NCCL_BASE + 100) return "an NCCL call failed (status - 2000 is its ncclResult_t)";
  return "unknown status";
}

int cogni_qmm_set_kernel_choice(int choice) {
#ifdef COGNI_QMM_DIAG_TIMING
  if (choice >= 16 && choice <= 21) {  // timing diagnostics of the tiled GEMV (results invalid)
    // 16 normal, 17 stream only, 18 stream + scale decode; 19-21 the same without the copies
    gemv_imma_set_debug(choice <= 18 ? choice - 16 : 4 + (choice == 19 ? 0 : choice - 19));
    return COGNI_QMM_OK;
  }
  if (choice >= 32 && choice < 48) {  // raw diagnostic bits of the tiled GEMV (results invalid)
    gemv_imma_set_debug(choice - 32);
    return COGNI_QMM_OK;
  }
#endif
  if (choice >= 48 && choice <= 51) {  // prefill token-tile width: automatic / 128 / 256 / 512
    gemm_prefill_set_tile(choice == 48 ? 0 : 64 << (choice - 48));
    return COGNI_QMM_OK;
  }
  if (choice == 55 || choice == 56) {  // prefill: raw superblocks staged by TMA (55, default) or read directly (56)
    gemm_prefill_set_stage_raw(choice == 55);
    return COGNI_QMM_OK;
  }
  if (choice == 57 || choice == 58) {  // prefill, 512-token tiles: CTA pairs (57, default) or single CTAs (58)
    gemm_prefill_set_pair(choice == 57);
    return COGNI_QMM_OK;
  }
  if (choice >= 52 && choice <= 54) {  // prefill split along K: automatic / never / two splits wherever allowed
    gemm_prefill_set_split(choice - 52);
    return COGNI_QMM_OK;
  }
  if (choice == 59) {  // prefill split along K: four ordered splits wherever allowed
    gemm_prefill_set_split(3);
    return COGNI_QMM_OK;
  }
  if (choice >= 27 && choice <= 30) {  // at least 1 .. 4 column ranges per row of the tiled GEMV
    gemv_imma_set_min_splits(choice - 26);
    return COGNI_QMM_OK;
  }
  if (choice >= 60 && choice <= 68) {  // K slabs of the tiled GEMV: off / 1 .. 8 wherever a plan allows
    gemv_imma_set_slabs(choice - 60);
    return COGNI_QMM_OK;
  }
  if (choice >= 24 && choice <= 26) {  // superblocks per work item of the tiled GEMV: automatic / 1 / 2
    gemv_imma_set_pair(choice - 24);
    return COGNI_QMM_OK;
  }
  if (choice != 0 && choice != 1) return COGNI_QMM_ERR_ARG;
  g_force_rowwarp = choice;
  return COGNI_QMM_OK;
}

int cogni_qmm_diag_expire_wait(unsigned limit_us, void *stream) {
  return launch_expire_wait(limit_us, static_cast<cudaStream_t>(stream));
}

unsigned cogni_qmm_wait_timeouts(void) { return gemv_imma_timeouts() + gemm_prefill_timeouts(); }

int cogni_qmm_reset_wait_timeouts(void) {
  int st = gemv_imma_reset_timeouts();
  if (st == COGNI_QMM_OK) st = gemm_prefill_reset_timeouts();
  return st;
}

int cogni_qmm_block_bytes(int type) { return block_bytes(type); }
int cogni_qmm_block_elements(int type) { return block_elems(type); }

int64_t cogni_qmm_row_bytes(int type, int in_dim) {
  int be = block_elems(type);
  if (be < 0 || in_dim <= 0 || in_dim % be != 0) return -1;
  return (int64_t)(in_dim / be) * block_bytes(type);
}

int64_t cogni_qmm_tensor_bytes(int type, int out_dim, int in_dim) {
  int64_t rb = cogni_qmm_row_bytes(type, in_dim);
  if (rb < 0 || out_dim <= 0) return -1;
  return rb * out_dim;
}

int cogni_qmm_dequantize(int type, const void *d_w, int64_t n_elements, float *d_out,
                         void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (!d_w || !d_out || n_elements < 0 || n_elements % block_elems(type) != 0)
    return COGNI_QMM_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(d_w) & 1) || (reinterpret_cast<uintptr_t>(d_out) & 3))
    return COGNI_QMM_ERR_ALIGN;
  return launch_dequantize(type, d_w, n_elements, d_out, static_cast<cudaStream_t>(stream));
}

static int gemv_common(int type, const void *d_w, const float *d_x, const float *d_addend,
                       int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                       int resident, void *stream) {
  int st = check_gemv_args(type, d_w, d_x, d_y, in_dim, out_dim, batch);
  if (st) return st;
  if (d_addend && addend_stride != 0 && addend_stride != out_dim) return COGNI_QMM_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  for (int b0 = 0; b0 < batch; b0 += 16) {
    int nb = batch - b0 < 16 ? batch - b0 : 16;
    const float *add = d_addend ? d_addend + (int64_t)b0 * addend_stride : nullptr;
    st = launch_gemv(type, d_w, d_x + (int64_t)b0 * in_dim, add, addend_stride,
                     d_y + (int64_t)b0 * out_dim, in_dim, out_dim, nb, resident, s);
    if (st) return st;
  }
  return COGNI_QMM_OK;
}

int cogni_qmm_gemv(int type, const void *d_w, const float *d_x, const float *d_addend,
                   int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                   void *stream) {
  return gemv_common(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, 0, stream);
}

int cogni_qmm_gemv_resident(int type, const void *d_w, const float *d_x, const float *d_addend,
                            int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                            void *stream) {
  return gemv_common(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, 1, stream);
}

int cogni_qmm_embedding_lookup(int type, const void *d_table, int vocab, int n_embd,
                               const int32_t *d_token_ids, int n_tokens, float *d_out,
                               int32_t *d_status, void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (!d_table || !d_token_ids || !d_out || vocab <= 0 || n_embd <= 0 || n_tokens < 0) return COGNI_QMM_ERR_ARG;
  if (n_embd % cogni_qmm_block_elements(type) != 0) return COGNI_QMM_ERR_ARG;
  return launch_embedding_rows(type, d_table, d_token_ids, n_tokens, vocab, n_embd, d_out, d_status,
                               static_cast<cudaStream_t>(stream));
}

int cogni_qmm_gemv_swiglu(int type, const void *d_w, const float *d_gate, const float *d_up,
                          const float *d_addend, int64_t addend_stride, float *d_y,
                          float *d_x_scratch, int in_dim, int out_dim, int batch, int resident,
                          void *stream) {
  int st = check_gemv_args(type, d_w, d_gate, d_y, in_dim, out_dim, batch);
  if (st) return st;
  if (!d_up) return COGNI_QMM_ERR_ARG;
  if (d_addend && addend_stride != 0 && addend_stride != out_dim) return COGNI_QMM_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (g_force_rowwarp == 0 && (reinterpret_cast<uintptr_t>(d_up) & 15) == 0 &&
      gemv_imma_supports(type, d_w, d_gate, in_dim, batch))
    return launch_gemv_swiglu_imma(type, d_w, d_gate, d_up, d_addend, addend_stride, d_y, in_dim,
                                   out_dim, batch, resident, s);
  // shapes the fused kernel does not take: form the product in the caller's scratch, then the GEMV
  if (!d_x_scratch) return COGNI_QMM_ERR_SCRATCH;
  st = launch_swiglu(d_gate, d_up, d_x_scratch, (int64_t)batch * in_dim, s);
  if (st) return st;
  return gemv_common(type, d_w, d_x_scratch, d_addend, addend_stride, d_y, in_dim, out_dim, batch, 0,
                     stream);
}

int cogni_qmm_gemv_many(int type, int n_weights, const void *const *d_w, const float *d_x,
                        const float *const *d_addend, int64_t addend_stride, float *const *d_y,
                        const int *out_dims, int in_dim, int batch, int resident, void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (n_weights <= 0 || !d_w || !d_y || !out_dims) return COGNI_QMM_ERR_ARG;
  bool tiled = g_force_rowwarp == 0;
  for (int j = 0; j < n_weights; j++) {
    int st = check_gemv_args(type, d_w[j], d_x, d_y[j], in_dim, out_dims[j], batch);
    if (st) return st;
    if (d_addend && d_addend[j] && addend_stride != 0 && addend_stride != out_dims[j])
      return COGNI_QMM_ERR_ARG;
    tiled = tiled && gemv_imma_supports(type, d_w[j], d_x, in_dim, batch);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tiled)
    return launch_gemv_imma_many(type, n_weights, d_w, d_x, d_addend, addend_stride, d_y, out_dims,
                                 in_dim, batch, resident, s);
  for (int j = 0; j < n_weights; j++) {
    int st = gemv_common(type, d_w[j], d_x, d_addend ? d_addend[j] : nullptr, addend_stride, d_y[j],
                         in_dim, out_dims[j], batch, resident, stream);
    if (st) return st;
  }
  return COGNI_QMM_OK;
}

int cogni_qmm_gemv_many_exchange(int type, int n_weights, const void *const *d_w, const float *d_x,
                                 const float *const *d_addend, int64_t addend_stride,
                                 float *const *d_y, int64_t y_pitch, const int *out_dims, int in_dim,
                                 int batch, int resident, const cogni_qmm_exchange *ex,
                                 int wait_previous, void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (n_weights <= 0 || !d_w || !d_y || !out_dims || !ex || y_pitch < 0) return COGNI_QMM_ERR_ARG;
  if (ex->world < 1 || ex->world > 8 || ex->rank < 0 || ex->rank >= ex->world || !ex->epoch || !ex->ticket)
    return COGNI_QMM_ERR_ARG;
  for (int g = 0; g < ex->world; g++)
    if (g != ex->rank && (ex->peer_offset[g] & 7)) return COGNI_QMM_ERR_ARG;
  for (int j = 0; j < n_weights; j++) {
    int st = check_gemv_args(type, d_w[j], d_x, d_y[j], in_dim, out_dims[j], batch);
    if (st) return st;
    if (reinterpret_cast<uintptr_t>(d_y[j]) & 7) return COGNI_QMM_ERR_ALIGN;   // 8-byte words
    if (d_addend && d_addend[j] && addend_stride != 0 && addend_stride != out_dims[j])
      return COGNI_QMM_ERR_ARG;
    if (g_force_rowwarp != 0 || !gemv_imma_supports(type, d_w[j], d_x, in_dim, batch)) return COGNI_QMM_ERR_LIMIT;
  }
  return launch_gemv_imma_many_exchange(type, n_weights, d_w, d_x, d_addend, addend_stride, d_y, out_dims,
                                        in_dim, batch, resident, ex, wait_previous, y_pitch,
                                        static_cast<cudaStream_t>(stream));
}

int cogni_qmm_exchange_unpack(const void *d_words, int64_t n, uint32_t epoch, float *d_out, void *stream) {
  if (!d_words || !d_out || n <= 0) return COGNI_QMM_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(d_words) & 7) return COGNI_QMM_ERR_ALIGN;
  return launch_exchange_unpack(d_words, n, epoch, d_out, static_cast<cudaStream_t>(stream));
}

int cogni_qmm_enable_peer_access(int peer_device) {
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();  // not an error for the caller: clear the sticky code
    return COGNI_QMM_OK;
  }
  return (int)e;
}

int cogni_qmm_gemv_many_rmsnorm(int type, int n_weights, const void *const *d_w, const float *d_x,
                                const float *d_norm_weight, float eps,
                                const float *const *d_addend, int64_t addend_stride,
                                float *const *d_y, const int *out_dims, float *d_x_scratch,
                                int in_dim, int batch, int resident, void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (n_weights <= 0 || !d_w || !d_y || !out_dims || !d_norm_weight) return COGNI_QMM_ERR_ARG;
  bool tiled = g_force_rowwarp == 0 && (reinterpret_cast<uintptr_t>(d_norm_weight) & 15) == 0;
  for (int j = 0; j < n_weights; j++) {
    int st = check_gemv_args(type, d_w[j], d_x, d_y[j], in_dim, out_dims[j], batch);
    if (st) return st;
    if (d_addend && d_addend[j] && addend_stride != 0 && addend_stride != out_dims[j])
      return COGNI_QMM_ERR_ARG;
    tiled = tiled && gemv_imma_supports(type, d_w[j], d_x, in_dim, batch);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (tiled && n_weights <= 32)
    return launch_gemv_many_rmsnorm_imma(type, n_weights, d_w, d_x, d_norm_weight, eps, d_addend,
                                         addend_stride, d_y, out_dims, in_dim, batch, resident, s);
  // shapes the fused kernel does not take: normalise into the caller's scratch, then the GEMVs
  if (!d_x_scratch) return COGNI_QMM_ERR_SCRATCH;
  int st = launch_rmsnorm(d_x, d_norm_weight, eps, d_x_scratch, batch, in_dim, s);
  if (st) return st;
  return cogni_qmm_gemv_many(type, n_weights, d_w, d_x_scratch, d_addend, addend_stride, d_y, out_dims,
                             in_dim, batch, 0, stream);
}

size_t cogni_qmm_gemv_top1_scratch_bytes(int out_dim, int batch) {
  if (out_dim <= 0 || batch <= 0) return 0;
  return top1_scratch_bytes(out_dim, batch);
}

int cogni_qmm_gemv_top1(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                        int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                        int32_t *d_top_index, float *d_top_value, int64_t *d_top_key,
                        void *stream) {
  int st = check_top1_args(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, scratch_bytes,
                           d_top_index, d_top_value);
  if (st) return st;
  return launch_gemv_top1(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                          d_top_index, d_top_value, reinterpret_cast<long long *>(d_top_key),
                          static_cast<cudaStream_t>(stream));
}

int cogni_qmm_gemv_top1_rmsnorm(int type, const void *d_w, const float *d_x,
                                const float *d_norm_weight, float eps, int in_dim, int out_dim,
                                int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                                float *d_x_scratch, int32_t *d_top_index, float *d_top_value,
                                int64_t *d_top_key, int resident, void *stream) {
  int st = check_gemv_args(type, d_w, d_x, d_top_value, in_dim, out_dim, batch);
  if (st) return st;
  if (!d_top_index || !d_scratch || !d_norm_weight || index_base < 0) return COGNI_QMM_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(d_scratch) & 7) return COGNI_QMM_ERR_ALIGN;
  if (scratch_bytes < top1_scratch_bytes(out_dim, batch)) return COGNI_QMM_ERR_SCRATCH;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (g_force_rowwarp == 0 && (reinterpret_cast<uintptr_t>(d_norm_weight) & 15) == 0 &&
      gemv_imma_supports(type, d_w, d_x, in_dim, batch, true))
    return launch_gemv_top1_imma(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                                 d_top_index, d_top_value, reinterpret_cast<long long *>(d_top_key),
                                 resident, s, d_norm_weight, eps);
  if (!d_x_scratch) return COGNI_QMM_ERR_SCRATCH;
  st = launch_rmsnorm(d_x, d_norm_weight, eps, d_x_scratch, batch, in_dim, s);
  if (st) return st;
  return launch_gemv_top1(type, d_w, d_x_scratch, in_dim, out_dim, batch, index_base, d_scratch,
                          d_top_index, d_top_value, reinterpret_cast<long long *>(d_top_key), s);
}

size_t cogni_qmm_gemv_top2_scratch_bytes(int out_dim, int batch) {
  if (out_dim <= 0 || batch <= 0) return 0;
  return top2_scratch_bytes(out_dim, batch);
}

int cogni_qmm_gemv_top2(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                        int batch, int32_t index_base, void *d_scratch, size_t scratch_bytes,
                        int32_t *d_top_index, float *d_top_value, int64_t *d_top_key, int resident,
                        void *stream) {
  int st = check_gemv_args(type, d_w, d_x, d_top_value, in_dim, out_dim, batch);
  if (st) return st;
  if (!d_top_index || !d_scratch || index_base < 0 || out_dim < 2) return COGNI_QMM_ERR_ARG;
  if (reinterpret_cast<uintptr_t>(d_scratch) & 7) return COGNI_QMM_ERR_ALIGN;
  if (scratch_bytes < top2_scratch_bytes(out_dim, batch)) return COGNI_QMM_ERR_SCRATCH;
  return launch_gemv_top2(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_top_index,
                          d_top_value, reinterpret_cast<long long *>(d_top_key), resident,
                          static_cast<cudaStream_t>(stream));
}

int cogni_qmm_top1_unpack_keys(const int64_t *d_keys, int batch, int32_t *d_top_index,
                               float *d_top_value, void *stream) {
  if (!d_keys || !d_top_index || !d_top_value || batch <= 0) return COGNI_QMM_ERR_ARG;
  return launch_top1_unpack(reinterpret_cast<const long long *>(d_keys), batch, d_top_index,
                            d_top_value, static_cast<cudaStream_t>(stream));
}

int cogni_qmm_gemm_bf16(int type, const void *d_w, const void *d_x_bf16, void *d_y, int out_type,
                        int m_rows, int n_out, int k_in, void *stream) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (!d_w || !d_x_bf16 || !d_y || m_rows <= 0 || n_out <= 0 || k_in <= 0 || k_in % 256 != 0)
    return COGNI_QMM_ERR_ARG;
  if (out_type != COGNI_QMM_OUT_F32 && out_type != COGNI_QMM_OUT_BF16) return COGNI_QMM_ERR_ARG;
  if ((reinterpret_cast<uintptr_t>(d_w) & 15) || (reinterpret_cast<uintptr_t>(d_x_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(d_y) & 15))
    return COGNI_QMM_ERR_ALIGN;
  return launch_gemm_prefill(type, d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in,
                             static_cast<cudaStream_t>(stream));
}

int cogni_qmm_matmul_add_host(const float *x, int rows, int in_dim, const void *w_raw,
                              int64_t w_bytes, int type, int out_dim, const float *bias, float *y) {
  if (!supported(type)) return COGNI_QMM_ERR_TYPE;
  if (!x || !w_raw || !y || rows <= 0 || in_dim <= 0 || out_dim <= 0) return COGNI_QMM_ERR_ARG;
  int64_t need = cogni_qmm_tensor_bytes(type, out_dim, in_dim);
  if (need < 0 || w_bytes < need) return COGNI_QMM_ERR_ARG;
  void *d_w = nullptr;
  float *d_x = nullptr, *d_b = nullptr, *d_y = nullptr;
  size_t xb = (size_t)rows * in_dim * 4, yb = (size_t)rows * out_dim * 4;
  int st = COGNI_QMM_OK;
  auto step = [&](cudaError_t e) {
    if (st == COGNI_QMM_OK && e != cudaSuccess) st = (int)e;
    return st == COGNI_QMM_OK;
  };
  if (step(cudaMalloc(&d_w, (size_t)need)) && step(cudaMalloc(&d_x, xb)) &&
      step(cudaMalloc(&d_y, yb)) && (!bias || step(cudaMalloc(&d_b, (size_t)out_dim * 4))) &&
      step(cudaMemcpy(d_w, w_raw, (size_t)need, cudaMemcpyHostToDevice)) &&
      step(cudaMemcpy(d_x, x, xb, cudaMemcpyHostToDevice)) &&
      (!bias || step(cudaMemcpy(d_b, bias, (size_t)out_dim * 4, cudaMemcpyHostToDevice)))) {
    st = cogni_qmm_gemv(type, d_w, d_x, d_b, 0, d_y, in_dim, out_dim, rows, nullptr);
    if (st == COGNI_QMM_OK) step(cudaMemcpy(y, d_y, yb, cudaMemcpyDeviceToHost));
    if (st == COGNI_QMM_OK && cogni_qmm_wait_timeouts() != 0) st = COGNI_QMM_ERR_TIMEOUT;
  }
  cudaFree(d_w);
  cudaFree(d_x);
  cudaFree(d_y);
  cudaFree(d_b);
  return st;
}

}  // extern "C"
