// Shared device/host helpers for the GGUF quantized-matmul kernels (sm_100a).
//
// Block layouts (src/ml/gguf/dequant.cr of the reference, field offsets in bytes):
//   Q8_0  34 B / 32 el : d f16 @0, qs int8[32] @2
//   Q4_K 144 B / 256 el: d f16 @0, dmin f16 @2, scales[12] @4, qs[128] @16
//   Q5_K 176 B / 256 el: d f16 @0, dmin f16 @2, scales[12] @4, qh[32] @16, ql[128] @48
//   Q6_K 210 B / 256 el: ql[128] @0, qh[64] @128, scales int8[16] @192, d f16 @208
//   IQ4_NL 18 B / 32 el: d f16 @0, qs[16] @2: element j < 16 = table[qs[j] & 15], 16 + j = table[qs[j] >> 4]
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "../../include/cogni_qmm.h"

namespace cogni {

constexpr int kQ8_0 = COGNI_QMM_TYPE_Q8_0;
constexpr int kQ4_K = COGNI_QMM_TYPE_Q4_K;
constexpr int kQ5_K = COGNI_QMM_TYPE_Q5_K;
constexpr int kQ6_K = COGNI_QMM_TYPE_Q6_K;
constexpr int kIQ4_NL = COGNI_QMM_TYPE_IQ4_NL;

template <int TYPE> struct BlockGeom;
template <> struct BlockGeom<kQ8_0> { static constexpr int bytes = 34, elems = 32; };
template <> struct BlockGeom<kQ4_K> { static constexpr int bytes = 144, elems = 256; };
template <> struct BlockGeom<kQ5_K> { static constexpr int bytes = 176, elems = 256; };
template <> struct BlockGeom<kQ6_K> { static constexpr int bytes = 210, elems = 256; };
template <> struct BlockGeom<kIQ4_NL> { static constexpr int bytes = 18, elems = 32; };

__host__ __device__ inline int block_bytes(int type) {
  switch (type) {
    case kQ8_0: return 34;
    case kQ4_K: return 144;
    case kQ5_K: return 176;
    case kQ6_K: return 210;
    case kIQ4_NL: return 18;
    default: return -1;
  }
}
__host__ __device__ inline int block_elems(int type) {
  switch (type) {
    case kQ8_0:
    case kIQ4_NL: return 32;
    case kQ4_K:
    case kQ5_K:
    case kQ6_K: return 256;
    default: return -1;
  }
}

// The 16 non-linear levels of IQ4_NL (dequant.cr:11-16), packed eight to a 64-bit constant.
__device__ __forceinline__ int iq4nl_value(int q) {
  // -127, -104, -83, -65, -49, -35, -22, -10 | 1, 13, 25, 38, 53, 69, 89, 113
  const unsigned long long lo = 0xF6EADDCFBFAD9881ull, hi = 0x7159453526190D01ull;
  return (int)(signed char)(((q & 8) ? hi : lo) >> (8 * (q & 7)));
}

// Exact IEEE half -> float of two little-endian bytes at a 2-byte aligned address
// (hardware conversion; subnormal halves convert exactly, as dequant.cr:265-272 does in software).
__device__ __forceinline__ float load_half_as_float(const uint8_t *p) {
  return __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(p)));
}

// 6-bit (scale, min) pair j of a Q4_K / Q5_K block (dequant.cr:240-249).
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *s, int &sc, int &m) {
  if (j < 4) {
    sc = s[j] & 63;
    m = s[j + 4] & 63;
  } else {
    sc = (s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4);
    m = (s[j + 4] >> 4) | ((s[j] >> 6) << 4);
  }
}

// Maps a float to an int32 whose signed order equals the float order (no NaNs expected).
__host__ __device__ __forceinline__ int32_t orderable_from_float(float v) {
#ifdef __CUDA_ARCH__
  int32_t b = __float_as_int(v);
#else
  int32_t b;
  memcpy(&b, &v, 4);
#endif
  return b >= 0 ? b : (b ^ 0x7FFFFFFF);
}
__host__ __device__ __forceinline__ float float_from_orderable(int32_t o) {
  int32_t b = o >= 0 ? o : (o ^ 0x7FFFFFFF);
#ifdef __CUDA_ARCH__
  return __int_as_float(b);
#else
  float v;
  memcpy(&v, &b, 4);
  return v;
#endif
}
// key = (orderable(value) << 32) | (0xFFFFFFFF - index): a signed MAX picks the highest
// value and, among equal values, the lowest index.
__host__ __device__ __forceinline__ long long top1_key(float v, uint32_t index) {
  v += 0.f;  // -0.0 -> +0.0: the CPU reference compares them equal
  return (long long)(((unsigned long long)(uint32_t)orderable_from_float(v) << 32) |
                     (unsigned long long)(0xFFFFFFFFu - index));
}
__host__ __device__ __forceinline__ void top1_unkey(long long key, float &v, uint32_t &index) {
  v = float_from_orderable((int32_t)((unsigned long long)key >> 32));
  index = 0xFFFFFFFFu - (uint32_t)((unsigned long long)key & 0xFFFFFFFFull);
}

// Launchers implemented in the .cu files; each returns a cogni_qmm status.
int launch_dequantize(int type, const void *d_w, int64_t n, float *d_out, cudaStream_t s);
int launch_gemv_rowwarp(int type, const void *d_w, const float *d_x, const float *d_addend,
                        int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                        cudaStream_t s);
int launch_gemv_top1_rowwarp(int type, const void *d_w, const float *d_x, int in_dim,
                             int out_dim, int batch, int32_t index_base, void *d_scratch,
                             int32_t *d_idx, float *d_val, long long *d_key, cudaStream_t s);
size_t top1_scratch_bytes(int out_dim, int batch);
int check_top1_args(int type, const void *d_w, const float *d_x, int in_dim, int out_dim, int batch,
                    int32_t index_base, const void *d_scratch, size_t scratch_bytes,
                    const int32_t *d_top_index, const float *d_top_value);
size_t top2_scratch_bytes(int out_dim, int batch);
int launch_gemv_top2(int type, const void *d_w, const float *d_x, int in_dim, int out_dim, int batch,
                     int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val,
                     long long *d_key, int resident, cudaStream_t s);

// Integer tensor-core GEMV (gemv_imma.cu): Q8_0 / Q4_K / Q5_K / Q6_K; the fused top-1 for batch 1-2.
bool gemv_imma_supports(int type, const void *d_w, const float *d_x, int in_dim, int batch,
                        bool top1 = false);
int launch_gemv_swiglu_imma(int type, const void *d_w, const float *d_gate, const float *d_up,
                            const float *d_addend, int64_t addend_stride, float *d_y, int in_dim,
                            int out_dim, int batch, int resident, cudaStream_t s);
int launch_embedding_rows(int type, const void *d_table, const int32_t *d_ids, int n_tokens, int vocab,
                          int n_embd, float *d_out, int32_t *d_status, cudaStream_t s);
int launch_gemv_many_rmsnorm_imma(int type, int njobs, const void *const *d_w, const float *d_x,
                                  const float *d_norm_w, float eps, const float *const *d_addend,
                                  int64_t addend_stride, float *const *d_y, const int *out_dims,
                                  int in_dim, int batch, int resident, cudaStream_t s);
int launch_rmsnorm(const float *d_x, const float *d_w, float eps, float *d_out, int rows, int dim,
                   cudaStream_t s);
int launch_swiglu(const float *d_gate, const float *d_up, float *d_out, int64_t n, cudaStream_t s);
int launch_gemv_imma(int type, const void *d_w, const float *d_x, const float *d_addend,
                     int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                     int resident, cudaStream_t s);
int launch_gemv_top1_imma(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                          int batch, int32_t index_base, void *d_scratch, int32_t *d_idx,
                          float *d_val, long long *d_key, int resident, cudaStream_t s,
                          const float *d_norm_w = nullptr, float norm_eps = 0.f);
int launch_gemv_imma_many(int type, int njobs, const void *const *d_w, const float *d_x,
                          const float *const *d_addend, int64_t addend_stride, float *const *d_y,
                          const int *out_dims, int in_dim, int batch, int resident, cudaStream_t s);
int launch_gemv_imma_many_exchange(int type, int njobs, const void *const *d_w, const float *d_x,
                                   const float *const *d_addend, int64_t addend_stride,
                                   float *const *d_y, const int *out_dims, int in_dim, int batch,
                                   int resident, const cogni_qmm_exchange *ex, int wait_previous,
                                   int64_t y_pitch, cudaStream_t s);
unsigned gemv_imma_timeouts();
unsigned gemm_prefill_timeouts();
int gemv_imma_reset_timeouts();   // also clears the K-slab tickets of every workspace region
int gemm_prefill_reset_timeouts();
int launch_expire_wait(unsigned limit_us, cudaStream_t s);
int launch_exchange_unpack(const void *d_words, int64_t n, unsigned epoch, float *d_out, cudaStream_t s);
void gemv_imma_set_debug(int mode);
void gemv_imma_set_pair(int pair);
void gemv_imma_set_min_splits(int n);
void gemv_imma_set_slabs(int n);
void gemm_prefill_set_tile(int bn);
void gemm_prefill_set_split(int mode);
void gemm_prefill_set_stage_raw(int on);
void gemm_prefill_set_pair(int on);

// Kernel selection (dispatch.cu): picks the tiled kernel when the shape allows it, else the
// general row-per-warp kernel.
int launch_gemv(int type, const void *d_w, const float *d_x, const float *d_addend,
                int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                int resident, cudaStream_t s);
int launch_gemv_top1(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                     int batch, int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val,
                     long long *d_key, cudaStream_t s);
int launch_top1_unpack(const long long *d_keys, int batch, int32_t *d_idx, float *d_val,
                       cudaStream_t s);
int launch_gemm_prefill(int type, const void *d_w, const void *d_x_bf16, void *d_y, int out_type,
                        int m_rows, int n_out, int k_in, cudaStream_t s);

}  // namespace cogni
