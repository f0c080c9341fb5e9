// Bulk dequantisation of raw GGUF blocks to f32 on the device.
//
// Bit-exact against the reference's CPU dequantiser (src/ml/gguf/dequant.cr): the same f32
// operations in the same order, written with the explicit round-to-nearest intrinsics so
// the compiler cannot contract a multiply and a subtract into one fused operation:
//   Q4_K/Q5_K  d1 = d*sc; m1 = dmin*m; w = d1*q - m1     (dequant.cr:120-133, 168-185)
//   Q6_K       w = (d*sc)*q                              (dequant.cr:224-227)
//   Q8_0       w = d*q                                   (dequant.cr:66-68)
//   IQ4_NL     w = d*table[nibble]                       (dequant.cr:76-101)
// One warp expands one 256-element superblock (one 32-element block for Q8_0); lane l
// writes element l of every 32-wide group, so each store instruction covers 128 contiguous
// bytes.  HBM-bound: 4 B written per element against 0.56-1.06 B read.
#include "qmm_common.cuh"

namespace cogni {
namespace {

template <int TYPE>
__device__ __forceinline__ void expand_block(const uint8_t *b, float *y, int lane);

template <>
__device__ __forceinline__ void expand_block<kQ8_0>(const uint8_t *b, float *y, int lane) {
  float d = load_half_as_float(b);
  int q = reinterpret_cast<const int8_t *>(b + 2)[lane];
  y[lane] = __fmul_rn(d, (float)q);
}

template <>
__device__ __forceinline__ void expand_block<kIQ4_NL>(const uint8_t *b, float *y, int lane) {
  float d = load_half_as_float(b);
  int q = b[2 + (lane & 15)];
  y[lane] = __fmul_rn(d, (float)iq4nl_value(lane < 16 ? (q & 0x0F) : (q >> 4)));
}

template <>
__device__ __forceinline__ void expand_block<kQ4_K>(const uint8_t *b, float *y, int lane) {
  float d = load_half_as_float(b), dmin = load_half_as_float(b + 2);
  const uint8_t *scales = b + 4, *qs = b + 16;
#pragma unroll
  for (int pair = 0; pair < 4; pair++) {
    int sc, m, sc2, m2;
    scale_min_k4(2 * pair, scales, sc, m);
    scale_min_k4(2 * pair + 1, scales, sc2, m2);
    float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)m);
    float d2 = __fmul_rn(d, (float)sc2), m2f = __fmul_rn(dmin, (float)m2);
    int q = qs[32 * pair + lane];
    y[64 * pair + lane] = __fsub_rn(__fmul_rn(d1, (float)(q & 0x0F)), m1);
    y[64 * pair + 32 + lane] = __fsub_rn(__fmul_rn(d2, (float)(q >> 4)), m2f);
  }
}

template <>
__device__ __forceinline__ void expand_block<kQ5_K>(const uint8_t *b, float *y, int lane) {
  float d = load_half_as_float(b), dmin = load_half_as_float(b + 2);
  const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
  int h = qh[lane];
#pragma unroll
  for (int pair = 0; pair < 4; pair++) {
    int sc, m, sc2, m2;
    scale_min_k4(2 * pair, scales, sc, m);
    scale_min_k4(2 * pair + 1, scales, sc2, m2);
    float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)m);
    float d2 = __fmul_rn(d, (float)sc2), m2f = __fmul_rn(dmin, (float)m2);
    int q = ql[32 * pair + lane];
    int qlo = (q & 0x0F) + (((h >> (2 * pair)) & 1) << 4);
    int qhi = (q >> 4) + (((h >> (2 * pair + 1)) & 1) << 4);
    y[64 * pair + lane] = __fsub_rn(__fmul_rn(d1, (float)qlo), m1);
    y[64 * pair + 32 + lane] = __fsub_rn(__fmul_rn(d2, (float)qhi), m2f);
  }
}

template <>
__device__ __forceinline__ void expand_block<kQ6_K>(const uint8_t *b, float *y, int lane) {
  const uint8_t *ql = b, *qh = b + 128;
  const int8_t *sc = reinterpret_cast<const int8_t *>(b + 192);
  float d = load_half_as_float(b + 208);
  int is = lane >> 4;
#pragma unroll
  for (int half = 0; half < 2; half++) {
    int l0 = ql[64 * half + lane], l1 = ql[64 * half + 32 + lane], h = qh[32 * half + lane];
    int q1 = ((l0 & 0xF) | (((h >> 0) & 3) << 4)) - 32;
    int q2 = ((l1 & 0xF) | (((h >> 2) & 3) << 4)) - 32;
    int q3 = ((l0 >> 4) | (((h >> 4) & 3) << 4)) - 32;
    int q4 = ((l1 >> 4) | (((h >> 6) & 3) << 4)) - 32;
    const int8_t *s = sc + 8 * half + is;
    float *yy = y + 128 * half + lane;
    yy[0] = __fmul_rn(__fmul_rn(d, (float)s[0]), (float)q1);
    yy[32] = __fmul_rn(__fmul_rn(d, (float)s[2]), (float)q2);
    yy[64] = __fmul_rn(__fmul_rn(d, (float)s[4]), (float)q3);
    yy[96] = __fmul_rn(__fmul_rn(d, (float)s[6]), (float)q4);
  }
}

template <int TYPE>
__global__ void __launch_bounds__(256) dequantize_blocks_kernel(const uint8_t *__restrict__ w,
                                                                float *__restrict__ out,
                                                                long long nblocks) {
  const int lane = threadIdx.x & 31;
  long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long blk = warp; blk < nblocks; blk += nwarps)
    expand_block<TYPE>(w + blk * BlockGeom<TYPE>::bytes, out + blk * BlockGeom<TYPE>::elems, lane);
}

// Token-embedding gather: out[t, :] = dequant(row token_ids[t] of the table), the same block
// expansion as the bulk dequantiser (bit-exact against Dequant.dequantize of that row,
// src/ml/gguf/qwen35_cpu.cr:3305-3332).  One warp per block of a token's row.  An id outside
// [0, vocab) yields a row of zeros and raises *status to 1 + the index of such a token.
template <int TYPE>
__global__ void __launch_bounds__(256) embedding_rows_kernel(const uint8_t *__restrict__ table,
                                                             const int32_t *__restrict__ token_ids,
                                                             int n_tokens, int vocab, int blocks_per_row,
                                                             float *__restrict__ out, int32_t *status) {
  constexpr int BE = BlockGeom<TYPE>::elems, BB = BlockGeom<TYPE>::bytes;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)n_tokens * blocks_per_row;
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long i = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < total; i += nwarps) {
    const int t = (int)(i / blocks_per_row), blk = (int)(i - (long long)t * blocks_per_row);
    const int id = token_ids[t];
    float *y = out + ((long long)t * blocks_per_row + blk) * BE;
    if (id < 0 || id >= vocab) {
      for (int e = lane; e < BE; e += 32) y[e] = 0.f;
      if (status && blk == 0 && lane == 0) atomicMax(status, t + 1);
      continue;
    }
    expand_block<TYPE>(table + ((long long)id * blocks_per_row + blk) * BB, y, lane);
  }
}

template <int TYPE>
int run_embedding(const void *d_table, const int32_t *d_ids, int n_tokens, int vocab, int n_embd,
                  float *d_out, int32_t *d_status, cudaStream_t s) {
  const int bpr = n_embd / BlockGeom<TYPE>::elems;
  const long long want = ((long long)n_tokens * bpr + 7) / 8;
  if (want == 0) return COGNI_QMM_OK;
  const int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
  embedding_rows_kernel<TYPE><<<grid, 256, 0, s>>>(static_cast<const uint8_t *>(d_table), d_ids,
                                                  n_tokens, vocab, bpr, d_out, d_status);
  return (int)cudaGetLastError();
}

template <int TYPE>
int run(const void *d_w, int64_t n, float *d_out, cudaStream_t s) {
  long long nblocks = n / BlockGeom<TYPE>::elems;
  if (nblocks == 0) return COGNI_QMM_OK;
  long long want = (nblocks + 7) / 8;
  int grid = (int)(want < 148LL * 16 ? want : 148LL * 16);
  dequantize_blocks_kernel<TYPE><<<grid, 256, 0, s>>>(static_cast<const uint8_t *>(d_w), d_out,
                                                     nblocks);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_dequantize(int type, const void *d_w, int64_t n, float *d_out, cudaStream_t s) {
  switch (type) {
    case kQ8_0: return run<kQ8_0>(d_w, n, d_out, s);
    case kIQ4_NL: return run<kIQ4_NL>(d_w, n, d_out, s);
    case kQ4_K: return run<kQ4_K>(d_w, n, d_out, s);
    case kQ5_K: return run<kQ5_K>(d_w, n, d_out, s);
    case kQ6_K: return run<kQ6_K>(d_w, n, d_out, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

int launch_embedding_rows(int type, const void *d_table, const int32_t *d_ids, int n_tokens, int vocab,
                          int n_embd, float *d_out, int32_t *d_status, cudaStream_t s) {
  switch (type) {
    case kQ8_0: return run_embedding<kQ8_0>(d_table, d_ids, n_tokens, vocab, n_embd, d_out, d_status, s);
    case kIQ4_NL: return run_embedding<kIQ4_NL>(d_table, d_ids, n_tokens, vocab, n_embd, d_out, d_status, s);
    case kQ4_K: return run_embedding<kQ4_K>(d_table, d_ids, n_tokens, vocab, n_embd, d_out, d_status, s);
    case kQ5_K: return run_embedding<kQ5_K>(d_table, d_ids, n_tokens, vocab, n_embd, d_out, d_status, s);
    case kQ6_K: return run_embedding<kQ6_K>(d_table, d_ids, n_tokens, vocab, n_embd, d_out, d_status, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

}  // namespace cogni
