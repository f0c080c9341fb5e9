// General-shape GEMV for raw GGUF blocks: one warp per output row, lane l takes element l
// of every 32-wide group, fp32 FMA accumulation, warp-shuffle reduction.
//
// This kernel accepts every legal shape (any out_dim, any in_dim that is a block multiple,
// any batch, 2-byte aligned rows) and is the path for shapes the tiled tensor-core GEMV
// does not take.  It also carries the fused lm_head variant: GEMV + per-part top-1 +
// last-CTA-done reduction, all in one launch.
//
// Weight value arithmetic follows src/ml/gguf/quant_matmul.cr (w = d*sc*q - dmin*m for
// Q4_K/Q5_K, w = d*sc*(q-32) for Q6_K, w = d*q for Q8_0) in fp32 instead of f64.
#include <climits>

#include "qmm_common.cuh"

namespace cogni {
namespace {

constexpr int kWarpsPerCta = 8;
constexpr int kTop1RowsPerPart = 64;  // rows whose best key one scratch slot holds

template <int NB>
__device__ __forceinline__ void fma_cols(float w, const float *x, int64_t xs, float (&acc)[NB]) {
#pragma unroll
  for (int c = 0; c < NB; c++) acc[c] = fmaf(w, x[c * xs], acc[c]);
}

template <int TYPE, int NB> struct BlockDot;

template <int NB> struct BlockDot<kQ8_0, NB> {
  static __device__ __forceinline__ void run(const uint8_t *b, const float *x, int64_t xs, int lane,
                                             float (&acc)[NB]) {
    float d = load_half_as_float(b);
    float w = d * (float)reinterpret_cast<const int8_t *>(b + 2)[lane];
    fma_cols<NB>(w, x + lane, xs, acc);
  }
};

template <int NB> struct BlockDot<kIQ4_NL, NB> {
  static __device__ __forceinline__ void run(const uint8_t *b, const float *x, int64_t xs, int lane,
                                             float (&acc)[NB]) {
    float d = load_half_as_float(b);
    int q = b[2 + (lane & 15)];
    float w = d * (float)iq4nl_value(lane < 16 ? (q & 0x0F) : (q >> 4));
    fma_cols<NB>(w, x + lane, xs, acc);
  }
};

template <int NB> struct BlockDot<kQ4_K, NB> {
  static __device__ __forceinline__ void run(const uint8_t *b, const float *x, int64_t xs, int lane,
                                             float (&acc)[NB]) {
    float d = load_half_as_float(b), dmin = load_half_as_float(b + 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
#pragma unroll
    for (int pair = 0; pair < 4; pair++) {
      int sc, m, sc2, m2;
      scale_min_k4(2 * pair, scales, sc, m);
      scale_min_k4(2 * pair + 1, scales, sc2, m2);
      int q = qs[32 * pair + lane];
      float wlo = fmaf(d * (float)sc, (float)(q & 0x0F), -(dmin * (float)m));
      float whi = fmaf(d * (float)sc2, (float)(q >> 4), -(dmin * (float)m2));
      fma_cols<NB>(wlo, x + 64 * pair + lane, xs, acc);
      fma_cols<NB>(whi, x + 64 * pair + 32 + lane, xs, acc);
    }
  }
};

template <int NB> struct BlockDot<kQ5_K, NB> {
  static __device__ __forceinline__ void run(const uint8_t *b, const float *x, int64_t xs, int lane,
                                             float (&acc)[NB]) {
    float d = load_half_as_float(b), dmin = load_half_as_float(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    int h = qh[lane];
#pragma unroll
    for (int pair = 0; pair < 4; pair++) {
      int sc, m, sc2, m2;
      scale_min_k4(2 * pair, scales, sc, m);
      scale_min_k4(2 * pair + 1, scales, sc2, m2);
      int q = ql[32 * pair + lane];
      int qlo = (q & 0x0F) + (((h >> (2 * pair)) & 1) << 4);
      int qhi = (q >> 4) + (((h >> (2 * pair + 1)) & 1) << 4);
      float wlo = fmaf(d * (float)sc, (float)qlo, -(dmin * (float)m));
      float whi = fmaf(d * (float)sc2, (float)qhi, -(dmin * (float)m2));
      fma_cols<NB>(wlo, x + 64 * pair + lane, xs, acc);
      fma_cols<NB>(whi, x + 64 * pair + 32 + lane, xs, acc);
    }
  }
};

template <int NB> struct BlockDot<kQ6_K, NB> {
  static __device__ __forceinline__ void run(const uint8_t *b, const float *x, int64_t xs, int lane,
                                             float (&acc)[NB]) {
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
      const float *xx = x + 128 * half + lane;
      fma_cols<NB>(d * (float)s[0] * (float)q1, xx, xs, acc);
      fma_cols<NB>(d * (float)s[2] * (float)q2, xx + 32, xs, acc);
      fma_cols<NB>(d * (float)s[4] * (float)q3, xx + 64, xs, acc);
      fma_cols<NB>(d * (float)s[6] * (float)q4, xx + 96, xs, acc);
    }
  }
};

template <int NB>
__device__ __forceinline__ void warp_sum(float (&acc)[NB]) {
#pragma unroll
  for (int c = 0; c < NB; c++) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc[c] += __shfl_xor_sync(0xffffffffu, acc[c], off);
  }
}

// y[b, o] = addend + W[o,:] . x[b,:] for NB batch columns starting at b0 (columns past the
// batch are clamped onto the last valid one and not stored).
template <int TYPE, int NB>
__device__ __forceinline__ void row_dot(const uint8_t *wrow, const float *x, int in_dim, int batch,
                                        int b0, int lane, float (&acc)[NB]) {
  constexpr int BE = BlockGeom<TYPE>::elems, BB = BlockGeom<TYPE>::bytes;
#pragma unroll
  for (int c = 0; c < NB; c++) acc[c] = 0.f;
  // Column c reads x row min(b0+c, batch-1); with a uniform stride this needs b0+NB <= batch,
  // so the launcher picks NB dividing the work and the tail is handled by clamping b0.
  const float *xb = x + (int64_t)b0 * in_dim;
  const int nblk = in_dim / BE;
  for (int blk = 0; blk < nblk; blk++)
    BlockDot<TYPE, NB>::run(wrow + (int64_t)blk * BB, xb + (int64_t)blk * BE, in_dim, lane, acc);
  warp_sum<NB>(acc);
}

template <int TYPE, int NB>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    gemv_rowwarp_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                        const float *addend, int64_t addend_stride, float *y, int in_dim,
                        int out_dim, int batch) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  if (row >= out_dim) return;
  const int64_t row_bytes = (int64_t)(in_dim / BlockGeom<TYPE>::elems) * BlockGeom<TYPE>::bytes;
  const uint8_t *wrow = w + (int64_t)row * row_bytes;
  for (int b0 = 0; b0 < batch; b0 += NB) {
    int bb = b0 + NB <= batch ? b0 : batch - NB;  // last group overlaps instead of overrunning
    float acc[NB];
    row_dot<TYPE, NB>(wrow, x, in_dim, batch, bb, lane, acc);
    if (lane == 0) {
#pragma unroll
      for (int c = 0; c < NB; c++) {
        int b = bb + c;
        if (b < b0) continue;  // already written by the previous group
        float a = addend ? addend[(int64_t)b * addend_stride + row] : 0.f;
        y[(int64_t)b * out_dim + row] = a + acc[c];
      }
    }
  }
}

// Fused lm_head: each CTA owns kTop1RowsPerPart consecutive rows of one batch row's logits,
// keeps the best (value, index) key, stores it in its scratch slot; the CTA that takes the
// last ticket of a batch row folds all slots and writes the result.
template <int TYPE>
__global__ void __launch_bounds__(kWarpsPerCta * 32)
    gemv_top1_rowwarp_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                             int in_dim, int out_dim, int32_t index_base, unsigned *counters,
                             long long *part_keys, int nparts, int32_t *top_idx, float *top_val,
                             long long *top_key) {
  __shared__ long long s_best[kWarpsPerCta];
  __shared__ bool s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y, part = blockIdx.x;
  const int64_t row_bytes = (int64_t)(in_dim / BlockGeom<TYPE>::elems) * BlockGeom<TYPE>::bytes;
  long long best = LLONG_MIN;
  const int row_end = min(out_dim, (part + 1) * kTop1RowsPerPart);
  for (int row = part * kTop1RowsPerPart + warp; row < row_end; row += kWarpsPerCta) {
    float acc[1];
    row_dot<TYPE, 1>(w + (int64_t)row * row_bytes, x, in_dim, gridDim.y, b, lane, acc);
    long long key = top1_key(acc[0], (uint32_t)(index_base + row));
    best = key > best ? key : best;
  }
  if (lane == 0) s_best[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < kWarpsPerCta; i++) best = s_best[i] > best ? s_best[i] : best;
    part_keys[(int64_t)b * nparts + part] = best;
    __threadfence();
    unsigned ticket = atomicAdd(&counters[b], 1u);
    s_last = (ticket == (unsigned)nparts - 1u);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  best = LLONG_MIN;
  for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
    long long k = __ldcg(&part_keys[(int64_t)b * nparts + i]);
    best = k > best ? k : best;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    long long o = __shfl_xor_sync(0xffffffffu, best, off);
    best = o > best ? o : best;
  }
  __syncthreads();
  if (lane == 0) s_best[warp] = best;
  __syncthreads();
  if (threadIdx.x == 0) {
#pragma unroll
    for (int i = 1; i < kWarpsPerCta; i++) best = s_best[i] > best ? s_best[i] : best;
    float v;
    uint32_t idx;
    top1_unkey(best, v, idx);
    top_idx[b] = (int32_t)idx;
    top_val[b] = v;
    if (top_key) top_key[b] = best;
    counters[b] = 0u;  // ready for the next call on this scratch buffer
  }
}

template <int TYPE>
int run_gemv(const void *d_w, const float *d_x, const float *d_addend, int64_t addend_stride,
             float *d_y, int in_dim, int out_dim, int batch, cudaStream_t s) {
  const uint8_t *w = static_cast<const uint8_t *>(d_w);
  dim3 grid((out_dim + kWarpsPerCta - 1) / kWarpsPerCta), block(kWarpsPerCta * 32);
  if (batch >= 4)
    gemv_rowwarp_kernel<TYPE, 4><<<grid, block, 0, s>>>(w, d_x, d_addend, addend_stride, d_y,
                                                        in_dim, out_dim, batch);
  else if (batch >= 2)
    gemv_rowwarp_kernel<TYPE, 2><<<grid, block, 0, s>>>(w, d_x, d_addend, addend_stride, d_y,
                                                        in_dim, out_dim, batch);
  else
    gemv_rowwarp_kernel<TYPE, 1><<<grid, block, 0, s>>>(w, d_x, d_addend, addend_stride, d_y,
                                                        in_dim, out_dim, batch);
  return (int)cudaGetLastError();
}

template <int TYPE>
int run_top1(const void *d_w, const float *d_x, int in_dim, int out_dim, int batch,
             int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val, long long *d_key,
             cudaStream_t s) {
  int nparts = (out_dim + kTop1RowsPerPart - 1) / kTop1RowsPerPart;
  unsigned *counters = static_cast<unsigned *>(d_scratch);
  long long *keys = reinterpret_cast<long long *>(static_cast<char *>(d_scratch) +
                                                  (((size_t)batch * 4 + 7) & ~(size_t)7));
  dim3 grid(nparts, batch), block(kWarpsPerCta * 32);
  gemv_top1_rowwarp_kernel<TYPE><<<grid, block, 0, s>>>(static_cast<const uint8_t *>(d_w), d_x,
                                                         in_dim, out_dim, index_base, counters,
                                                         keys, nparts, d_idx, d_val, d_key);
  return (int)cudaGetLastError();
}

}  // namespace

size_t top1_scratch_bytes(int out_dim, int batch) {
  // one slot per 64 rows, and never fewer than 256 so a one-CTA-per-SM kernel always has a slot
  size_t nparts = ((size_t)out_dim + kTop1RowsPerPart - 1) / kTop1RowsPerPart;
  if (nparts < 256) nparts = 256;
  return (((size_t)batch * 4 + 7) & ~(size_t)7) + (size_t)batch * nparts * 8;
}

int launch_gemv_rowwarp(int type, const void *d_w, const float *d_x, const float *d_addend,
                        int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                        cudaStream_t s) {
  switch (type) {
    case kQ8_0: return run_gemv<kQ8_0>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
    case kIQ4_NL: return run_gemv<kIQ4_NL>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
    case kQ4_K: return run_gemv<kQ4_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
    case kQ5_K: return run_gemv<kQ5_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
    case kQ6_K: return run_gemv<kQ6_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

int launch_gemv_top1_rowwarp(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                             int batch, int32_t index_base, void *d_scratch, int32_t *d_idx,
                             float *d_val, long long *d_key, cudaStream_t s) {
  switch (type) {
    case kQ8_0: return run_top1<kQ8_0>(d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_idx, d_val, d_key, s);
    case kIQ4_NL: return run_top1<kIQ4_NL>(d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_idx, d_val, d_key, s);
    case kQ4_K: return run_top1<kQ4_K>(d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_idx, d_val, d_key, s);
    case kQ5_K: return run_top1<kQ5_K>(d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_idx, d_val, d_key, s);
    case kQ6_K: return run_top1<kQ6_K>(d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch, d_idx, d_val, d_key, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

}  // namespace cogni
