// Kernel selection for the C-ABI entry points.
#include <climits>

#include "qmm_common.cuh"

namespace cogni {

// 1 = route every GEMV to the general row-per-warp kernel (testing and A/B timing)
int g_force_rowwarp = 0;

namespace {
__global__ void top1_unpack_kernel(const long long *keys, int batch, int32_t *idx, float *val) {
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  float v;
  uint32_t i;
  top1_unkey(keys[b], v, i);
  idx[b] = (int32_t)i;
  val[b] = v;
}
}  // namespace

int launch_gemv(int type, const void *d_w, const float *d_x, const float *d_addend,
                int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                int resident, cudaStream_t s) {
  if (g_force_rowwarp == 0 && gemv_imma_supports(type, d_w, d_x, in_dim, batch))
    return launch_gemv_imma(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch,
                            resident, s);
  return launch_gemv_rowwarp(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
}

int launch_gemv_top1(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                     int batch, int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val,
                     long long *d_key, cudaStream_t s) {
  if (g_force_rowwarp == 0 && gemv_imma_supports(type, d_w, d_x, in_dim, batch, true))
    return launch_gemv_top1_imma(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                                 d_idx, d_val, d_key, 0, s);
  return launch_gemv_top1_rowwarp(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                                  d_idx, d_val, d_key, s);
}

namespace {
// out = silu(gate) * up, silu(v) = v / (1 + exp(-v)) in f32 (qwen35_cpu.cr:512-519, 1716-1717)
__global__ void swiglu_kernel(const float *gate, const float *up, float *out, int64_t n) {
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const float g = gate[i];
    out[i] = g / (1.f + expf(-g)) * up[i];
  }
}
// out[r, :] = x[r, :] * (1 / sqrt(mean(x[r, :]^2) + eps)) * w, sum of squares in f64, the products
// in f32 left to right (qwen35_cpu.cr:484-490, 1492-1504).  One CTA per row.
__global__ void __launch_bounds__(256) rmsnorm_kernel(const float *x, const float *w, float eps,
                                                      float *out, int dim) {
  __shared__ double s_ss[8];
  __shared__ float s_inv;
  const float *xr = x + (long long)blockIdx.x * dim;
  double ss = 0.0;
  for (int k = threadIdx.x; k < dim; k += blockDim.x) ss += (double)xr[k] * xr[k];
  for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if ((threadIdx.x & 31) == 0) s_ss[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < 8; i++) t += s_ss[i];
    s_inv = (float)(1.0 / sqrt(t / (double)dim + (double)eps));
  }
  __syncthreads();
  const float r = s_inv;
  for (int k = threadIdx.x; k < dim; k += blockDim.x)
    out[(long long)blockIdx.x * dim + k] = xr[k] * r * w[k];
}
// ---- top-2 of materialised logits (the reference scans logits the same way:
// output_top2_partial_scan_probe / _reduce_probe, src/ml/cuda/qwen_output_head_runner.cr:158-338).
// Keys order by value, then by lower index (qmm_common.cuh), so "the two largest keys" are the
// reference's top-1 and top-2 with its tie rule.
struct KeyPair {
  long long k1, k2;  // k1 >= k2
};
__device__ __forceinline__ void pair_insert(KeyPair &p, long long k) {
  if (k > p.k1) {
    p.k2 = p.k1;
    p.k1 = k;
  } else if (k > p.k2) {
    p.k2 = k;
  }
}
__device__ __forceinline__ void pair_merge_shfl(KeyPair &p, int off) {
  const long long o1 = __shfl_xor_sync(0xffffffffu, p.k1, off);
  const long long o2 = __shfl_xor_sync(0xffffffffu, p.k2, off);
  pair_insert(p, o1);
  pair_insert(p, o2);
}

constexpr int kTop2Threads = 256;

__global__ void __launch_bounds__(kTop2Threads)
    top2_scan_kernel(const float *logits, int out_dim, int32_t index_base, unsigned *counters,
                     long long *part_keys, int nparts, int32_t *top_idx, float *top_val,
                     long long *top_key) {
  __shared__ KeyPair s_pair[kTop2Threads / 32];
  __shared__ bool s_last;
  const int b = blockIdx.y, part = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float *row = logits + (long long)b * out_dim;
  KeyPair p{LLONG_MIN, LLONG_MIN};
  for (int i = part * kTop2Threads + threadIdx.x; i < out_dim; i += nparts * kTop2Threads)
    pair_insert(p, top1_key(row[i], (uint32_t)(index_base + i)));
  auto block_merge = [&](KeyPair &q) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) pair_merge_shfl(q, off);
    if (lane == 0) s_pair[warp] = q;
    __syncthreads();
    if (threadIdx.x == 0)
      for (int w = 1; w < kTop2Threads / 32; w++) {
        pair_insert(q, s_pair[w].k1);
        pair_insert(q, s_pair[w].k2);
      }
  };
  block_merge(p);
  if (threadIdx.x == 0) {
    long long *slot = part_keys + ((long long)b * nparts + part) * 2;
    slot[0] = p.k1;
    slot[1] = p.k2;
    __threadfence();
    const unsigned ticket = atomicAdd(&counters[b], 1u);
    s_last = ticket == (unsigned)nparts - 1u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  KeyPair q{LLONG_MIN, LLONG_MIN};
  for (int i = threadIdx.x; i < nparts; i += kTop2Threads) {
    const long long *slot = part_keys + ((long long)b * nparts + i) * 2;
    pair_insert(q, __ldcg(slot));
    pair_insert(q, __ldcg(slot + 1));
  }
  __syncthreads();
  block_merge(q);
  if (threadIdx.x == 0) {
    const long long keys[2] = {q.k1, q.k2};
    for (int i = 0; i < 2; i++) {
      float v;
      uint32_t idx;
      top1_unkey(keys[i], v, idx);
      top_idx[b * 2 + i] = (int32_t)idx;
      top_val[b * 2 + i] = v;
      if (top_key) top_key[b * 2 + i] = keys[i];
    }
    counters[b] = 0u;  // ready for the next call on this scratch buffer
  }
}
}  // namespace

// scratch: counters[batch] (8-byte aligned total) | part keys [batch][nparts][2] | logits [batch][out_dim]
int top2_parts(int out_dim) {
  const int want = (out_dim + kTop2Threads * 8 - 1) / (kTop2Threads * 8);
  return want < 1 ? 1 : (want > 592 ? 592 : want);
}
size_t top2_scratch_bytes(int out_dim, int batch) {
  const size_t counters = ((size_t)batch * 4 + 7) & ~(size_t)7;
  return counters + (size_t)batch * top2_parts(out_dim) * 16 + (size_t)batch * out_dim * 4;
}
int launch_gemv_top2(int type, const void *d_w, const float *d_x, int in_dim, int out_dim, int batch,
                     int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val,
                     long long *d_key, int resident, cudaStream_t s) {
  const int nparts = top2_parts(out_dim);
  const size_t counters = ((size_t)batch * 4 + 7) & ~(size_t)7;
  unsigned *ctr = static_cast<unsigned *>(d_scratch);
  long long *parts = reinterpret_cast<long long *>(static_cast<char *>(d_scratch) + counters);
  float *logits = reinterpret_cast<float *>(parts + (size_t)batch * nparts * 2);
  for (int b0 = 0; b0 < batch; b0 += 16) {  // the GEMV kernels take up to 16 rows a call
    const int nb = batch - b0 < 16 ? batch - b0 : 16;
    const int st = launch_gemv(type, d_w, d_x + (long long)b0 * in_dim, nullptr, 0,
                               logits + (long long)b0 * out_dim, in_dim, out_dim, nb, resident, s);
    if (st) return st;
  }
  top2_scan_kernel<<<dim3(nparts, batch), kTop2Threads, 0, s>>>(logits, out_dim, index_base, ctr, parts,
                                                               nparts, d_idx, d_val, d_key);
  return (int)cudaGetLastError();
}

int launch_rmsnorm(const float *d_x, const float *d_w, float eps, float *d_out, int rows, int dim,
                   cudaStream_t s) {
  rmsnorm_kernel<<<rows, 256, 0, s>>>(d_x, d_w, eps, d_out, dim);
  return (int)cudaGetLastError();
}

int launch_swiglu(const float *d_gate, const float *d_up, float *d_out, int64_t n, cudaStream_t s) {
  swiglu_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(d_gate, d_up, d_out, n);
  return (int)cudaGetLastError();
}

int launch_top1_unpack(const long long *d_keys, int batch, int32_t *d_idx, float *d_val,
                       cudaStream_t s) {
  top1_unpack_kernel<<<(batch + 127) / 128, 128, 0, s>>>(d_keys, batch, d_idx, d_val);
  return (int)cudaGetLastError();
}


}  // namespace cogni
