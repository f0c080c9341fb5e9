// Kernel selection for the C-ABI entry points.
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
  if (g_force_rowwarp == 0 && gemv_mma_supports(type, d_w, d_x, in_dim))
    return launch_gemv_mma(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
  return launch_gemv_rowwarp(type, d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, s);
}

int launch_gemv_top1(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                     int batch, int32_t index_base, void *d_scratch, int32_t *d_idx, float *d_val,
                     long long *d_key, cudaStream_t s) {
  if (g_force_rowwarp == 0 && gemv_imma_supports(type, d_w, d_x, in_dim, batch))
    return launch_gemv_top1_imma(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                                 d_idx, d_val, d_key, 0, s);
  if (g_force_rowwarp == 0 && gemv_mma_supports(type, d_w, d_x, in_dim))
    return launch_gemv_top1_mma(type, d_w, d_x, in_dim, out_dim, batch, index_base, d_scratch,
                                d_idx, d_val, d_key, s);
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
}  // namespace

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
