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
}  // namespace

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
