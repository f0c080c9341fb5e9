// cogni_qmm.hpp — C++17 host-side mirror of the reference's call surface for the quantized
// matmul, layered on the C ABI in cogni_qmm.h (header only; link with -lcogni_qmm).
//
// The names, argument meaning and error behaviour follow the reference's Crystal module so that
// a caller reads the same on both sides:
//   * cogni_qmm::TensorType          ML::GGUF::TensorType            (src/ml/gguf/reader.cr:36-50)
//   * TensorType block geometry      #block_bytes / #block_elements  (src/ml/gguf/reader.cr:53-80)
//   * cogni_qmm::QuantWeight         ML::GGUF::QuantWeight           (src/ml/gguf/compute.cr:20-45)
//   * cogni_qmm::QuantMatmul::matmul_add   ML::GGUF::QuantMatmul.matmul_add
//                                                                    (src/ml/gguf/quant_matmul.cr:13-36)
// Unsupported tensor types raise with the reference's message ("Unsupported quant type for fused
// matmul", quant_matmul.cr:34); any other non-zero status raises std::runtime_error carrying
// cogni_qmm_status_string().  There is no CPU path behind these calls: without a CUDA device the
// compute entry points fail with the CUDA error.
#ifndef COGNI_QMM_HPP
#define COGNI_QMM_HPP

#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "cogni_qmm.h"

namespace cogni_qmm {

enum class TensorType : int {
  Q8_0 = COGNI_QMM_TYPE_Q8_0,
  Q4_K = COGNI_QMM_TYPE_Q4_K,
  Q5_K = COGNI_QMM_TYPE_Q5_K,
  Q6_K = COGNI_QMM_TYPE_Q6_K,
  IQ4_NL = COGNI_QMM_TYPE_IQ4_NL,
};

inline void check(int status, const char *what) {
  if (status == COGNI_QMM_OK) return;
  if (status == COGNI_QMM_ERR_TYPE) throw std::invalid_argument("Unsupported quant type for fused matmul");
  throw std::runtime_error(std::string(what) + ": " + cogni_qmm_status_string(status));
}

// Bytes / elements of one block; throws for a type this engine does not handle.
inline int block_bytes(TensorType t) {
  const int v = cogni_qmm_block_bytes(static_cast<int>(t));
  if (v < 0) throw std::invalid_argument("Unsupported quant type for fused matmul");
  return v;
}
inline int block_elements(TensorType t) {
  const int v = cogni_qmm_block_elements(static_cast<int>(t));
  if (v < 0) throw std::invalid_argument("Unsupported quant type for fused matmul");
  return v;
}
// Bytes of one weight row: in_dim / block_elements blocks (quant_matmul.cr:46-48).
inline std::int64_t row_bytes(TensorType t, int in_dim) {
  const std::int64_t v = cogni_qmm_row_bytes(static_cast<int>(t), in_dim);
  if (v < 0) throw std::invalid_argument("in_dim is not a multiple of the block size, or unsupported type");
  return v;
}

// Raw GGUF bytes of a weight matrix plus its type and dimensions; the bytes are borrowed.
struct QuantWeight {
  const std::uint8_t *raw = nullptr;
  std::int64_t raw_bytes = 0;
  TensorType type = TensorType::Q4_K;
  int out_dim = 0;
  int in_dim = 0;
};

struct QuantMatmul {
  // result[r * out_dim + o] = bias[o] + sum_j x[r * in_dim + j] * dequant(W[o, j]); host buffers in
  // and out, one device round trip per call.
  static std::vector<float> matmul_add(const std::vector<float> &x, int rows, int in_dim,
                                       const std::uint8_t *w_raw, std::int64_t w_bytes,
                                       TensorType w_type, int out_dim, const std::vector<float> &bias) {
    if (static_cast<std::int64_t>(x.size()) < static_cast<std::int64_t>(rows) * in_dim ||
        static_cast<int>(bias.size()) < out_dim)
      throw std::invalid_argument("x or bias shorter than rows*in_dim / out_dim");
    std::vector<float> y(static_cast<std::size_t>(rows) * out_dim);
    check(cogni_qmm_matmul_add_host(x.data(), rows, in_dim, w_raw, w_bytes, static_cast<int>(w_type),
                                    out_dim, bias.data(), y.data()),
          "cogni_qmm_matmul_add_host");
    return y;
  }
  static std::vector<float> matmul_add(const std::vector<float> &x, int rows, const QuantWeight &w,
                                       const std::vector<float> &bias) {
    return matmul_add(x, rows, w.in_dim, w.raw, w.raw_bytes, w.type, w.out_dim, bias);
  }
};

// Device-resident form: the caller owns the device buffers (CUdeviceptr values), as the
// reference's runners do (src/ml/cuda/qwen_recurrent_layer_runner.cr:570-587).
struct DeviceQuantWeight {
  const void *d_raw = nullptr;
  TensorType type = TensorType::Q4_K;
  int out_dim = 0;
  int in_dim = 0;
  bool resident = false;  // bytes complete before the preceding kernel of the stream was launched

  // y[b, :] = addend + W x[b, :]; addend_stride 0 = bias shared by the rows, out_dim = residual
  void gemv(const float *d_x, float *d_y, int batch, const float *d_addend = nullptr,
            std::int64_t addend_stride = 0, void *stream = nullptr) const {
    const auto fn = resident ? cogni_qmm_gemv_resident : cogni_qmm_gemv;
    check(fn(static_cast<int>(type), d_raw, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch,
             stream),
          "cogni_qmm_gemv");
  }
  // y[b, :] = residual[b, :] + W (silu(gate[b, :]) * up[b, :]) (qwen35_cpu.cr:1716-1718);
  // d_x_scratch (f32 [batch, in_dim]) is only needed for shapes the fused kernel does not take
  void gemv_swiglu(const float *d_gate, const float *d_up, float *d_y, int batch,
                   const float *d_residual = nullptr, float *d_x_scratch = nullptr,
                   void *stream = nullptr) const {
    check(cogni_qmm_gemv_swiglu(static_cast<int>(type), d_raw, d_gate, d_up, d_residual,
                                d_residual ? out_dim : 0, d_y, d_x_scratch, in_dim, out_dim, batch,
                                resident ? 1 : 0, stream),
          "cogni_qmm_gemv_swiglu");
  }
  // y[M, out_dim] = x_bf16[M, in_dim] W^T on the tensor cores
  void gemm_bf16(const void *d_x_bf16, void *d_y, int m_rows, int out_type = COGNI_QMM_OUT_F32,
                 void *stream = nullptr) const {
    check(cogni_qmm_gemm_bf16(static_cast<int>(type), d_raw, d_x_bf16, d_y, out_type, m_rows, out_dim,
                              in_dim, stream),
          "cogni_qmm_gemm_bf16");
  }
};

}  // namespace cogni_qmm

#endif  // COGNI_QMM_HPP
