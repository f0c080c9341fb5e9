// Compiled and run by tests/test_cpp_host_mirror.py: the C++ host mirror against the C ABI,
// on the paths that need no GPU (geometry, argument checks, the reference's error text).
#include <cstdio>
#include <cstring>
#include <vector>

#include "cogni_qmm.hpp"

#define EXPECT(cond)                                              \
  do {                                                            \
    if (!(cond)) {                                                \
      std::printf("FAILED: %s (line %d)\n", #cond, __LINE__);     \
      return 1;                                                   \
    }                                                             \
  } while (0)

int main() {
  using namespace cogni_qmm;
  EXPECT(cogni_qmm_abi_version() == COGNI_QMM_ABI_VERSION);
  // block geometry, TensorType#block_bytes / #block_elements (src/ml/gguf/reader.cr:53-80)
  EXPECT(block_bytes(TensorType::Q8_0) == 34 && block_elements(TensorType::Q8_0) == 32);
  EXPECT(block_bytes(TensorType::Q4_K) == 144 && block_elements(TensorType::Q4_K) == 256);
  EXPECT(block_bytes(TensorType::Q5_K) == 176 && block_elements(TensorType::Q5_K) == 256);
  EXPECT(block_bytes(TensorType::Q6_K) == 210 && block_elements(TensorType::Q6_K) == 256);
  EXPECT(row_bytes(TensorType::Q4_K, 4096) == 16 * 144);
  EXPECT(row_bytes(TensorType::Q6_K, 12288) == 48 * 210);
  bool threw = false;
  try {
    row_bytes(TensorType::Q4_K, 100);
  } catch (const std::invalid_argument &) {
    threw = true;
  }
  EXPECT(threw);
  // an unsupported type raises with the reference's message before anything touches a device
  threw = false;
  std::vector<float> x(256, 1.f), bias(4, 0.f);
  std::vector<std::uint8_t> raw(4 * 144, 0);
  try {
    QuantMatmul::matmul_add(x, 1, 256, raw.data(), (std::int64_t)raw.size(), static_cast<TensorType>(2), 4, bias);
  } catch (const std::invalid_argument &e) {
    threw = std::strcmp(e.what(), "Unsupported quant type for fused matmul") == 0;
  }
  EXPECT(threw);
  // too few weight bytes is an argument error, not a crash
  threw = false;
  try {
    QuantMatmul::matmul_add(x, 1, 256, raw.data(), 10, TensorType::Q4_K, 4, bias);
  } catch (const std::runtime_error &e) {
    threw = std::strstr(e.what(), "cogni_qmm_matmul_add_host") != nullptr;
  }
  EXPECT(threw);
  // short x is caught on the host side of the mirror
  threw = false;
  try {
    std::vector<float> shortx(10, 0.f);
    QuantMatmul::matmul_add(shortx, 1, 256, raw.data(), (std::int64_t)raw.size(), TensorType::Q4_K, 4, bias);
  } catch (const std::invalid_argument &) {
    threw = true;
  }
  EXPECT(threw);
  std::printf("ok\n");
  return 0;
}
