/*
 * CPU oracle for the GGUF quantized-matmul path.  TEST INFRASTRUCTURE ONLY.
 *
 * This is a plain-C restatement of the reference's CPU algorithm
 * (src/ml/gguf/dequant.cr and src/ml/gguf/quant_matmul.cr).  It is the checker the
 * CUDA path is compared against and the timed CPU baseline; it is never part of
 * the shipped product path.  Only tests, the smoke check and the CPU-baseline
 * legs of the benchmark may link or load it.
 *
 * PARITY PIN STATUS: pinned by the reference's own CUDA kernels.  The reference is written in
 * Crystal, which cannot be built where this oracle is developed, and it holds no golden vectors
 * for Q8_0/Q4_K/Q5_K/Q6_K; but it ships an independent implementation of the same arithmetic as
 * PTX text (src/ml/cuda/kernels/q4k_gemv_probe.ptx, q5k_gemv_probe.ptx, q6k_gemv_probe.ptx,
 * q4k_dual_gemv_probe.ptx, bin/cuda_q8_gemv_probe.cr:39-227,
 * src/ml/cuda/qwen_output_head_runner.cr:14-625).  oracle/make_ref.py assembles that text,
 * unmodified, into oracle/_ref/*.cubin and tests/test_gpu_reference_ptx.py runs it on the GPU
 * against this oracle on the same seeded tensors, inside the reference probes' own thresholds
 * (cos >= 0.99999, max_diff <= 1e-3; Q8_0: 0.999999, 1e-4), for the single-token, four-token,
 * row-batched, residual-add, dual and fused top-1 kernels.  The helpers shared by every type
 * (fp16_to_f32, the bias-seeded f64 accumulator, the nibble order) are also pinned through the one
 * synthetic known-answer spec the reference has (spec/iq4_nl_dequant_spec.cr:34-106).
 */
#ifndef QMM_ORACLE_H
#define QMM_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ggml tensor type ids, src/ml/gguf/reader.cr:36-50 */
enum {
  QMM_TYPE_F32 = 0,
  QMM_TYPE_F16 = 1,
  QMM_TYPE_Q8_0 = 8,
  QMM_TYPE_Q4_K = 12,
  QMM_TYPE_Q5_K = 13,
  QMM_TYPE_Q6_K = 14,
  QMM_TYPE_IQ4_NL = 20
};

/* reader.cr:53-78 */
int qmm_oracle_block_bytes(int type);
int qmm_oracle_block_elements(int type);
/* bytes of one weight row of in_dim elements (quant_matmul.cr:46-48, 245-246) */
int64_t qmm_oracle_row_bytes(int type, int in_dim);

/* dequant.cr:252-283 */
float qmm_oracle_fp16_to_f32(uint16_t h);
/* dequant.cr:240-249 */
void qmm_oracle_get_scale_min_k4(int j, const uint8_t *scales, float *sc, float *m);

/* dequant.cr:20-32 dispatch; returns 0, or -1 for an unsupported type */
int qmm_oracle_dequantize(int type, const uint8_t *data, int64_t n, float *out);

/* quant_matmul.cr:20-36 dispatch; y is [rows, out_dim]; bias has out_dim entries.
 * Returns 0, or -1 for an unsupported type. Single thread, reference loop order. */
int qmm_oracle_matmul_add(int type, const float *x, int rows, int in_dim,
                          const uint8_t *w_raw, int out_dim, const float *bias,
                          float *y);

/* Same arithmetic per output element, output rows spread over `threads` OpenMP
 * threads (each y[r,o] is still one sequential f64 sum, so results are identical). */
int qmm_oracle_matmul_add_mt(int type, const float *x, int rows, int in_dim,
                             const uint8_t *w_raw, int out_dim, const float *bias,
                             float *y, int threads);

/* Only output rows [o_begin, o_end) of W are evaluated; y keeps the full
 * [rows, out_dim] shape and untouched entries are left as they were.
 * Used for bounded CPU-baseline samples and prefill row-subset checks. */
int qmm_oracle_matmul_add_range(int type, const float *x, int rows, int in_dim,
                                const uint8_t *w_raw, int out_dim, const float *bias,
                                float *y, int o_begin, int o_end, int threads);

/* qwen35_cpu.cr:2052-2055: max value, then its first index (highest value,
 * lowest index wins ties). */
void qmm_oracle_top1(const float *logits, int64_t n, int32_t *index, float *value);

/* SwiGLU product of the FFN: out[i] = silu(gate[i]) * up[i], silu(v) = v / (1 + exp(-v)), all in
 * f32 (src/ml/gguf/qwen35_cpu.cr:512-519 silu, :1716-1717 gate_ff * up_ff). */
void qmm_oracle_swiglu(const float *gate, const float *up, int64_t n, float *out);

/* RMSNorm of `rows` rows of `dim` elements: out = x * inv_rms * w with the sum of squares in f64,
 * inv_rms = (float)(1 / sqrt(ss / dim + eps)) and the two products in f32 from left to right
 * (src/ml/gguf/qwen35_cpu.cr:484-490 rms_norm, :1492-1504 rms_norm_rows). */
void qmm_oracle_rmsnorm(const float *x, int rows, int dim, const float *w, float eps, float *out);

int qmm_oracle_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
