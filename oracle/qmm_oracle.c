/*
 * CPU oracle for the GGUF quantized-matmul path.  TEST INFRASTRUCTURE ONLY —
 * see qmm_oracle.h for what may use it and for the parity-pin status
 * ("parity unpinned" for the Q8_0/Q4_K/Q5_K/Q6_K block arithmetic).
 *
 * Every function names the reference lines it restates.  Arithmetic types follow
 * the reference exactly: bulk dequantisation is all-f32 (dequant.cr), the fused
 * matmul promotes to f64 before the first multiply and keeps one f64 running sum
 * per output that starts at bias[o] (quant_matmul.cr).
 *
 * Build: see the Makefile beside this file (-O2 -ffp-contract=off -fopenmp).
 */
#include "qmm_oracle.h"

#include <math.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QK_K 256

static const int8_t k_iq4nl_values[16] = { /* dequant.cr:11-16 */
    -127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};

int qmm_oracle_block_bytes(int type) { /* reader.cr:53-70 */
  switch (type) {
    case QMM_TYPE_F32: return 4;
    case QMM_TYPE_F16: return 2;
    case QMM_TYPE_Q8_0: return 34;
    case QMM_TYPE_Q4_K: return 144;
    case QMM_TYPE_Q5_K: return 176;
    case QMM_TYPE_Q6_K: return 210;
    case QMM_TYPE_IQ4_NL: return 18;
    default: return -1;
  }
}

int qmm_oracle_block_elements(int type) { /* reader.cr:73-80 */
  switch (type) {
    case QMM_TYPE_F32:
    case QMM_TYPE_F16: return 1;
    case QMM_TYPE_Q8_0:
    case QMM_TYPE_IQ4_NL: return 32;
    case QMM_TYPE_Q4_K:
    case QMM_TYPE_Q5_K:
    case QMM_TYPE_Q6_K: return QK_K;
    default: return -1;
  }
}

int64_t qmm_oracle_row_bytes(int type, int in_dim) {
  int be = qmm_oracle_block_elements(type);
  int bb = qmm_oracle_block_bytes(type);
  if (be < 0) return -1;
  /* K-quants use in_dim // 256 (quant_matmul.cr:47); Q8_0 / IQ4_NL round up
   * (quant_matmul.cr:245, 283). in_dim is a block multiple in every caller. */
  int64_t blocks = (type == QMM_TYPE_Q4_K || type == QMM_TYPE_Q5_K || type == QMM_TYPE_Q6_K)
                       ? in_dim / be
                       : ((int64_t)in_dim + be - 1) / be;
  return blocks * bb;
}

/* dequant.cr:257-283 — software half -> float. Subnormals: mant/1024 * 2^-14,
 * any NaN payload -> the canonical quiet NaN, all in f32 arithmetic. */
float qmm_oracle_fp16_to_f32(uint16_t h) {
  unsigned sign = (h >> 15) & 1u;
  unsigned exp = (h >> 10) & 0x1Fu;
  unsigned mant = h & 0x03FFu;
  float f;
  if (exp == 0) {
    if (mant == 0) return sign ? -0.0f : 0.0f;
    f = (float)mant / 1024.0f;
    f *= 6.103515625e-05f; /* 2^-14 */
    return sign ? -f : f;
  }
  if (exp == 31) {
    if (mant == 0) return sign ? -INFINITY : INFINITY;
    return NAN;
  }
  f = (1.0f + (float)mant / 1024.0f) * ldexpf(1.0f, (int)exp - 15);
  return sign ? -f : f;
}

static inline float half_at(const uint8_t *p) { /* dequant.cr:252-255, little endian */
  return qmm_oracle_fp16_to_f32((uint16_t)(p[0] | ((uint16_t)p[1] << 8)));
}

/* dequant.cr:240-249 */
void qmm_oracle_get_scale_min_k4(int j, const uint8_t *s, float *sc, float *m) {
  if (j < 4) {
    *sc = (float)(s[j] & 63);
    *m = (float)(s[j + 4] & 63);
  } else {
    *sc = (float)((s[j + 4] & 0x0F) | ((s[j - 4] >> 6) << 4));
    *m = (float)((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
  }
}

/* ---------------------------------------------------------------- bulk dequant */

static void deq_q8_0(const uint8_t *data, int64_t n, float *out) { /* dequant.cr:53-71 */
  int64_t nb = (n + 31) / 32;
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t *b = data + i * 34;
    float d = half_at(b);
    const int8_t *qs = (const int8_t *)(b + 2);
    int64_t base = i * 32;
    int64_t count = n - base < 32 ? n - base : 32;
    for (int64_t j = 0; j < count; j++) out[base + j] = d * (float)qs[j];
  }
}

static void deq_iq4_nl(const uint8_t *data, int64_t n, float *out) { /* dequant.cr:76-101 */
  int64_t nb = (n + 31) / 32;
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t *b = data + i * 18;
    float d = half_at(b);
    const uint8_t *qs = b + 2;
    int64_t base = i * 32;
    int64_t c1 = n - base < 16 ? n - base : 16;
    for (int64_t j = 0; j < c1; j++) out[base + j] = d * (float)k_iq4nl_values[qs[j] & 0x0F];
    int64_t base2 = base + 16;
    int64_t c2 = n - base2 < 16 ? n - base2 : 16;
    for (int64_t j = 0; j < c2; j++) out[base2 + j] = d * (float)k_iq4nl_values[qs[j] >> 4];
  }
}

static void deq_q4_k(const uint8_t *data, int64_t n, float *out) { /* dequant.cr:106-142 */
  int64_t nb = n / QK_K;
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t *b = data + i * 144;
    float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
    float *y = out + i * QK_K;
    for (int pair = 0; pair < 4; pair++) {
      float sc, m, sc2, m2;
      qmm_oracle_get_scale_min_k4(2 * pair, scales, &sc, &m);
      qmm_oracle_get_scale_min_k4(2 * pair + 1, scales, &sc2, &m2);
      float d1 = d * sc, m1 = dmin * m;
      float d2 = d * sc2, m2f = dmin * m2;
      for (int l = 0; l < 32; l++) y[l] = d1 * (float)(qs[l] & 0x0F) - m1;
      for (int l = 0; l < 32; l++) y[32 + l] = d2 * (float)(qs[l] >> 4) - m2f;
      qs += 32;
      y += 64;
    }
  }
}

static void deq_q5_k(const uint8_t *data, int64_t n, float *out) { /* dequant.cr:146-193 */
  int64_t nb = n / QK_K;
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t *b = data + i * 176;
    float d = half_at(b), dmin = half_at(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    float *y = out + i * QK_K;
    uint8_t u1 = 1, u2 = 2;
    for (int pair = 0; pair < 4; pair++) {
      float sc, m, sc2, m2v;
      qmm_oracle_get_scale_min_k4(2 * pair, scales, &sc, &m);
      qmm_oracle_get_scale_min_k4(2 * pair + 1, scales, &sc2, &m2v);
      float d1 = d * sc, m1 = dmin * m;
      float d2 = d * sc2, m2 = dmin * m2v;
      for (int l = 0; l < 32; l++) {
        int q = (ql[l] & 0x0F) + ((qh[l] & u1) ? 16 : 0);
        y[l] = d1 * (float)q - m1;
      }
      for (int l = 0; l < 32; l++) {
        int q = ((ql[l] >> 4) & 0x0F) + ((qh[l] & u2) ? 16 : 0);
        y[32 + l] = d2 * (float)q - m2;
      }
      ql += 32;
      y += 64;
      u1 = (uint8_t)(u1 << 2);
      u2 = (uint8_t)(u2 << 2);
    }
  }
}

/* The four 6-bit quants a Q6_K lane produces (dequant.cr:214-217, quant_matmul.cr:198-201) */
static inline void q6k_quads(const uint8_t *ql, const uint8_t *qh, int l, int q[4]) {
  int h = qh[l];
  q[0] = ((ql[l] & 0xF) | (((h >> 0) & 3) << 4)) - 32;
  q[1] = ((ql[l + 32] & 0xF) | (((h >> 2) & 3) << 4)) - 32;
  q[2] = ((ql[l] >> 4) | (((h >> 4) & 3) << 4)) - 32;
  q[3] = ((ql[l + 32] >> 4) | (((h >> 6) & 3) << 4)) - 32;
}

static void deq_q6_k(const uint8_t *data, int64_t n, float *out) { /* dequant.cr:197-236 */
  int64_t nb = n / QK_K;
  for (int64_t i = 0; i < nb; i++) {
    const uint8_t *b = data + i * 210;
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    float d = half_at(b + 208);
    float *y = out + i * QK_K;
    for (int half = 0; half < 2; half++) {
      for (int l = 0; l < 32; l++) {
        int is = l / 16, q[4];
        q6k_quads(ql, qh, l, q);
        /* left-associative: (d * sc) * q, dequant.cr:224-227 */
        y[l] = d * (float)sc[is] * (float)q[0];
        y[l + 32] = d * (float)sc[is + 2] * (float)q[1];
        y[l + 64] = d * (float)sc[is + 4] * (float)q[2];
        y[l + 96] = d * (float)sc[is + 6] * (float)q[3];
      }
      y += 128;
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
}

int qmm_oracle_dequantize(int type, const uint8_t *data, int64_t n, float *out) {
  switch (type) { /* dequant.cr:20-32 */
    case QMM_TYPE_F32: memcpy(out, data, (size_t)n * 4); return 0;
    case QMM_TYPE_F16:
      for (int64_t i = 0; i < n; i++) out[i] = half_at(data + 2 * i);
      return 0;
    case QMM_TYPE_Q8_0: deq_q8_0(data, n, out); return 0;
    case QMM_TYPE_Q4_K: deq_q4_k(data, n, out); return 0;
    case QMM_TYPE_Q5_K: deq_q5_k(data, n, out); return 0;
    case QMM_TYPE_Q6_K: deq_q6_k(data, n, out); return 0;
    case QMM_TYPE_IQ4_NL: deq_iq4_nl(data, n, out); return 0;
    default: return -1;
  }
}

/* ---------------------------------------------------------------- fused matmul
 * One function per type returns the f64 sum for one (x row, W row) pair, started
 * at `sum` (= bias[o]) and advanced in the reference's block/group/lane order. */

static double dot_q4_k(const float *x, const uint8_t *w, int in_dim, double sum) {
  int nblk = in_dim / QK_K; /* quant_matmul.cr:46-96 */
  for (int blk = 0; blk < nblk; blk++) {
    const uint8_t *b = w + (size_t)blk * 144;
    double d = (double)half_at(b), dmin = (double)half_at(b + 2);
    const uint8_t *scales = b + 4, *qs = b + 16;
    const float *xb = x + (size_t)blk * QK_K;
    for (int pair = 0; pair < 4; pair++) {
      float sc, m, sc2, m2;
      qmm_oracle_get_scale_min_k4(2 * pair, scales, &sc, &m);
      qmm_oracle_get_scale_min_k4(2 * pair + 1, scales, &sc2, &m2);
      double d1 = d * (double)sc, m1 = dmin * (double)m;
      double d2 = d * (double)sc2, m2v = dmin * (double)m2;
      for (int l = 0; l < 32; l++) {
        double val = d1 * (double)(int)(qs[l] & 0x0F) - m1;
        sum += (double)xb[pair * 64 + l] * val;
      }
      for (int l = 0; l < 32; l++) {
        double val = d2 * (double)(int)(qs[l] >> 4) - m2v;
        sum += (double)xb[pair * 64 + 32 + l] * val;
      }
      qs += 32;
    }
  }
  return sum;
}

static double dot_q5_k(const float *x, const uint8_t *w, int in_dim, double sum) {
  int nblk = in_dim / QK_K; /* quant_matmul.cr:108-165 */
  for (int blk = 0; blk < nblk; blk++) {
    const uint8_t *b = w + (size_t)blk * 176;
    double d = (double)half_at(b), dmin = (double)half_at(b + 2);
    const uint8_t *scales = b + 4, *qh = b + 16, *ql = b + 48;
    const float *xb = x + (size_t)blk * QK_K;
    uint8_t u1 = 1, u2 = 2;
    for (int pair = 0; pair < 4; pair++) {
      float sc, m, sc2, m2;
      qmm_oracle_get_scale_min_k4(2 * pair, scales, &sc, &m);
      qmm_oracle_get_scale_min_k4(2 * pair + 1, scales, &sc2, &m2);
      double d1 = d * (double)sc, m1 = dmin * (double)m;
      double d2 = d * (double)sc2, m2v = dmin * (double)m2;
      for (int l = 0; l < 32; l++) {
        int q = (ql[l] & 0x0F) + ((qh[l] & u1) ? 16 : 0);
        sum += (double)xb[pair * 64 + l] * (d1 * (double)q - m1);
      }
      for (int l = 0; l < 32; l++) {
        int q = ((ql[l] >> 4) & 0x0F) + ((qh[l] & u2) ? 16 : 0);
        sum += (double)xb[pair * 64 + 32 + l] * (d2 * (double)q - m2v);
      }
      ql += 32;
      u1 = (uint8_t)(u1 << 2);
      u2 = (uint8_t)(u2 << 2);
    }
  }
  return sum;
}

static double dot_q6_k(const float *x, const uint8_t *w, int in_dim, double sum) {
  int nblk = in_dim / QK_K; /* quant_matmul.cr:176-228 */
  for (int blk = 0; blk < nblk; blk++) {
    const uint8_t *b = w + (size_t)blk * 210;
    const uint8_t *ql = b, *qh = b + 128;
    const int8_t *sc = (const int8_t *)(b + 192);
    double d = (double)half_at(b + 208);
    const float *xb = x + (size_t)blk * QK_K;
    for (int half = 0; half < 2; half++) {
      const float *xh = xb + half * 128;
      for (int l = 0; l < 32; l++) {
        int is = l / 16, q[4];
        q6k_quads(ql, qh, l, q);
        sum += (double)xh[l] * (d * (double)sc[is] * (double)q[0]);
        sum += (double)xh[l + 32] * (d * (double)sc[is + 2] * (double)q[1]);
        sum += (double)xh[l + 64] * (d * (double)sc[is + 4] * (double)q[2]);
        sum += (double)xh[l + 96] * (d * (double)sc[is + 6] * (double)q[3]);
      }
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
  return sum;
}

static double dot_q8_0(const float *x, const uint8_t *w, int in_dim, double sum) {
  int nblk = (in_dim + 31) / 32; /* quant_matmul.cr:240-267 */
  for (int blk = 0; blk < nblk; blk++) {
    const uint8_t *b = w + (size_t)blk * 34;
    double d = (double)half_at(b);
    const int8_t *qs = (const int8_t *)(b + 2);
    int base = blk * 32;
    int count = in_dim - base < 32 ? in_dim - base : 32;
    for (int j = 0; j < count; j++) sum += (double)x[base + j] * (d * (double)qs[j]);
  }
  return sum;
}

static double dot_iq4_nl(const float *x, const uint8_t *w, int in_dim, double sum) {
  int nblk = (in_dim + 31) / 32; /* quant_matmul.cr:278-316 */
  for (int blk = 0; blk < nblk; blk++) {
    const uint8_t *b = w + (size_t)blk * 18;
    double d = (double)half_at(b);
    const uint8_t *qs = b + 2;
    int base = blk * 32;
    int c1 = in_dim - base < 16 ? in_dim - base : 16;
    for (int j = 0; j < c1; j++)
      sum += (double)x[base + j] * (d * (double)k_iq4nl_values[qs[j] & 0x0F]);
    int base2 = base + 16;
    int c2 = in_dim - base2 < 16 ? in_dim - base2 : 16;
    for (int j = 0; j < c2; j++)
      sum += (double)x[base2 + j] * (d * (double)k_iq4nl_values[qs[j] >> 4]);
  }
  return sum;
}

typedef double (*dot_fn)(const float *, const uint8_t *, int, double);

static dot_fn pick_dot(int type) { /* quant_matmul.cr:25-35 */
  switch (type) {
    case QMM_TYPE_Q4_K: return dot_q4_k;
    case QMM_TYPE_Q5_K: return dot_q5_k;
    case QMM_TYPE_Q6_K: return dot_q6_k;
    case QMM_TYPE_Q8_0: return dot_q8_0;
    case QMM_TYPE_IQ4_NL: return dot_iq4_nl;
    default: return NULL;
  }
}

int qmm_oracle_matmul_add_range(int type, const float *x, int rows, int in_dim,
                                const uint8_t *w_raw, int out_dim, const float *bias,
                                float *y, int o_begin, int o_end, int threads) {
  dot_fn dot = pick_dot(type);
  if (!dot) return -1;
  int64_t row_bytes = qmm_oracle_row_bytes(type, in_dim);
  if (o_begin < 0) o_begin = 0;
  if (o_end > out_dim) o_end = out_dim;
  if (threads < 1) threads = 1;
  for (int r = 0; r < rows; r++) { /* rows outermost, quant_matmul.cr:52 */
    const float *xr = x + (size_t)r * in_dim;
    float *yr = y + (size_t)r * out_dim;
#ifdef _OPENMP
#pragma omp parallel for schedule(static) num_threads(threads) if (threads > 1)
#endif
    for (int o = o_begin; o < o_end; o++) {
      double sum = dot(xr, w_raw + (size_t)o * row_bytes, in_dim, (double)bias[o]);
      yr[o] = (float)sum; /* .to_f32, quant_matmul.cr:93 */
    }
  }
  return 0;
}

int qmm_oracle_matmul_add(int type, const float *x, int rows, int in_dim,
                          const uint8_t *w_raw, int out_dim, const float *bias, float *y) {
  return qmm_oracle_matmul_add_range(type, x, rows, in_dim, w_raw, out_dim, bias, y, 0,
                                     out_dim, 1);
}

int qmm_oracle_matmul_add_mt(int type, const float *x, int rows, int in_dim,
                             const uint8_t *w_raw, int out_dim, const float *bias,
                             float *y, int threads) {
  return qmm_oracle_matmul_add_range(type, x, rows, in_dim, w_raw, out_dim, bias, y, 0,
                                     out_dim, threads);
}

/* src/ml/gguf/qwen35_cpu.cr:517-519 (silu) and :1716-1717 (combined = silu(gate) * up), f32 */
void qmm_oracle_swiglu(const float *gate, const float *up, int64_t n, float *out) {
  for (int64_t i = 0; i < n; i++) {
    const float v = gate[i];
    const float s = v / (1.0f + expf(-v));
    out[i] = s * up[i];
  }
}

/* src/ml/gguf/qwen35_cpu.cr:484-490 / 1492-1504 */
void qmm_oracle_rmsnorm(const float *x, int rows, int dim, const float *w, float eps, float *out) {
  for (int r = 0; r < rows; r++) {
    const float *xr = x + (int64_t)r * dim;
    double ss = 0.0;
    for (int j = 0; j < dim; j++) ss += (double)xr[j] * (double)xr[j];
    const float inv_rms = (float)(1.0 / sqrt(ss / (double)dim + (double)eps));
    for (int j = 0; j < dim; j++) {
      const float t = xr[j] * inv_rms;
      out[(int64_t)r * dim + j] = t * w[j];
    }
  }
}

void qmm_oracle_top1(const float *logits, int64_t n, int32_t *index, float *value) {
  /* qwen35_cpu.cr:2053-2055: maxv = logits.max; index of its first occurrence.
   * Equivalent to an ascending scan that replaces only on strict '>'. */
  int64_t best = 0;
  float bv = logits[0];
  for (int64_t i = 1; i < n; i++) {
    if (logits[i] > bv) {
      bv = logits[i];
      best = i;
    }
  }
  *index = (int32_t)best;
  *value = bv;
}

int qmm_oracle_max_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
