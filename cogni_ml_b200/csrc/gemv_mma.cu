// Tiled decode GEMV for Q4_K / Q5_K / Q6_K straight from the raw GGUF superblocks (sm_100a).
//
// The kernel is HBM-bound: its job is to keep ~100 KB of weight bytes in flight per SM and to
// spend as few issue slots per byte as possible.
//
//  * A persistent CTA per SM walks row tiles of 16 output rows.  One producer warp streams the
//    tile's rows with 1-D bulk async copies (cp.async.bulk, completion on an mbarrier) into a ring
//    of shared-memory stages, KB superblocks of every row per stage; 16 consumer warps split the
//    stage by superblock (Q4_K/Q5_K: KB = 16, one superblock per warp; Q6_K: KB = 8, half a
//    superblock per warp).  Raw rows that are only 2/8-byte aligned (Q6_K) are fetched from the
//    16-byte boundary below and indexed with the remainder.
//  * The activations are split once per CTA into two bf16 planes (x = hi + lo, 16 significant
//    bits) that stay resident in shared memory, with per-group sums for the offset terms.
//  * Quants are widened to bf16 integers with one byte-permute per pair (byte b -> 0x43bb =
//    128 + b, exact) and multiplied on the tensor cores (mma.sync m16n8k16, fp32 accumulate)
//    against the hi and lo planes, one MMA chain per scale group.  The group scale d*sc, decoded
//    once per (row, superblock), is applied in fp32 to the MMA result; the terms that do not
//    depend on the quants (the +128 widening offset, Q6_K's -32, Q4_K/Q5_K's -dmin*m) are folded
//    into one correction per (row, superblock, column) from the per-group sums of x.
//    Integer quants are exact in bf16, so the only deviation from fp32 arithmetic is the 2^-18
//    relative truncation of x.
//  * Per tile the warps' partial sums are added in a fixed order through shared memory, the
//    addend (bias or residual) is added and y is stored.  Results are deterministic.
//
// Every mbarrier wait is bounded by a wall-clock limit; on expiry the kernel records the event in
// a device counter, treats the wait as satisfied and runs to completion (results of that launch
// are then invalid; cogni::gemv_mma_timeouts() reports it).
#include <cuda_bf16.h>

#include <climits>

#include "qmm_common.cuh"

namespace cogni {
namespace {

constexpr int kNW = 16;                      // consumer warps
// One warp issues bulk copies at roughly one per 70-90 cycles however many of its lanes take
// part; the copy unit accepts several times that, so four producer warps share a stage's rows.
constexpr int kPW = 4;                       // producer warps
constexpr int kThreads = (kNW + kPW) * 32;
constexpr int kR = 16;                       // rows per tile
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
// 227 KB per CTA on sm_100, minus room for the kernel's few static __shared__ variables
constexpr size_t kDynSmemMax = 227 * 1024 - 1024;

__device__ unsigned int g_mma_wait_timeouts;
int g_gemv_mma_debug = 0;  // host side: copied into Params::debug

// Row stride of a stage: KB superblocks (+16 B of slack for rows fetched from the 16-byte
// boundary below their start), bumped until the per-lane loads of the MMA phase fall in
// distinct banks (64-bit loads of 4 rows: stride = 32 or 96 mod 128; 32-bit loads of 8 rows:
// stride = odd multiple of 16 mod 128).
constexpr int stage_row_stride(int bb, int kb, bool unaligned_rows) {
  int rs = (bb * kb + (unaligned_rows ? 16 : 0) + 15) / 16 * 16;
  for (;; rs += 16) {
    const int m = rs % 128;
    if (unaligned_rows ? ((m / 16) % 2 == 1) : (m == 32 || m == 96)) return rs;
  }
}

template <int TYPE> struct Cfg;
template <> struct Cfg<kQ4_K> {
  static constexpr int BB = 144, KB = 16, HV = 1, GROUP = 32, NGRP = 8, XPAD = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr float OFF = 128.f;
  static constexpr bool HAS_MIN = true;
};
template <> struct Cfg<kQ5_K> {
  static constexpr int BB = 176, KB = 16, HV = 1, GROUP = 32, NGRP = 8, XPAD = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr float OFF = 128.f;
  static constexpr bool HAS_MIN = true;
};
template <> struct Cfg<kQ6_K> {
  static constexpr int BB = 210, KB = 8, HV = 2, GROUP = 16, NGRP = 16, XPAD = 16;
  static constexpr int RS = stage_row_stride(BB, KB, true);
  static constexpr float OFF = 160.f;  // 128 from the bf16 widening + the format's own -32
  static constexpr bool HAS_MIN = false;
};
static_assert(Cfg<kQ4_K>::RS == 2336 && Cfg<kQ5_K>::RS == 2848 && Cfg<kQ6_K>::RS == 1712, "");

// Batch modes: how the bf16 planes map onto MMA columns.
//   kB1  batch 1      one n-tile, columns (hi, lo), 2-column tables
//   kP4  batch 2..4   one n-tile, columns (hi_0, lo_0, hi_1, lo_1, ...), 8-column tables
//   kN8  batch 5..8   two n-tiles (all hi | all lo) into one accumulator, 8-column tables
enum { kB1 = 0, kP4 = 1, kN8 = 2 };

struct Params {
  const uint8_t *w;
  const float *x;
  const float *addend;
  long long addend_stride;
  float *y;
  int in_dim, out_dim, batch;
  int nblk, nchunks, ntiles, stages;
  long long row_bytes;
  int cs;  // x plane stride in elements
  // shared-memory offsets (bytes)
  int off_red, off_scale, off_xx, off_x, off_stage, stage_bytes;
  // fused top-1 (part_keys == nullptr: plain GEMV)
  long long *part_keys;
  unsigned *counter;
  int32_t *top_idx;
  float *top_val;
  long long *top_key;
  int index_base;
  int debug;  // diagnostics: 1 = stream the stages only, 2 = stream + scale decode
};

// ---------------------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity; gives up after kWaitLimitNs.
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 1;; spin++) {
    if (mbar_try_wait(bar, parity)) return;
    if ((spin & 63u) == 0 && global_ns() - t0 > kWaitLimitNs) {
      atomicAdd(&g_mma_wait_timeouts, 1u);
      return;
    }
  }
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(kNW * 32) : "memory");
}
// d = a * b (fp32 accumulate from zero), m16n8k16, bf16 operands
__device__ __forceinline__ void mma_bf16_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// d += a * b
__device__ __forceinline__ void mma_bf16_acc(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// bytes (b0,b1) / (b2,b3) of v widened to two bf16 values 128 + b (0x43bb), b < 128
__device__ __forceinline__ uint32_t widen01(uint32_t v) { return __byte_perm(v, 0x43434343u, 0x4140); }
__device__ __forceinline__ uint32_t widen23(uint32_t v) { return __byte_perm(v, 0x43434343u, 0x4342); }
// byte i of v as a float, exactly: 0x4B0000bb is 2^23 + b
__device__ __forceinline__ float byte_to_float(uint32_t v, int i) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i)) - 8388608.f;
}

// ---------------------------------------------------------------------------- per-warp decode
// Scale area of one warp: dsc[8][16] floats (the 8 scale groups of this warp's part of the
// superblock, 16 rows), then corr[NCOLS][16] floats.

// Q4_K / Q5_K: lanes (r = lane & 15, half = lane >> 4) decode sub-blocks 4*half .. 4*half+3 of
// row r; the two halves' corrections are combined with one shuffle.
template <int TYPE, int NCOLS>
__device__ __forceinline__ void decode_q45(const uint8_t *blk_row0, int lane, int kblk,
                                           const float *XX, float *area) {
  using C = Cfg<TYPE>;
  const int r = lane & 15, half = lane >> 4;
  const uint4 h = *reinterpret_cast<const uint4 *>(blk_row0 + r * C::RS);
  const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
  const float d = __low2float(dd), dmin = __high2float(dd);
  const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
  // four 6-bit scales / mins of this half as bytes (dequant.cr:240-249, four at a time)
  const uint32_t scw = half ? ((u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u)) : (u0 & 0x3f3f3f3fu);
  const uint32_t mnw = half ? (((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u)) : (u1 & 0x3f3f3f3fu);
  float corr[NCOLS];
#pragma unroll
  for (int c = 0; c < NCOLS; c++) corr[c] = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int s = 4 * half + i;
    const float dsc = d * byte_to_float(scw, i);
    const float dm = dmin * byte_to_float(mnw, i);
    area[s * 16 + r] = dsc;
    const float k = -fmaf(C::OFF, dsc, dm);  // -(128*d*sc + dmin*m)
    const float *xr = XX + (kblk * 8 + s) * NCOLS;
#pragma unroll
    for (int c = 0; c < NCOLS; c += 2) {
      const float2 xv = *reinterpret_cast<const float2 *>(xr + c);
      corr[c] = fmaf(k, xv.x, corr[c]);
      corr[c + 1] = fmaf(k, xv.y, corr[c + 1]);
    }
  }
#pragma unroll
  for (int c = 0; c < NCOLS; c++) {
    corr[c] += __shfl_xor_sync(0xffffffffu, corr[c], 16);
    if (half == 0) area[8 * 16 + c * 16 + r] = corr[c];
  }
}

// Q6_K: this warp owns half `hv` of the superblock (8 scale groups); lanes (r, part) decode
// groups 4*part .. 4*part+3 of that half.
template <int NCOLS>
__device__ __forceinline__ void decode_q6(const uint8_t *blk_row, int lane, int hv, int kblk,
                                          const float *XX, float *area) {
  const int r = lane & 15, part = lane >> 4;
  const float d = load_half_as_float(blk_row + 208);
  const int8_t *sc = reinterpret_cast<const int8_t *>(blk_row + 192 + 8 * hv + 4 * part);
  float corr[NCOLS];
#pragma unroll
  for (int c = 0; c < NCOLS; c++) corr[c] = 0.f;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int j = 4 * part + i;  // group within this half
    const float dsc = d * (float)sc[i];
    area[j * 16 + r] = dsc;
    const float k = -Cfg<kQ6_K>::OFF * dsc;
    const float *xr = XX + (kblk * 16 + 8 * hv + j) * NCOLS;
#pragma unroll
    for (int c = 0; c < NCOLS; c += 2) {
      const float2 xv = *reinterpret_cast<const float2 *>(xr + c);
      corr[c] = fmaf(k, xv.x, corr[c]);
      corr[c + 1] = fmaf(k, xv.y, corr[c + 1]);
    }
  }
#pragma unroll
  for (int c = 0; c < NCOLS; c++) {
    corr[c] += __shfl_xor_sync(0xffffffffu, corr[c], 16);
    if (part == 0) area[8 * 16 + c * 16 + r] = corr[c];
  }
}

// ---------------------------------------------------------------------------- MMA phase
// xcol[j]: this lane's column of n-tile j (lanes whose column is beyond the batch read column 0:
// their MMA output columns are never used).
template <int TYPE, int NT>
__device__ __forceinline__ void process_q45(const uint8_t *blk_row0, int kblk, const float *dsc,
                                            const __nv_bfloat16 *const (&xcol)[NT], int lane,
                                            float (&acc)[4]) {
  using C = Cfg<TYPE>;
  constexpr bool Q5 = TYPE == kQ5_K;
  constexpr int QOFF = Q5 ? 48 : 16;
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const int g = lane >> 2, t = lane & 3;
  const uint8_t *ra = blk_row0 + g * C::RS + 8 * t, *rb = ra + 8 * C::RS;
  uint2 qha = make_uint2(0, 0), qhb = make_uint2(0, 0);
  if constexpr (Q5) {
    qha = *reinterpret_cast<const uint2 *>(ra + 16);
    qhb = *reinterpret_cast<const uint2 *>(rb + 16);
  }
  const __nv_bfloat16 *xk[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) xk[j] = xcol[j] + kblk * 256 + 8 * t;
#pragma unroll
  for (int g4 = 0; g4 < 4; g4++) {
    uint4 blo[NT], bhi[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
      blo[j] = *reinterpret_cast<const uint4 *>(xk[j] + 64 * g4);
      bhi[j] = *reinterpret_cast<const uint4 *>(xk[j] + 64 * g4 + 32);
    }
    const uint2 qa = *reinterpret_cast<const uint2 *>(ra + QOFF + 32 * g4);
    const uint2 qb = *reinterpret_cast<const uint2 *>(rb + QOFF + 32 * g4);
    uint32_t la0 = qa.x & M4, la1 = qa.y & M4, lb0 = qb.x & M4, lb1 = qb.y & M4;
    uint32_t ha0 = (qa.x >> 4) & M4, ha1 = (qa.y >> 4) & M4;
    uint32_t hb0 = (qb.x >> 4) & M4, hb1 = (qb.y >> 4) & M4;
    if constexpr (Q5) {
      // fifth bit: bit 2*g4 of qh for the low-nibble elements, bit 2*g4+1 for the high ones
      constexpr uint32_t M1 = 0x10101010u;
      auto bit = [&](uint32_t q, int b) { return b <= 4 ? ((q << (4 - b)) & M1) : ((q >> (b - 4)) & M1); };
      la0 |= bit(qha.x, 2 * g4);     la1 |= bit(qha.y, 2 * g4);
      lb0 |= bit(qhb.x, 2 * g4);     lb1 |= bit(qhb.y, 2 * g4);
      ha0 |= bit(qha.x, 2 * g4 + 1); ha1 |= bit(qha.y, 2 * g4 + 1);
      hb0 |= bit(qhb.x, 2 * g4 + 1); hb1 |= bit(qhb.y, 2 * g4 + 1);
    }
    float c0[4], c1[4];
    mma_bf16_zero(c0, widen01(la0), widen01(lb0), widen23(la0), widen23(lb0), blo[0].x, blo[0].y);
    mma_bf16_zero(c1, widen01(ha0), widen01(hb0), widen23(ha0), widen23(hb0), bhi[0].x, bhi[0].y);
    mma_bf16_acc(c0, widen01(la1), widen01(lb1), widen23(la1), widen23(lb1), blo[0].z, blo[0].w);
    mma_bf16_acc(c1, widen01(ha1), widen01(hb1), widen23(ha1), widen23(hb1), bhi[0].z, bhi[0].w);
#pragma unroll
    for (int j = 1; j < NT; j++) {
      mma_bf16_acc(c0, widen01(la0), widen01(lb0), widen23(la0), widen23(lb0), blo[j].x, blo[j].y);
      mma_bf16_acc(c1, widen01(ha0), widen01(hb0), widen23(ha0), widen23(hb0), bhi[j].x, bhi[j].y);
      mma_bf16_acc(c0, widen01(la1), widen01(lb1), widen23(la1), widen23(lb1), blo[j].z, blo[j].w);
      mma_bf16_acc(c1, widen01(ha1), widen01(hb1), widen23(ha1), widen23(hb1), bhi[j].z, bhi[j].w);
    }
    const float sa0 = dsc[(2 * g4) * 16 + g], sb0 = dsc[(2 * g4) * 16 + g + 8];
    const float sa1 = dsc[(2 * g4 + 1) * 16 + g], sb1 = dsc[(2 * g4 + 1) * 16 + g + 8];
    acc[0] = fmaf(sa0, c0[0], acc[0]);
    acc[1] = fmaf(sa0, c0[1], acc[1]);
    acc[2] = fmaf(sb0, c0[2], acc[2]);
    acc[3] = fmaf(sb0, c0[3], acc[3]);
    acc[0] = fmaf(sa1, c1[0], acc[0]);
    acc[1] = fmaf(sa1, c1[1], acc[1]);
    acc[2] = fmaf(sb1, c1[2], acc[2]);
    acc[3] = fmaf(sb1, c1[3], acc[3]);
  }
}

// One half (128 elements) of a Q6_K superblock.  base_a / base_b: 4-byte aligned addresses at or
// just below this lane's first byte (ql[64*hv + 4*t]) of rows g and g+8; sh_a / sh_b: 0 or 16,
// the bit offset of the data inside those words.
template <int NT>
__device__ __forceinline__ void process_q6(const uint8_t *base_a, uint32_t sh_a,
                                           const uint8_t *base_b, uint32_t sh_b, int hv, int kblk,
                                           const float *dsc, const __nv_bfloat16 *const (&xcol)[NT],
                                           int lane, float (&acc)[4]) {
  constexpr uint32_t M4 = 0x0f0f0f0fu, M2 = 0x30303030u;
  const int g = lane >> 2, t = lane & 3;
  auto ld = [](const uint8_t *p, uint32_t sh) {
    const uint32_t lo = reinterpret_cast<const uint32_t *>(p)[0];
    const uint32_t hi = reinterpret_cast<const uint32_t *>(p)[1];
    return __funnelshift_r(lo, hi, sh);
  };
  // qh[32*hv + ...] sits 128 - 32*hv bytes after ql[64*hv + ...]
  const int qh_off = 128 - 32 * hv;
  const __nv_bfloat16 *xk[NT];
#pragma unroll
  for (int j = 0; j < NT; j++) xk[j] = xcol[j] + kblk * 256 + 128 * hv + 4 * t;
#pragma unroll
  for (int h = 0; h < 2; h++) {
    uint32_t q[2][4];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      const uint8_t *p = r ? base_b : base_a;
      const uint32_t sh = r ? sh_b : sh_a;
      const uint32_t ql0 = ld(p + 16 * h, sh);
      const uint32_t ql1 = ld(p + 32 + 16 * h, sh);
      const uint32_t qhw = ld(p + qh_off + 16 * h, sh);
      q[r][0] = (ql0 & M4) | ((qhw << 4) & M2);
      q[r][1] = (ql1 & M4) | ((qhw << 2) & M2);
      q[r][2] = ((ql0 >> 4) & M4) | (qhw & M2);
      q[r][3] = ((ql1 >> 4) & M4) | ((qhw >> 2) & M2);
    }
#pragma unroll
    for (int k = 0; k < 4; k++) {
      float c[4];
      const uint2 b0 = *reinterpret_cast<const uint2 *>(xk[0] + 32 * k + 16 * h);
      mma_bf16_zero(c, widen01(q[0][k]), widen01(q[1][k]), widen23(q[0][k]), widen23(q[1][k]),
                    b0.x, b0.y);
#pragma unroll
      for (int j = 1; j < NT; j++) {
        const uint2 bj = *reinterpret_cast<const uint2 *>(xk[j] + 32 * k + 16 * h);
        mma_bf16_acc(c, widen01(q[0][k]), widen01(q[1][k]), widen23(q[0][k]), widen23(q[1][k]),
                     bj.x, bj.y);
      }
      const int j8 = h + 2 * k;  // scale group within this half
      const float sa = dsc[j8 * 16 + g], sb = dsc[j8 * 16 + g + 8];
      acc[0] = fmaf(sa, c[0], acc[0]);
      acc[1] = fmaf(sa, c[1], acc[1]);
      acc[2] = fmaf(sb, c[2], acc[2]);
      acc[3] = fmaf(sb, c[3], acc[3]);
    }
  }
}

// ---------------------------------------------------------------------------- the kernel
template <int TYPE, int MODE>
__global__ void __launch_bounds__(kThreads, 1) gemv_mma_kernel(const Params p) {
  using C = Cfg<TYPE>;
  constexpr bool PAIRED = MODE != kN8;
  constexpr int NT = PAIRED ? 1 : 2;
  constexpr int NCOLS = MODE == kB1 ? 2 : 8;
  constexpr int AREA_FLOATS = 8 * 16 + NCOLS * 16;  // dsc (8 groups) + corr
  static_assert(C::NGRP / C::HV == 8 && C::KB * C::HV == kNW, "each warp handles 8 scale groups");
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);  // full[S], empty[S]
  const int S = p.stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(smem_u32(&bars[s]), kPW);
      mbar_init(smem_u32(&bars[S + s]), kNW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  uint8_t *stages = smem + p.off_stage;

  if (warp >= kNW) {
    // ------------------------------------------------------------------ producer warps
    // every producer warp walks the same chunk sequence; warp pw issues rows 4*pw .. 4*pw+3 and
    // arrives once per chunk with the byte count of its own rows
    const int pw = warp - kNW;
    int it = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
      const int row = tile * kR + lane;
      const bool rvalid = lane < kR && row < p.out_dim;
      const uint8_t *rsrc = p.w + (long long)row * p.row_bytes;
      for (int c = 0; c < p.nchunks; c++, it++) {
        const int s = it % S;
        mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1);
        const int nb = min(C::KB, p.nblk - c * C::KB);
        const uint8_t *src = rsrc + (long long)c * C::KB * C::BB;
        const uint32_t padb = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
        const uint32_t bytes = rvalid ? ((padb + nb * C::BB + 15u) & ~15u) : 0u;
        const bool mine = rvalid && (lane >> 2) == pw;
        const uint32_t my_bytes = __reduce_add_sync(0xffffffffu, mine ? bytes : 0u);
        const uint32_t full = smem_u32(&bars[s]);
        if (lane == 0) mbar_arrive_expect_tx(full, my_bytes);
        __syncwarp();
        if (mine)
          bulk_g2s(smem_u32(stages + (size_t)s * p.stage_bytes + lane * C::RS), src - padb, bytes,
                   full);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int ctid = threadIdx.x;  // 0 .. 511
  __nv_bfloat16 *xsm = reinterpret_cast<__nv_bfloat16 *>(smem + p.off_x);
  float *XX = reinterpret_cast<float *>(smem + p.off_xx);
  const int B = p.batch, K = p.in_dim, CS = p.cs;

  {  // split x into bf16 hi/lo planes and build the per-group sum table
    const int k8n = K >> 3, items = B * k8n;
    constexpr int LPG = C::GROUP / 8;  // lanes per scale group
    for (int i = ctid; i < items; i += kNW * 32) {
      const int b = i / k8n, k = (i - b * k8n) * 8;
      const float4 v0 = __ldg(reinterpret_cast<const float4 *>(p.x + (long long)b * K + k));
      const float4 v1 = __ldg(reinterpret_cast<const float4 *>(p.x + (long long)b * K + k + 4));
      const float v[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
      __nv_bfloat16 hi[8], lo[8];
      float shi = 0.f, slo = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        hi[e] = __float2bfloat16_rn(v[e]);
        const float hf = __bfloat162float(hi[e]);
        lo[e] = __float2bfloat16_rn(v[e] - hf);
        shi += hf;
        slo += __bfloat162float(lo[e]);
      }
      *reinterpret_cast<uint4 *>(xsm + (size_t)b * CS + k) = *reinterpret_cast<uint4 *>(hi);
      *reinterpret_cast<uint4 *>(xsm + (size_t)(B + b) * CS + k) = *reinterpret_cast<uint4 *>(lo);
#pragma unroll
      for (int off = 1; off < LPG; off <<= 1) {
        shi += __shfl_xor_sync(0xffffffffu, shi, off);
        slo += __shfl_xor_sync(0xffffffffu, slo, off);
      }
      if ((lane & (LPG - 1)) == 0) {
        const int grp = k / C::GROUP;
        if (PAIRED) {
          XX[grp * NCOLS + 2 * b] = shi;
          XX[grp * NCOLS + 2 * b + 1] = slo;
        } else {
          XX[grp * NCOLS + b] = shi + slo;
        }
      }
    }
    // table columns beyond the batch are read by the correction loop: keep them finite
    const int used = PAIRED ? 2 * B : B;
    if (used < NCOLS) {
      const int ngroups = K / C::GROUP;
      for (int i = ctid; i < ngroups * (NCOLS - used); i += kNW * 32) {
        const int grp = i / (NCOLS - used), c = used + i % (NCOLS - used);
        XX[grp * NCOLS + c] = 0.f;
      }
    }
  }
  consumer_sync();

  const int g = lane >> 2, t = lane & 3;
  const __nv_bfloat16 *xcol[NT];
  if (PAIRED) {
    const int b = g >> 1, pl = g & 1;
    xcol[0] = xsm + (size_t)(b < B ? (pl ? B : 0) + b : 0) * CS;
  } else {
    const int b = g < B ? g : 0;
    xcol[0] = xsm + (size_t)b * CS;
    xcol[NT - 1] = xsm + (size_t)(B + b) * CS;
  }
  const int xc = 2 * t < NCOLS - 2 ? 2 * t : NCOLS - 2;
  // warp -> (superblock of the stage, half of that superblock)
  const int wkb = warp / C::HV, whv = warp % C::HV;
  float *area = reinterpret_cast<float *>(smem + p.off_scale) + warp * AREA_FLOATS;
  float4 *red = reinterpret_cast<float4 *>(smem + p.off_red);

  long long best[2] = {LLONG_MIN, LLONG_MIN};  // fused top-1: this thread's running maxima

  int it = 0, tcount = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, tcount++) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // byte offset of each row's data inside its stage slot (rows fetched from the boundary below)
    const uintptr_t wbase = reinterpret_cast<uintptr_t>(p.w);
    const int pad_a = (int)((wbase + ((long long)tile * kR + g) * p.row_bytes) & 15);
    const int pad_b = (int)((wbase + ((long long)tile * kR + g + 8) * p.row_bytes) & 15);
    const int pad_d = (int)((wbase + ((long long)tile * kR + (lane & 15)) * p.row_bytes) & 15);

    for (int c = 0; c < p.nchunks; c++, it++) {
      const int s = it % S;
      mbar_wait(smem_u32(&bars[s]), (it / S) & 1);
      const int kblk = c * C::KB + wkb;
      if (kblk < p.nblk && p.debug != 1) {
        const uint8_t *stage = stages + (size_t)s * p.stage_bytes + wkb * C::BB;
        if constexpr (C::HAS_MIN) {
          decode_q45<TYPE, NCOLS>(stage, lane, kblk, XX, area);
          __syncwarp();
          if (p.debug != 2) process_q45<TYPE, NT>(stage, kblk, area, xcol, lane, acc);
        } else {
          decode_q6<NCOLS>(stage + (lane & 15) * C::RS + pad_d, lane, whv, kblk, XX, area);
          __syncwarp();
          const uintptr_t aa = reinterpret_cast<uintptr_t>(stage + g * C::RS + pad_a + 64 * whv + 4 * t);
          const uintptr_t ab = reinterpret_cast<uintptr_t>(stage + (g + 8) * C::RS + pad_b + 64 * whv + 4 * t);
          if (p.debug != 2) process_q6<NT>(reinterpret_cast<const uint8_t *>(aa & ~(uintptr_t)3), (uint32_t)(aa & 2) * 8,
                         reinterpret_cast<const uint8_t *>(ab & ~(uintptr_t)3), (uint32_t)(ab & 2) * 8,
                         whv, kblk, area, xcol, lane, acc);
        }
        const float *corr = area + 8 * 16;
        acc[0] += corr[xc * 16 + g];
        acc[1] += corr[(xc + 1) * 16 + g];
        acc[2] += corr[xc * 16 + g + 8];
        acc[3] += corr[(xc + 1) * 16 + g + 8];
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[S + s]));
    }

    // fixed-order sum of the warps' partial tiles
    float4 *rbuf = red + (size_t)(tcount & 1) * (kNW * 32);
    rbuf[warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    consumer_sync();
    if (ctid < 64) {
      const int hh = ctid & 1, ln = ctid >> 1;
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int ww = 0; ww < kNW; ww++) {
        const float2 pr = reinterpret_cast<const float2 *>(&rbuf[ww * 32 + ln])[hh];
        v0 += pr.x;
        v1 += pr.y;
      }
      const int row = tile * kR + (ln >> 2) + 8 * hh;
      if (row < p.out_dim) {
#pragma unroll
        for (int e = 0; e < (PAIRED ? 1 : 2); e++) {
          // paired modes: the two columns are the hi and lo parts of batch row (ln & 3)
          const int b = PAIRED ? (ln & 3) : 2 * (ln & 3) + e;
          if (b >= B) continue;
          const float val = PAIRED ? v0 + v1 : (e ? v1 : v0);
          if (p.part_keys) {
            const long long key = top1_key(val, (uint32_t)(p.index_base + row));
            best[e] = key > best[e] ? key : best[e];
          } else {
            const float a = p.addend ? p.addend[(long long)b * p.addend_stride + row] : 0.f;
            p.y[(long long)b * p.out_dim + row] = a + val;
          }
        }
      }
    }
  }

  if (p.part_keys == nullptr) return;

  // ------------------------------------------------------------ fused top-1 epilogue
  // per-CTA maximum per batch row -> scratch slot; the CTA with the last ticket folds all slots
  __shared__ long long s_best[16];
  __shared__ bool s_last;
  if (ctid < 16) s_best[ctid] = LLONG_MIN;
  consumer_sync();
  if (ctid < 64) {
    const int ln = ctid >> 1;
    if (PAIRED) {
      if ((ln & 3) < B) atomicMax(&s_best[ln & 3], best[0]);
    } else {
#pragma unroll
      for (int e = 0; e < 2; e++)
        if (2 * (ln & 3) + e < B) atomicMax(&s_best[2 * (ln & 3) + e], best[e]);
    }
  }
  consumer_sync();
  const int nparts = gridDim.x;
  if (ctid < B) p.part_keys[(long long)ctid * nparts + blockIdx.x] = s_best[ctid];
  __threadfence();
  consumer_sync();
  if (ctid == 0) {
    const unsigned ticket = atomicAdd(p.counter, 1u);
    s_last = ticket == (unsigned)nparts - 1u;
  }
  consumer_sync();
  if (!s_last) return;
  __threadfence();
  for (int b = warp; b < B; b += kNW) {
    long long m = LLONG_MIN;
    for (int i = lane; i < nparts; i += 32) {
      const long long k = __ldcg(&p.part_keys[(long long)b * nparts + i]);
      m = k > m ? k : m;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      const long long o = __shfl_xor_sync(0xffffffffu, m, off);
      m = o > m ? o : m;
    }
    if (lane == 0) {
      float v;
      uint32_t idx;
      top1_unkey(m, v, idx);
      p.top_idx[b] = (int32_t)idx;
      p.top_val[b] = v;
      if (p.top_key) p.top_key[b] = m;
    }
  }
  if (ctid == 0) *p.counter = 0u;  // ready for the next call on this scratch buffer
}

// ---------------------------------------------------------------------------- host side
struct Plan {
  size_t smem;
  Params p;
};

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev] > 0 ? cached[dev] : 148;
}

int mode_for_batch(int batch) { return batch == 1 ? kB1 : (batch <= 4 ? kP4 : kN8); }

template <int TYPE>
bool make_plan(int in_dim, int out_dim, int batch, Plan &plan) {
  using C = Cfg<TYPE>;
  const int mode = mode_for_batch(batch);
  const int ncols = mode == kB1 ? 2 : 8;
  const int nblk = in_dim / 256;
  const int ngroups = in_dim / C::GROUP;
  const int cs = in_dim + C::XPAD;
  auto al = [](size_t v) { return (v + 127) & ~(size_t)127; };
  size_t off = 128;
  const size_t off_red = off;    off = al(off + 2ull * kNW * 32 * 16);
  const size_t off_scale = off;  off = al(off + (size_t)kNW * (8 * 16 + ncols * 16) * 4);
  const size_t off_xx = off;     off = al(off + (size_t)ngroups * ncols * 4);
  const size_t off_x = off;      off = al(off + (size_t)2 * batch * cs * 2);
  const size_t off_stage = off;
  const size_t stage_bytes = al((size_t)kR * C::RS);
  if (off_stage + 3 * stage_bytes > kDynSmemMax) return false;
  int stages = (int)((kDynSmemMax - off_stage) / stage_bytes);
  if (stages > 8) stages = 8;
  Params &p = plan.p;
  p.in_dim = in_dim; p.out_dim = out_dim; p.batch = batch;
  p.nblk = nblk; p.nchunks = (nblk + C::KB - 1) / C::KB; p.ntiles = (out_dim + kR - 1) / kR;
  p.stages = stages; p.row_bytes = (long long)nblk * C::BB; p.cs = cs;
  p.off_red = (int)off_red; p.off_scale = (int)off_scale; p.off_xx = (int)off_xx;
  p.off_x = (int)off_x; p.off_stage = (int)off_stage; p.stage_bytes = (int)stage_bytes;
  plan.smem = off_stage + (size_t)stages * stage_bytes;
  return true;
}

template <int TYPE, int MODE>
int launch_instance(const Plan &plan, int grid, cudaStream_t s) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<TYPE, MODE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kDynSmemMax);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  gemv_mma_kernel<TYPE, MODE><<<grid, kThreads, plan.smem, s>>>(plan.p);
  return (int)cudaGetLastError();
}

template <int TYPE>
int run(const Plan &plan, cudaStream_t s) {
  const int sms = sm_count();
  const int grid = plan.p.ntiles < sms ? plan.p.ntiles : sms;
  switch (mode_for_batch(plan.p.batch)) {
    case kB1: return launch_instance<TYPE, kB1>(plan, grid, s);
    case kP4: return launch_instance<TYPE, kP4>(plan, grid, s);
    default: return launch_instance<TYPE, kN8>(plan, grid, s);
  }
}

template <int TYPE>
int gemv_typed(const void *d_w, const float *d_x, const float *d_addend, int64_t addend_stride,
               float *d_y, int in_dim, int out_dim, int batch, const Params *top1, cudaStream_t s) {
  for (int b0 = 0; b0 < batch;) {
    // largest column group (<= 8) whose bf16 planes fit beside three stages
    int nb = batch - b0 > 8 ? 8 : batch - b0;
    Plan plan{};
    while (nb >= 1 && !make_plan<TYPE>(in_dim, out_dim, nb, plan)) nb--;
    if (nb < 1) return COGNI_QMM_ERR_LIMIT;
    Params &p = plan.p;
    p.debug = g_gemv_mma_debug;
    p.w = static_cast<const uint8_t *>(d_w);
    p.x = d_x + (long long)b0 * in_dim;
    p.addend = d_addend ? d_addend + (long long)b0 * addend_stride : nullptr;
    p.addend_stride = addend_stride;
    p.y = d_y ? d_y + (long long)b0 * out_dim : nullptr;
    if (top1) {
      const int sms = sm_count();
      const int grid = p.ntiles < sms ? p.ntiles : sms;
      p.part_keys = top1->part_keys + (long long)b0 * grid;
      p.counter = top1->counter;
      p.top_idx = top1->top_idx + b0;
      p.top_val = top1->top_val + b0;
      p.top_key = top1->top_key ? top1->top_key + b0 : nullptr;
      p.index_base = top1->index_base;
    }
    int st = run<TYPE>(plan, s);
    if (st) return st;
    b0 += nb;
  }
  return COGNI_QMM_OK;
}

}  // namespace

void gemv_mma_set_debug(int mode) { g_gemv_mma_debug = mode; }

bool gemv_mma_supports(int type, const void *d_w, const float *d_x, int in_dim) {
  if (type != kQ4_K && type != kQ5_K && type != kQ6_K) return false;
  if ((reinterpret_cast<uintptr_t>(d_w) & 15) || (reinterpret_cast<uintptr_t>(d_x) & 15)) return false;
  // every batch row of x must start on a 16-byte boundary: in_dim is a multiple of 256
  return in_dim % 256 == 0 && in_dim <= 32768;
}

int launch_gemv_mma(int type, const void *d_w, const float *d_x, const float *d_addend,
                    int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                    cudaStream_t s) {
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, nullptr, s);
    case kQ5_K: return gemv_typed<kQ5_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, nullptr, s);
    case kQ6_K: return gemv_typed<kQ6_K>(d_w, d_x, d_addend, addend_stride, d_y, in_dim, out_dim, batch, nullptr, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

int launch_gemv_top1_mma(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                         int batch, int32_t index_base, void *d_scratch, int32_t *d_idx,
                         float *d_val, long long *d_key, cudaStream_t s) {
  Params t{};
  t.counter = static_cast<unsigned *>(d_scratch);
  t.part_keys = reinterpret_cast<long long *>(static_cast<char *>(d_scratch) +
                                              (((size_t)batch * 4 + 7) & ~(size_t)7));
  t.top_idx = d_idx;
  t.top_val = d_val;
  t.top_key = d_key;
  t.index_base = index_base;
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(d_w, d_x, nullptr, 0, nullptr, in_dim, out_dim, batch, &t, s);
    case kQ5_K: return gemv_typed<kQ5_K>(d_w, d_x, nullptr, 0, nullptr, in_dim, out_dim, batch, &t, s);
    case kQ6_K: return gemv_typed<kQ6_K>(d_w, d_x, nullptr, 0, nullptr, in_dim, out_dim, batch, &t, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

unsigned gemv_mma_timeouts() {
  unsigned v = 0;
  cudaMemcpyFromSymbol(&v, g_mma_wait_timeouts, sizeof(v));
  return v;
}

}  // namespace cogni
