// Tiled decode GEMV for Q4_K / Q5_K / Q6_K straight from the raw GGUF superblocks (sm_100a).
//
// The kernel is HBM-bound: its job is to keep ~100 KB of weight bytes in flight per SM and to
// spend as few issue slots per byte as possible.
//
//  * A persistent CTA per SM walks row tiles of 16*MT output rows.  One producer warp streams the
//    tile's rows with 1-D bulk async copies (cp.async.bulk, completion on an mbarrier) into a ring
//    of shared-memory stages, 8 superblocks (2048 columns) of every row per stage; 8 consumer
//    warps each take one superblock of the stage.  Raw rows that are only 2/8-byte aligned
//    (Q6_K) are fetched from the 16-byte boundary below and indexed with the remainder.
//  * The activations are split once per CTA into two bf16 planes (x = hi + lo, 16 significant
//    bits) that stay resident in shared memory, with per-group sums for the offset terms.
//  * Quants are widened to bf16 integers with one byte-permute per pair (byte b -> 0x43bb =
//    128 + b, exact), multiplied on the tensor cores (mma.sync m16n8k16, fp32 accumulate) against
//    the hi and lo planes; the accumulator is pre-loaded with -offset * sum(x) so the MMA result
//    is sum(q * x) of one scale group.  The per-group scale d*sc (and -dmin*m for Q4_K/Q5_K),
//    decoded once per (row, superblock) by one lane, is applied in fp32 to the MMA result.
//    Integer quants are exact in bf16, so the only deviation from fp32 arithmetic is the 2^-18
//    relative truncation of x.
//  * Per tile the 8 warps' partial sums are added in a fixed order through shared memory, the
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

constexpr int kNW = 8;                       // consumer warps = superblocks per stage
constexpr int kThreads = (kNW + 1) * 32;     // + 1 producer warp
constexpr unsigned long long kWaitLimitNs = 2000000000ull;
// 227 KB per CTA on sm_100, minus room for the kernel's few static __shared__ variables
constexpr size_t kDynSmemMax = 227 * 1024 - 1024;

__device__ unsigned int g_mma_wait_timeouts;

template <int TYPE> struct Cfg;
template <> struct Cfg<kQ4_K> {
  static constexpr int BB = 144, RS = 1184, GROUP = 32, NGRP = 8, XPAD = 32, SCB = 8;
  static constexpr float OFF = 128.f;
  static constexpr bool HAS_MIN = true;
};
template <> struct Cfg<kQ5_K> {
  static constexpr int BB = 176, RS = 1440, GROUP = 32, NGRP = 8, XPAD = 32, SCB = 8;
  static constexpr float OFF = 128.f;
  static constexpr bool HAS_MIN = true;
};
template <> struct Cfg<kQ6_K> {
  static constexpr int BB = 210, RS = 1712, GROUP = 16, NGRP = 16, XPAD = 16, SCB = 4;
  static constexpr float OFF = 160.f;  // 128 from the bf16 widening + the format's own -32
  static constexpr bool HAS_MIN = false;
};

struct Params {
  const uint8_t *w;
  const float *x;
  const float *addend;
  long long addend_stride;
  float *y;
  int in_dim, out_dim, batch;
  int nblk, nchunks, ntiles, stages;
  long long row_bytes;
  int ncols;      // columns of the X tables
  int cs;         // x plane stride in elements
  // shared-memory offsets (bytes)
  int off_red, off_scale, off_xn, off_xx, off_x, off_stage, stage_bytes;
  // fused top-1 (nullptr = plain GEMV)
  long long *part_keys;
  unsigned *counter;
  int32_t *top_idx;
  float *top_val;
  long long *top_key;
  int index_base;
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
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// bytes (b0,b1) / (b2,b3) of v widened to two bf16 values 128 + b (0x43bb), b < 128
__device__ __forceinline__ uint32_t widen01(uint32_t v) { return __byte_perm(v, 0x43434343u, 0x4140); }
__device__ __forceinline__ uint32_t widen23(uint32_t v) { return __byte_perm(v, 0x43434343u, 0x4342); }
// 32-bit load from a 2-byte aligned shared address
__device__ __forceinline__ uint32_t lds32_unaligned(const uint8_t *p) {
  uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
  return __funnelshift_r(q[0], q[1], (uint32_t)(a & 2) * 8);
}

// ---------------------------------------------------------------------------- scale decode
// Lane r (< 16*MT) decodes the scales of (row r, this warp's superblock) into the warp's area.
template <int TYPE, int MT>
__device__ __forceinline__ void decode_scales(const uint8_t *blk, int lane, void *area) {
  using C = Cfg<TYPE>;
  constexpr int R = 16 * MT;
  if (lane >= R) return;
  if constexpr (C::HAS_MIN) {
    const uint4 h = *reinterpret_cast<const uint4 *>(blk);
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    const float d = __low2float(dd), dmin = __high2float(dd);
    const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
    const uint32_t sc_lo = u0 & 0x3f3f3f3fu, mn_lo = u1 & 0x3f3f3f3fu;
    const uint32_t sc_hi = (u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u);
    const uint32_t mn_hi = ((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u);
    float2 *out = reinterpret_cast<float2 *>(area);
#pragma unroll
    for (int s = 0; s < 8; s++) {
      const uint32_t scw = s < 4 ? sc_lo : sc_hi, mnw = s < 4 ? mn_lo : mn_hi;
      const float sc = (float)((scw >> (8 * (s & 3))) & 0xff);
      const float mn = (float)((mnw >> (8 * (s & 3))) & 0xff);
      out[s * R + lane] = make_float2(d * sc, -(dmin * mn));
    }
  } else {
    const float d = load_half_as_float(blk + 208);
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192);
    float *out = reinterpret_cast<float *>(area);
#pragma unroll
    for (int j = 0; j < 16; j++) out[j * R + lane] = d * (float)sc[j];
  }
}

// ---------------------------------------------------------------------------- MMA phase
template <int NT>
struct XCols {
  const __nv_bfloat16 *col[NT];  // this lane's column of each n-tile
  bool valid;                    // lane's column holds data (else it multiplies zeros)
};

template <int TYPE, int MT, int NT>
__device__ __forceinline__ void process_q45(const uint8_t *stage, int wblk, int kblk,
                                            const float2 *sc, const float *XN, const float *XX,
                                            int ncols, int xc, const XCols<NT> &xs, int lane,
                                            float (&acc)[MT][4]) {
  using C = Cfg<TYPE>;
  constexpr bool Q5 = TYPE == kQ5_K;
  constexpr int QOFF = Q5 ? 48 : 16, R = 16 * MT;
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const int g = lane >> 2, t = lane & 3;
  const uint8_t *rb = stage + wblk * C::BB;
  uint2 qh[MT][2];
  if constexpr (Q5) {
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      qh[mt][0] = *reinterpret_cast<const uint2 *>(rb + (16 * mt + g) * C::RS + 16 + 8 * t);
      qh[mt][1] = *reinterpret_cast<const uint2 *>(rb + (16 * mt + g + 8) * C::RS + 16 + 8 * t);
    }
  }
#pragma unroll
  for (int g4 = 0; g4 < 4; g4++) {
    const int kel = kblk * 256 + 64 * g4 + 8 * t;
    uint4 blo[NT], bhi[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) {
      blo[j] = bhi[j] = make_uint4(0, 0, 0, 0);
      if (xs.valid) {
        blo[j] = *reinterpret_cast<const uint4 *>(xs.col[j] + kel);
        bhi[j] = *reinterpret_cast<const uint4 *>(xs.col[j] + kel + 32);
      }
    }
    const int grp = kblk * 8 + 2 * g4;
    const float2 xn0 = *reinterpret_cast<const float2 *>(XN + grp * ncols + xc);
    const float2 xn1 = *reinterpret_cast<const float2 *>(XN + (grp + 1) * ncols + xc);
    const float2 xx0 = *reinterpret_cast<const float2 *>(XX + grp * ncols + xc);
    const float2 xx1 = *reinterpret_cast<const float2 *>(XX + (grp + 1) * ncols + xc);
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      const int ra = 16 * mt + g, rbw = ra + 8;
      const uint2 qa = *reinterpret_cast<const uint2 *>(rb + ra * C::RS + QOFF + 32 * g4 + 8 * t);
      const uint2 qb = *reinterpret_cast<const uint2 *>(rb + rbw * C::RS + QOFF + 32 * g4 + 8 * t);
      uint32_t la0 = qa.x & M4, la1 = qa.y & M4, lb0 = qb.x & M4, lb1 = qb.y & M4;
      uint32_t ha0 = (qa.x >> 4) & M4, ha1 = (qa.y >> 4) & M4;
      uint32_t hb0 = (qb.x >> 4) & M4, hb1 = (qb.y >> 4) & M4;
      if constexpr (Q5) {
        // fifth bit: bit 2*g4 of qh for the low-nibble elements, bit 2*g4+1 for the high ones
        constexpr uint32_t M1 = 0x10101010u;
        auto bit = [&](uint32_t q, int b) { return b <= 4 ? ((q << (4 - b)) & M1) : ((q >> (b - 4)) & M1); };
        la0 |= bit(qh[mt][0].x, 2 * g4);     la1 |= bit(qh[mt][0].y, 2 * g4);
        lb0 |= bit(qh[mt][1].x, 2 * g4);     lb1 |= bit(qh[mt][1].y, 2 * g4);
        ha0 |= bit(qh[mt][0].x, 2 * g4 + 1); ha1 |= bit(qh[mt][0].y, 2 * g4 + 1);
        hb0 |= bit(qh[mt][1].x, 2 * g4 + 1); hb1 |= bit(qh[mt][1].y, 2 * g4 + 1);
      }
      const float2 sa0 = sc[(2 * g4) * R + ra], sb0 = sc[(2 * g4) * R + rbw];
      const float2 sa1 = sc[(2 * g4 + 1) * R + ra], sb1 = sc[(2 * g4 + 1) * R + rbw];
      float c0[4] = {xn0.x, xn0.y, xn0.x, xn0.y};
      float c1[4] = {xn1.x, xn1.y, xn1.x, xn1.y};
#pragma unroll
      for (int j = 0; j < NT; j++) {
        mma_bf16(c0, widen01(la0), widen01(lb0), widen23(la0), widen23(lb0), blo[j].x, blo[j].y);
        mma_bf16(c1, widen01(ha0), widen01(hb0), widen23(ha0), widen23(hb0), bhi[j].x, bhi[j].y);
        mma_bf16(c0, widen01(la1), widen01(lb1), widen23(la1), widen23(lb1), blo[j].z, blo[j].w);
        mma_bf16(c1, widen01(ha1), widen01(hb1), widen23(ha1), widen23(hb1), bhi[j].z, bhi[j].w);
      }
      acc[mt][0] = fmaf(sa0.x, c0[0], fmaf(sa0.y, xx0.x, acc[mt][0]));
      acc[mt][1] = fmaf(sa0.x, c0[1], fmaf(sa0.y, xx0.y, acc[mt][1]));
      acc[mt][2] = fmaf(sb0.x, c0[2], fmaf(sb0.y, xx0.x, acc[mt][2]));
      acc[mt][3] = fmaf(sb0.x, c0[3], fmaf(sb0.y, xx0.y, acc[mt][3]));
      acc[mt][0] = fmaf(sa1.x, c1[0], fmaf(sa1.y, xx1.x, acc[mt][0]));
      acc[mt][1] = fmaf(sa1.x, c1[1], fmaf(sa1.y, xx1.y, acc[mt][1]));
      acc[mt][2] = fmaf(sb1.x, c1[2], fmaf(sb1.y, xx1.x, acc[mt][2]));
      acc[mt][3] = fmaf(sb1.x, c1[3], fmaf(sb1.y, xx1.y, acc[mt][3]));
    }
  }
}

template <int MT, int NT>
__device__ __forceinline__ void process_q6(const uint8_t *stage, int wblk, int kblk,
                                           const float *sc, const float *XN, int ncols, int xc,
                                           const XCols<NT> &xs, const int (&pad)[MT][2], int lane,
                                           float (&acc)[MT][4]) {
  using C = Cfg<kQ6_K>;
  constexpr int R = 16 * MT;
  constexpr uint32_t M4 = 0x0f0f0f0fu, M2 = 0x30303030u;
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int nh = 0; nh < 4; nh++) {
    const int n = nh >> 1, h = nh & 1;
    uint2 bx[NT][4];
    float2 xn[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
      const int kel = kblk * 256 + 128 * n + 32 * k + 16 * h + 4 * t;
#pragma unroll
      for (int j = 0; j < NT; j++) {
        bx[j][k] = make_uint2(0, 0);
        if (xs.valid) bx[j][k] = *reinterpret_cast<const uint2 *>(xs.col[j] + kel);
      }
      xn[k] = *reinterpret_cast<const float2 *>(XN + (kblk * 16 + 8 * n + h + 2 * k) * ncols + xc);
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
      uint32_t q[2][4];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const uint8_t *rb = stage + (16 * mt + g + 8 * r) * C::RS + pad[mt][r] + wblk * C::BB;
        const uint32_t ql0 = lds32_unaligned(rb + 64 * n + 16 * h + 4 * t);
        const uint32_t ql1 = lds32_unaligned(rb + 64 * n + 32 + 16 * h + 4 * t);
        const uint32_t qhw = lds32_unaligned(rb + 128 + 32 * n + 16 * h + 4 * t);
        q[r][0] = (ql0 & M4) | ((qhw << 4) & M2);
        q[r][1] = (ql1 & M4) | ((qhw << 2) & M2);
        q[r][2] = ((ql0 >> 4) & M4) | (qhw & M2);
        q[r][3] = ((ql1 >> 4) & M4) | ((qhw >> 2) & M2);
      }
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const int j16 = 8 * n + h + 2 * k;
        float c[4] = {xn[k].x, xn[k].y, xn[k].x, xn[k].y};
#pragma unroll
        for (int j = 0; j < NT; j++)
          mma_bf16(c, widen01(q[0][k]), widen01(q[1][k]), widen23(q[0][k]), widen23(q[1][k]),
                   bx[j][k].x, bx[j][k].y);
        const float sa = sc[j16 * R + 16 * mt + g], sb = sc[j16 * R + 16 * mt + g + 8];
        acc[mt][0] = fmaf(sa, c[0], acc[mt][0]);
        acc[mt][1] = fmaf(sa, c[1], acc[mt][1]);
        acc[mt][2] = fmaf(sb, c[2], acc[mt][2]);
        acc[mt][3] = fmaf(sb, c[3], acc[mt][3]);
      }
    }
  }
}

// ---------------------------------------------------------------------------- the kernel
// PAIRED: batch <= 4, one n-tile whose columns are (hi_0, lo_0, hi_1, lo_1, ...).
// else  : batch <= 8, two n-tiles (all hi columns, all lo columns) into the same accumulator.
template <int TYPE, int MT, bool PAIRED>
__global__ void __launch_bounds__(kThreads, 1) gemv_mma_kernel(const Params p) {
  using C = Cfg<TYPE>;
  constexpr int NT = PAIRED ? 1 : 2;
  constexpr int R = 16 * MT;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);  // full[S], empty[S]
  const int S = p.stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; s++) {
      mbar_init(smem_u32(&bars[s]), 1);
      mbar_init(smem_u32(&bars[S + s]), kNW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  uint8_t *stages = smem + p.off_stage;

  if (warp == kNW) {
    // ------------------------------------------------------------------ producer warp
    int it = 0;
    for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x) {
      const int row = tile * R + lane;
      const bool rvalid = lane < R && row < p.out_dim;
      const uint8_t *rsrc = p.w + (long long)row * p.row_bytes;
      for (int c = 0; c < p.nchunks; c++, it++) {
        const int s = it % S;
        mbar_wait(smem_u32(&bars[S + s]), ((it / S) & 1) ^ 1);
        const int nb = min(kNW, p.nblk - c * kNW);
        const uint8_t *src = rsrc + (long long)c * kNW * C::BB;
        const uint32_t padb = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
        const uint32_t bytes = rvalid ? ((padb + nb * C::BB + 15u) & ~15u) : 0u;
        const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
        const uint32_t full = smem_u32(&bars[s]);
        if (lane == 0) mbar_arrive_expect_tx(full, total);
        __syncwarp();
        if (rvalid)
          bulk_g2s(smem_u32(stages + (size_t)s * p.stage_bytes + lane * C::RS), src - padb, bytes,
                   full);
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int ctid = threadIdx.x;  // 0 .. 255
  __nv_bfloat16 *xsm = reinterpret_cast<__nv_bfloat16 *>(smem + p.off_x);
  float *XN = reinterpret_cast<float *>(smem + p.off_xn);
  float *XX = reinterpret_cast<float *>(smem + p.off_xx);
  const int B = p.batch, K = p.in_dim, CS = p.cs, ncols = p.ncols;

  {  // split x into bf16 hi/lo planes and build the group-sum tables
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
          XN[grp * ncols + 2 * b] = -C::OFF * shi;
          XN[grp * ncols + 2 * b + 1] = -C::OFF * slo;
          if (C::HAS_MIN) {
            XX[grp * ncols + 2 * b] = shi;
            XX[grp * ncols + 2 * b + 1] = slo;
          }
        } else {
          XN[grp * ncols + b] = -C::OFF * (shi + slo);
          if (C::HAS_MIN) XX[grp * ncols + b] = shi + slo;
        }
      }
    }
  }
  consumer_sync();

  const int g = lane >> 2, t = lane & 3;
  XCols<NT> xs;
  if (PAIRED) {
    const int b = g >> 1, pl = g & 1;
    xs.valid = b < B;
    xs.col[0] = xsm + (size_t)((pl ? B : 0) + (xs.valid ? b : 0)) * CS;
  } else {
    xs.valid = g < B;
    xs.col[0] = xsm + (size_t)(xs.valid ? g : 0) * CS;
    if (NT > 1) xs.col[NT - 1] = xsm + (size_t)(B + (xs.valid ? g : 0)) * CS;
  }
  const int xc = min(2 * t, ncols - 2);
  uint8_t *scale_area = smem + p.off_scale + warp * (C::NGRP * R * C::SCB);
  float4 *red = reinterpret_cast<float4 *>(smem + p.off_red);

  long long best[2] = {LLONG_MIN, LLONG_MIN};  // fused top-1: this thread's running maxima

  int it = 0, tcount = 0;
  for (int tile = blockIdx.x; tile < p.ntiles; tile += gridDim.x, tcount++) {
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
    int pad[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int r = 0; r < 2; r++) {
        const long long row = (long long)tile * R + 16 * mt + g + 8 * r;
        pad[mt][r] = (int)((reinterpret_cast<uintptr_t>(p.w) + row * p.row_bytes) & 15);
      }
    const int dpad = (int)((reinterpret_cast<uintptr_t>(p.w) +
                            ((long long)tile * R + (lane < R ? lane : 0)) * p.row_bytes) & 15);

    for (int c = 0; c < p.nchunks; c++, it++) {
      const int s = it % S;
      mbar_wait(smem_u32(&bars[s]), (it / S) & 1);
      const int kblk = c * kNW + warp;
      if (kblk < p.nblk) {
        const uint8_t *stage = stages + (size_t)s * p.stage_bytes;
        decode_scales<TYPE, MT>(stage + (lane < R ? lane : 0) * C::RS + dpad + warp * C::BB, lane,
                                scale_area);
        __syncwarp();
        if constexpr (C::HAS_MIN)
          process_q45<TYPE, MT, NT>(stage, warp, kblk, reinterpret_cast<const float2 *>(scale_area),
                                    XN, XX, ncols, xc, xs, lane, acc);
        else
          process_q6<MT, NT>(stage, warp, kblk, reinterpret_cast<const float *>(scale_area), XN,
                             ncols, xc, xs, pad, lane, acc);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&bars[S + s]));
    }

    // fixed-order sum of the 8 warps' partial tiles
    float4 *rbuf = red + (size_t)(tcount & 1) * (kNW * MT * 32);
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
      rbuf[(warp * MT + mt) * 32 + lane] = make_float4(acc[mt][0], acc[mt][1], acc[mt][2], acc[mt][3]);
    consumer_sync();
    for (int u = ctid; u < MT * 64; u += kNW * 32) {
      const int hh = u & 1, ln = (u >> 1) & 31, mt = u >> 6;
      float v0 = 0.f, v1 = 0.f;
#pragma unroll
      for (int ww = 0; ww < kNW; ww++) {
        const float2 pr = reinterpret_cast<const float2 *>(&rbuf[(ww * MT + mt) * 32 + ln])[hh];
        v0 += pr.x;
        v1 += pr.y;
      }
      const int row = tile * R + 16 * mt + (ln >> 2) + 8 * hh;
      if (row >= p.out_dim) continue;
      const int c0 = 2 * (ln & 3);
      if (PAIRED) {
        const int b = ln & 3;
        if (b < B) {
          const float val = v0 + v1;
          if (p.part_keys) {
            const long long key = top1_key(val, (uint32_t)(p.index_base + row));
            best[0] = key > best[0] ? key : best[0];
          } else {
            const float a = p.addend ? p.addend[(long long)b * p.addend_stride + row] : 0.f;
            p.y[(long long)b * p.out_dim + row] = a + val;
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < 2; e++) {
          const int b = c0 + e;
          if (b >= B) continue;
          const float val = e ? v1 : v0;
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
  consumer_sync();  // everyone is done with the reduction buffers
  if (ctid < 16) s_best[ctid] = LLONG_MIN;
  consumer_sync();
  if (ctid < MT * 64) {
    const int ln = (ctid >> 1) & 31;
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
  int mt, stages;
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

template <int TYPE>
bool make_plan(int in_dim, int out_dim, int batch, bool paired, Plan &plan) {
  using C = Cfg<TYPE>;
  constexpr size_t kSmemMax = kDynSmemMax;
  const int nblk = in_dim / 256;
  const int ncols = paired ? (batch * 2 < 2 ? 2 : batch * 2) : 8;
  const int ngroups = in_dim / C::GROUP;
  const int cs = in_dim + C::XPAD;
  auto al = [](size_t v) { return (v + 127) & ~(size_t)127; };
  // prefer 32-row tiles when there are enough of them to fill the machine twice over
  for (int mt = (out_dim >= 32 * 2 * sm_count() ? 2 : 1); mt >= 1; mt--) {
    const int R = 16 * mt;
    size_t off = 128;
    const size_t off_red = off;       off = al(off + 2ull * kNW * mt * 32 * 16);
    const size_t off_scale = off;     off = al(off + (size_t)kNW * C::NGRP * R * C::SCB);
    const size_t off_xn = off;        off = al(off + (size_t)ngroups * ncols * 4);
    const size_t off_xx = off;        if (C::HAS_MIN) off = al(off + (size_t)ngroups * ncols * 4);
    const size_t off_x = off;         off = al(off + (size_t)2 * batch * cs * 2);
    const size_t off_stage = off;
    const size_t stage_bytes = al((size_t)R * C::RS);
    if (off_stage + 3 * stage_bytes > kSmemMax) continue;
    int stages = (int)((kSmemMax - off_stage) / stage_bytes);
    if (stages > 8) stages = 8;
    Params &p = plan.p;
    p.in_dim = in_dim; p.out_dim = out_dim; p.batch = batch;
    p.nblk = nblk; p.nchunks = (nblk + kNW - 1) / kNW; p.ntiles = (out_dim + R - 1) / R;
    p.stages = stages; p.row_bytes = (long long)nblk * C::BB; p.ncols = ncols; p.cs = cs;
    p.off_red = (int)off_red; p.off_scale = (int)off_scale; p.off_xn = (int)off_xn;
    p.off_xx = (int)off_xx; p.off_x = (int)off_x; p.off_stage = (int)off_stage;
    p.stage_bytes = (int)stage_bytes;
    plan.mt = mt; plan.stages = stages; plan.smem = off_stage + (size_t)stages * stage_bytes;
    return true;
  }
  return false;
}

template <int TYPE, int MT, bool PAIRED>
int launch_instance(const Plan &plan, int grid, cudaStream_t s) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_mma_kernel<TYPE, MT, PAIRED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kDynSmemMax);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  gemv_mma_kernel<TYPE, MT, PAIRED><<<grid, kThreads, plan.smem, s>>>(plan.p);
  return (int)cudaGetLastError();
}

template <int TYPE>
int run(Plan &plan, bool paired, cudaStream_t s) {
  const int sms = sm_count();
  const int grid = plan.p.ntiles < sms ? plan.p.ntiles : sms;
  if (plan.mt == 2) return paired ? launch_instance<TYPE, 2, true>(plan, grid, s)
                                  : launch_instance<TYPE, 2, false>(plan, grid, s);
  return paired ? launch_instance<TYPE, 1, true>(plan, grid, s)
                : launch_instance<TYPE, 1, false>(plan, grid, s);
}

template <int TYPE>
int gemv_typed(const void *d_w, const float *d_x, const float *d_addend, int64_t addend_stride,
               float *d_y, int in_dim, int out_dim, int batch, const Params *top1, cudaStream_t s) {
  // largest column group whose bf16 planes fit beside three stages
  for (int b0 = 0; b0 < batch;) {
    int nb = batch - b0 > 8 ? 8 : batch - b0;
    Plan plan{};
    bool paired = false, ok = false;
    for (; nb >= 1; nb--) {
      paired = nb <= 4;
      if (make_plan<TYPE>(in_dim, out_dim, nb, paired, plan)) { ok = true; break; }
    }
    if (!ok) return COGNI_QMM_ERR_LIMIT;
    Params &p = plan.p;
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
    int st = run<TYPE>(plan, paired, s);
    if (st) return st;
    b0 += nb;
  }
  return COGNI_QMM_OK;
}

}  // namespace

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
