// Chunked-prefill GEMM with dequantisation fused into the tile loop (sm_100a, tcgen05 + TMEM).
//
//     y[m, n] = sum_k bf16(x[m, k]) * bf16(dequant(W[n, k]))        fp32 accumulation in TMEM
//
// One CTA computes a 128 (weight rows n) x BN (tokens m) tile of y^T, BN = 128, 256 or 512; for
// Q4_K / Q5_K a 512-token tile is computed by a pair of CTAs over 256 weight rows (the 2-CTA
// kernel further down, tcgen05 cta_group::2):
//   * A operand = weights.  The raw GGUF superblocks of the tile's 128 rows reach shared memory by
//     TMA, one superblock column at a time (the weights as a byte matrix [rows, row bytes]; double
//     buffered), so the fetch is one instruction per column instead of one uncoalesced load per
//     row and word.  Dequant warps (sixteen for Q4_K / Q5_K: four threads per row, one per
//     16-element quarter of a k-step; eight otherwise: two threads per row) read their row's block
//     from there, rebuild the f32 weight (src/ml/gguf/dequant.cr), round it to bf16 and write a
//     128 x 64 K-major tile into shared memory in the 128-byte-swizzled canonical layout.  Q6_K
//     rows that are not multiples of 16 bytes (in_dim not a multiple of 2048) cannot be described
//     to TMA: their threads read global memory directly (four warps, one thread per row).
//   * B operand = activations.  One thread issues TMA tile loads (bf16 [<= 256 x 64] boxes,
//     128-byte swizzle) per k-step; every box has its own full and empty barrier.
//   * One thread issues tcgen05.mma (kind::f16, M = 128, N = min(BN, 256), K = 16) four times per
//     k-step and box (a 512-token tile: two accumulators of 256 columns fill the tensor memory);
//     tcgen05.commit releases the boxes and the weight tile.
//   * After the last k-step warps read the accumulator back with tcgen05.ld (each warp may read
//     the 32 TMEM lanes = 32 weight rows of its residue mod 4; the warps of a lane quarter share
//     the columns) and store y[m, n]: for a fixed token a warp's 32 lanes write 32 consecutive n,
//     one 128-byte segment.
// mbarrier rings decouple the three roles.  Every wait is bounded (tma_pipe.cuh).
#include <cuda.h>
#include <mutex>
#include <cuda_bf16.h>

#include "qmm_common.cuh"
#include "tma_pipe.cuh"

namespace cogni {
namespace {

constexpr int kBM = 128;      // weight rows per tile (UMMA M)
constexpr int kBK = 64;       // k elements per stage: 128 bytes of bf16 = one swizzle row
// stages of the ring: four 48 KB stages for 256-token tiles, two 80 KB stages for 512-token tiles
// Staged raw superblocks (rows that are multiples of 16 bytes): per superblock column the raw
// block of each of the tile's 128 rows is fetched by TMA from the weights seen as a byte matrix,
// double-buffered.  Q4_K / Q5_K: one box of 128 rows x 144 / 176 bytes, unswizzled (the row pitch
// already spreads 16-byte loads of eight rows over all banks).  Q6_K: the 256-byte window around
// the 210-byte block (it starts on a 2-byte boundary) as two boxes of 128 rows x 128 bytes with
// the 128-byte swizzle.
// bytes of 256 consecutive weights of a row (a K-quant superblock; eight Q8_0 blocks)
template <int TYPE> struct Sb { static constexpr int bytes = BlockGeom<TYPE>::bytes * (256 / BlockGeom<TYPE>::elems); };
constexpr int kRawBox = 128 * 128;
__host__ __device__ constexpr int raw_stage_bytes(int type) {
  return type == kQ6_K ? 2 * kRawBox : 128 * (type == kQ5_K ? 176 : 144);  // Q4_K, IQ4_NL: 144
}
__host__ __device__ constexpr int raw_bytes(int type, bool staged) { return staged ? 2 * raw_stage_bytes(type) : 0; }
// stages of the ring that fit beside the raw windows (227 KB per CTA)
__host__ __device__ constexpr int stages_for(int bn, int raw = 0) {
  const int want = bn > 256 ? 2 : 4;
  const int fit = (227 * 1024 - 1024 - 256 - raw) / (128 * 64 * 2 + bn * 64 * 2);
  return fit < want ? fit : want;
}
// Dequant warps: sixteen for Q4_K / Q5_K staged by TMA (four threads per tile row, one per
// 16-element quarter of a k-step: the expansion is a chain of dependent conversions, and two warps
// per scheduler could not hide its latencies; Q6_K measured slower that way on one CTA, 1144
// against 1216 TFLOP/s, and the same on a CTA pair); eight (two threads
// per tile row, one per 32-element half of a k-step); four (one thread per row, both halves) for
// Q6_K read directly from global memory, whose loads are the bound there.
__host__ __device__ constexpr int dequant_warps(int type, bool staged = false) {
  if (staged && (type == kQ4_K || type == kQ5_K)) return 16;
  return type == kQ6_K && !staged ? 4 : 8;
}
// Warp roles.  A warp scheduler serves the warps w with the same w % 4, and the thread that issues
// the MMAs must not queue behind dequant warps for an issue slot: the tensor pipe idles whenever it
// is late (measured on the 2-CTA kernel, Q4_K 12288 x 4096, 4096 tokens: 972 TFLOP/s with four
// dequant warps on its scheduler, 945 with two, 1131 with none).  With sixteen dequant warps,
// scheduler 1 therefore hosts only the MMA warp (1), the TMA warp (5) and four warps (9, 13, 17,
// 21) that sleep until the epilogue, where they read the TMEM lane quarter 1 that only warps of
// their residue can; the dequant warps are the other warps up to 20.  With eight or four dequant
// warps: warp 0 TMA, warp 1 MMA, the rest dequant.
// Tiles narrower than 512 tokens are bound by the expansion, not by the MMAs: there the sixteen
// dequant warps use all four schedulers (measured tile times at in_dim 4096, Q4_K, 128 / 256
// tokens: 44.1 / 48.4 us with the isolated layout against 39.1 / 44.5 us without).
constexpr int kIsoWarps = 22;
__host__ __device__ constexpr bool isolate_mma_warp(int type, bool staged, int bn) {
  return dequant_warps(type, staged) == 16 && bn == 512;
}
__host__ __device__ constexpr int threads_for(int type, bool staged = false, int bn = 512) {
  return isolate_mma_warp(type, staged, bn) ? 32 * kIsoWarps : 64 + 32 * dequant_warps(type, staged);
}
template <bool ISO> struct Roles {
  static constexpr int tma_warp = ISO ? 5 : 0;
  __device__ static bool is_dequant(int warp) { return ISO ? (warp & 3) != 1 && warp <= 20 : warp >= 2; }
  // dense index over the dequant warps
  __device__ static int dequant_index(int warp) { return ISO ? warp - ((warp + 2) >> 2) : warp - 2; }
  // the epilogue: four warps (ISO; else all dequant warps) per TMEM lane quarter warp % 4, each
  // taking an equal chunk of the token columns
  __device__ static bool in_epilogue(int warp) {
    return ISO ? ((warp & 3) == 1 ? warp >= 9 : warp < 16) : warp >= 2;
  }
  __device__ static int epilogue_chunk(int warp) {
    return ISO ? ((warp & 3) == 1 ? (warp >> 2) - 2 : warp >> 2) : (warp - 2) >> 2;
  }
};
constexpr int kATile = kBM * kBK * 2;  // 16 KB

struct GemmParams {
  const uint8_t *w;
  void *y;
  int m_rows, n_out, k_in, out_bf16;
  int ks_per_split;  // k-steps per blockIdx.z; with two splits the partial tiles are added onto a zeroed y
  int splits;
  unsigned *turns;   // four splits: [tile][4] turn counters that order the partial tiles' additions (else nullptr)
  long long row_bytes;
};

// ---------------------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The four K = 16 MMAs of a 64-element k-step as one block of instructions.  The thread that
// issues the MMAs shares its warp scheduler with other warps and the tensor pipe idles whenever
// it is late, so its instruction count per k-step matters: descriptors are formed here from their
// 32-bit halves (a step of 16 bf16 along K is 32 bytes = 2 in the descriptor's address field),
// one predicate decides whether the first MMA accumulates, the others always do.
// a_lo / b_lo: low descriptor words of the operand tiles (smem_desc_lo), desc_hi: kDescHi.
constexpr uint32_t kDescHi = 64u | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t smem_addr) {
  return ((smem_addr & 0x3FFFF) >> 4) | (1u << 16);
}
#define COGNI_UMMA4(GROUP)                                                                      \
  asm volatile(                                                                                  \
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"                      \
      "setp.ne.b32 p0, %5, 0;\n\t"                                                               \
      "setp.eq.b32 p1, %4, %4;\n\t"                                                              \
      "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"                                       \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], da, db, %4, p0;\n\t"                      \
      "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t" \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], da, db, %4, p1;\n\t"                      \
      "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t" \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], da, db, %4, p1;\n\t"                      \
      "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t" \
      "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%0], da, db, %4, p1;\n\t}"                     \
      ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate_first)         \
      : "memory")
__device__ __forceinline__ void umma4_bf16(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate_first) {
  COGNI_UMMA4("1");
}
__device__ __forceinline__ void umma4_bf16_pair(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo,
                                                uint32_t idesc, uint32_t accumulate_first) {
  COGNI_UMMA4("2");
}
#undef COGNI_UMMA4
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,"
      "%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 2-D TMA tile load (no multicast), completion in bytes on an mbarrier.  c0 (the innermost
// coordinate) times the element size must be a multiple of 16 bytes: here c0 = 64 * k-step.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *tmap, int c0, int c1,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], "
      "[%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Shared-memory matrix descriptor: K-major tile, rows of 128 bytes, SWIZZLE_128B, 8-row groups
// 1024 bytes apart (start >> 4 | LBO 1 | SBO 64 | version 1 | layout type 2).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: D = f32, A = B = bf16, both K-major, M x N.
__host__ __device__ constexpr uint32_t idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
// byte i of v as an exact float
__device__ __forceinline__ float byte_f(uint32_t v, int i) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i)) - 8388608.f;
}
// byte i of v minus 32 as an exact float: (2^23 + b) - (2^23 + 32)
__device__ __forceinline__ float byte_f_m32(uint32_t v, int i) {
  return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i)) - 8388640.f;
}
// Packed pairs of f32 (sm_100 has two-wide f32 add / mul / fma: same IEEE results per element, half
// the instructions in the expansion, which is what the dequant warps are bound by).
__device__ __forceinline__ uint64_t f2_pack(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint32_t f2_to_bf16x2(uint64_t v) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
  return pack_bf16(a, b);
}
// bytes (i, i+1) of v as the floats 2^23 + b, packed
__device__ __forceinline__ uint64_t bytes2_biased(uint32_t v, int i) {
  return f2_pack(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i)),
                 __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i + 1)));
}
// Stores chunk c (8 consecutive k elements = 16 bytes) of tile row r at its swizzled position.
__device__ __forceinline__ void store_chunk(uint8_t *tile, int r, int c, uint4 v) {
  *reinterpret_cast<uint4 *>(tile + r * 128 + ((c ^ (r & 7)) << 4)) = v;
}

// ---------------------------------------------------------------------------- raw block fetch
// N 32-bit words starting at a 2-byte aligned global address (aligned loads + funnel shift).
template <int N>
__device__ __forceinline__ void ldg_words_unaligned(const uint8_t *p, uint32_t (&out)[N]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint32_t *q = reinterpret_cast<const uint32_t *>(a & ~(uintptr_t)3);
  const uint32_t sh = (uint32_t)(a & 2) * 8;
  uint32_t prev = __ldg(q);
#pragma unroll
  for (int i = 0; i < N; i++) {
    const uint32_t next = __ldg(q + i + 1);
    out[i] = __funnelshift_r(prev, next, sh);
    prev = next;
  }
}
// Eight 32-bit words (32 bytes) starting at a 2-byte aligned global address, fetched as three
// 16-byte vectors from the 16-byte boundary below it: the rows of a tile are kilobytes apart, so
// every lane's load is its own L1 wavefront whatever its width, and 4-byte loads would cost four
// times as many.  Reads at most 15 bytes beyond the 32 (still inside the 210-byte block for the
// ql and qh fields this is used on).
__device__ __forceinline__ void ldg_8words_wide(const uint8_t *p, uint32_t (&out)[8]) {
  const uintptr_t a = reinterpret_cast<uintptr_t>(p);
  const uint4 *q = reinterpret_cast<const uint4 *>(a & ~(uintptr_t)15);
  const uint4 v0 = __ldg(q), v1 = __ldg(q + 1), v2 = __ldg(q + 2);
  const uint32_t w[12] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w};
  const uint32_t sh = (uint32_t)(a & 2) * 8;
  switch ((a & 15) >> 2) {  // word offset inside the first vector; the same for all rows of a tile
    case 0:                 // whenever the row size is a multiple of 16 bytes
#pragma unroll
      for (int i = 0; i < 8; i++) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
      break;
    case 1:
#pragma unroll
      for (int i = 0; i < 8; i++) out[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < 8; i++) out[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
      break;
    default:
#pragma unroll
      for (int i = 0; i < 8; i++) out[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
      break;
  }
}

// Row r of a staged raw window: 16-byte chunk w (0 .. 15) of the 256-byte window.
__device__ __forceinline__ uint4 raw_chunk(const uint8_t *win, int r, int w) {
  return *reinterpret_cast<const uint4 *>(win + (w >> 3) * kRawBox + r * 128 + (((w & 7) ^ (r & 7)) << 4));
}
// N (<= 8) 32-bit words starting at the even byte offset `off` of row r's window (off is the same
// for every row of the tile): aligned 16-byte chunks + funnel shifts.
template <int N>
__device__ __forceinline__ void lds_words(const uint8_t *win, int r, int off, uint32_t (&out)[N]) {
  constexpr int NC = (4 * N + 14) / 16 + 1;  // chunks that can be touched
  uint32_t w[4 * NC + 1];
  const int c0 = off >> 4;
#pragma unroll
  for (int i = 0; i < NC; i++) {
    // the last chunk is only needed when the words run into it; the window has 16 chunks
    const uint4 v = raw_chunk(win, r, min(c0 + i, 15));
    w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
  }
  w[4 * NC] = 0;
  const uint32_t sh = (uint32_t)(off & 2) * 8;
  switch ((off & 15) >> 2) {
    case 0:
#pragma unroll
      for (int i = 0; i < N; i++) out[i] = __funnelshift_r(w[i], w[i + 1], sh);
      break;
    case 1:
#pragma unroll
      for (int i = 0; i < N; i++) out[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
      break;
    case 2:
#pragma unroll
      for (int i = 0; i < N; i++) out[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
      break;
    default:
#pragma unroll
      for (int i = 0; i < N; i++) out[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
      break;
  }
}

// The raw bytes one thread needs to rebuild 64 consecutive weights (one k-step) of its row.
template <int TYPE> struct Raw;
template <> struct Raw<kQ4_K> { uint4 hdr, q0, q1; };
template <> struct Raw<kQ5_K> { uint4 hdr, h0, h1, q0, q1; };
template <> struct Raw<kQ6_K> { uint32_t ql[8], qh[8], sc; uint32_t d; uint32_t scw[4]; };  // scw: the superblock's 16 scales (staged path)
template <> struct Raw<kQ8_0> { uint32_t q[8]; uint32_t d; };  // one 34-byte block: half a k-step
template <> struct Raw<kIQ4_NL> { uint32_t q[4]; uint32_t d; };  // one 18-byte block: half a k-step

// `h`: which 32-element half of the k-step this thread expands (Q6_K fetches only that half's ql).
// SHARED_TOO = false skips what both halves of a Q6_K k-step share (qh, d): a thread that expands
// both halves copies them from its first half.
template <int TYPE, bool SHARED_TOO = true>
__device__ __forceinline__ void fetch_raw(const uint8_t *row, int ks, int h, Raw<TYPE> &r) {
  const uint8_t *blk = row + (size_t)(ks >> 2) * Sb<TYPE>::bytes;
  const int j = ks & 3;
  if constexpr (TYPE == kQ4_K) {
    r.hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
    r.q0 = __ldg(reinterpret_cast<const uint4 *>(blk + 16 + 32 * j));
    r.q1 = __ldg(reinterpret_cast<const uint4 *>(blk + 32 + 32 * j));
  } else if constexpr (TYPE == kQ5_K) {
    r.hdr = __ldg(reinterpret_cast<const uint4 *>(blk));
    r.h0 = __ldg(reinterpret_cast<const uint4 *>(blk + 16));
    r.h1 = __ldg(reinterpret_cast<const uint4 *>(blk + 32));
    r.q0 = __ldg(reinterpret_cast<const uint4 *>(blk + 48 + 32 * j));
    r.q1 = __ldg(reinterpret_cast<const uint4 *>(blk + 64 + 32 * j));
  } else if constexpr (TYPE == kIQ4_NL) {
    // block 2j + h of the eight: fp16 d, then 16 bytes of nibble pairs, at an even address; two
    // 16-byte vectors from the boundary below cover its 18 bytes
    const uintptr_t a = reinterpret_cast<uintptr_t>(blk + 36 * j + 18 * h);
    const uint4 *q = reinterpret_cast<const uint4 *>(a & ~(uintptr_t)15);
    const uint4 v0 = __ldg(q), v1 = __ldg(q + 1);
    const uint32_t w[9] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, 0u};
    const uint32_t o = (uint32_t)(a & 15);
    const uint32_t sh = ((o + 2) & 2) * 8;
    uint32_t dw = 0;
    switch (o >> 2) {
      case 0: dw = w[0]; break;
      case 1: dw = w[1]; break;
      case 2: dw = w[2]; break;
      default: dw = w[3]; break;
    }
    r.d = (dw >> ((o & 2) * 8)) & 0xffffu;
    switch ((o + 2) >> 2) {
      case 0:
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i], w[i + 1], sh);
        break;
      case 1:
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
        break;
      case 2:
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
        break;
      case 3:
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
        break;
      default:
#pragma unroll
        for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i + 4], w[i + 5], sh);
        break;
    }
  } else if constexpr (TYPE == kQ8_0) {
    // block 2j + h of the eight: fp16 d, then 32 int8, at an even address.  Three 16-byte vectors
    // from the boundary below cover its 34 bytes; the offset is the same for all rows of a tile.
    const uintptr_t a = reinterpret_cast<uintptr_t>(blk + 68 * j + 34 * h);
    const uint4 *q = reinterpret_cast<const uint4 *>(a & ~(uintptr_t)15);
    const uint4 v0 = __ldg(q), v1 = __ldg(q + 1), v2 = __ldg(q + 2);
    const uint32_t w[13] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w, 0u};
    const uint32_t o = (uint32_t)(a & 15);
    const uint32_t sh = ((o + 2) & 2) * 8;
    uint32_t dw = 0;
    switch (o >> 2) {
      case 0: dw = w[0]; break;
      case 1: dw = w[1]; break;
      case 2: dw = w[2]; break;
      default: dw = w[3]; break;
    }
    r.d = (dw >> ((o & 2) * 8)) & 0xffffu;
    switch ((o + 2) >> 2) {
      case 0:
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = __funnelshift_r(w[i], w[i + 1], sh);
        break;
      case 1:
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = __funnelshift_r(w[i + 1], w[i + 2], sh);
        break;
      case 2:
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = __funnelshift_r(w[i + 2], w[i + 3], sh);
        break;
      case 3:
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = __funnelshift_r(w[i + 3], w[i + 4], sh);
        break;
      default:
#pragma unroll
        for (int i = 0; i < 8; i++) r.q[i] = __funnelshift_r(w[i + 4], w[i + 5], sh);
        break;
    }
  } else {
    const int n = j >> 1;
    ldg_8words_wide(blk + 64 * n + 32 * h, r.ql);
    if constexpr (SHARED_TOO) {
      ldg_8words_wide(blk + 128 + 32 * n, r.qh);
      uint32_t scw[1];
      ldg_words_unaligned<1>(blk + 192 + 8 * n + 4 * (j & 1), scw);
      r.sc = scw[0];
      r.d = __ldg(reinterpret_cast<const unsigned short *>(blk + 208));
    }
  }
}

// 6-bit (scale, min) pair s of a Q4_K / Q5_K header held in registers (dequant.cr:240-249)
__device__ __forceinline__ void scale_min_regs(const uint4 &h, int s, float &sc, float &mn) {
  const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
  uint32_t a, b;
  if (s < 4) {
    a = (u0 >> (8 * s)) & 63;
    b = (u1 >> (8 * s)) & 63;
  } else {
    const int t = 8 * (s - 4);
    a = ((u2 >> t) & 0xF) | (((u0 >> (t + 6)) & 3) << 4);
    b = ((u2 >> (t + 4)) & 0xF) | (((u1 >> (t + 6)) & 3) << 4);
  }
  sc = (float)a;
  mn = (float)b;
}

// Q4_K / Q5_K, staged: the words of k-step j of the block at blk (shared memory, 16-byte aligned)
// Q4_K / Q5_K, staged, one thread per quarter: the header and the 16 bytes (q0, h0) that hold the
// quarter's nibbles and fifth bits.
template <int TYPE>
__device__ __forceinline__ void fetch_quarter_from(const uint8_t *blk, int j, int q2, Raw<TYPE> &r) {
  static_assert(TYPE == kQ4_K || TYPE == kQ5_K, "K-quants with 32-element groups");
  r.hdr = *reinterpret_cast<const uint4 *>(blk);
  if constexpr (TYPE == kQ4_K) {
    r.q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * j + 16 * q2);
  } else {
    r.h0 = *reinterpret_cast<const uint4 *>(blk + 16 + 16 * q2);
    r.q0 = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * j + 16 * q2);
  }
}

template <int TYPE>
__device__ __forceinline__ void fetch_raw_from(const uint8_t *blk, int j, int h, Raw<TYPE> &r) {
  if constexpr (TYPE == kIQ4_NL) {
    // block 2j + h: d at 36j + 18h, the quants 2 bytes on (a word boundary only for odd blocks)
    const uint8_t *b = blk + 36 * j + 18 * h;
    r.d = *reinterpret_cast<const unsigned short *>(b);
    const uint32_t *q = reinterpret_cast<const uint32_t *>(b + 2 - 2 * (1 - h));  // word at or below the quants
    const uint32_t sh = (uint32_t)(1 - h) * 16;
    uint32_t w[5];
#pragma unroll
    for (int i = 0; i < 5; i++) w[i] = q[i < 4 || h == 0 ? i : 3];
#pragma unroll
    for (int i = 0; i < 4; i++) r.q[i] = __funnelshift_r(w[i], w[i + 1], sh);
  } else if constexpr (TYPE == kQ4_K) {
    r.hdr = *reinterpret_cast<const uint4 *>(blk);
    r.q0 = *reinterpret_cast<const uint4 *>(blk + 16 + 32 * j);
    r.q1 = *reinterpret_cast<const uint4 *>(blk + 32 + 32 * j);
  } else if constexpr (TYPE == kQ5_K) {
    r.hdr = *reinterpret_cast<const uint4 *>(blk);
    r.h0 = *reinterpret_cast<const uint4 *>(blk + 16);
    r.h1 = *reinterpret_cast<const uint4 *>(blk + 32);
    r.q0 = *reinterpret_cast<const uint4 *>(blk + 48 + 32 * j);
    r.q1 = *reinterpret_cast<const uint4 *>(blk + 64 + 32 * j);
  }
}

// Start of the 256-byte window that holds Q6_K superblock sb of a row: the 16-byte boundary below
// the block, moved down where the window would otherwise reach beyond the row (boxes that reach
// outside the matrix are avoided altogether: with boxes whose last rows lay beyond the matrix,
// about one launch in twenty read stale bytes in the rows that were inside).
__device__ __forceinline__ int q6_window_start(int sb, int row_bytes) {
  return min((210 * sb) & ~15, row_bytes - 256);
}

// Q6_K, staged: both halves of k-step j (= ks & 3) of row r from the superblock's window in
// shared memory; pad = offset of the 210-byte block inside the window.
template <int NH>
__device__ __forceinline__ void fetch_staged_q6(const uint8_t *win, int r, int pad, int j, int h0,
                                                Raw<kQ6_K> (&dst)[NH]) {
  const int n = j >> 1;
  // The two k-steps of a half n of the superblock (j = 2n, 2n + 1) use the same ql bytes (low /
  // high nibbles) and the same qh bytes (bit pairs 2 kk): they are fetched at the even k-step and
  // stay in `dst` for the odd one (a CTA's first k-step is a multiple of four).
  if ((j & 1) == 0) {
    lds_words<8>(win, r, pad + 64 * n + 32 * h0, dst[0].ql);
    if constexpr (NH == 2) lds_words<8>(win, r, pad + 64 * n + 32, dst[1].ql);
    lds_words<8>(win, r, pad + 128 + 32 * n, dst[0].qh);
    const int doff = pad + 208;
    dst[0].d = *reinterpret_cast<const unsigned short *>(
        win + (doff >> 7) * kRawBox + r * 128 + ((((doff >> 4) & 7) ^ (r & 7)) << 4) + (doff & 15));
    if constexpr (NH == 2) {
#pragma unroll
      for (int w = 0; w < 8; w++) dst[1].qh[w] = dst[0].qh[w];
      dst[1].d = dst[0].d;
    }
  }
  // the 16 scales of the superblock: fetched with its first k-step; k-step j uses word j
  if (j == 0) lds_words<4>(win, r, pad + 192, dst[0].scw);
  dst[0].sc = j == 0 ? dst[0].scw[0] : j == 1 ? dst[0].scw[1] : j == 2 ? dst[0].scw[2] : dst[0].scw[3];
  if constexpr (NH == 2) dst[1].sc = dst[0].sc;
}

// Rebuilds half h (32 weights: chunks 4h .. 4h+3) of k-step ks of tile row r as bf16 and stores
// them swizzled.  QUARTER: only quarter q2 of the half (chunks 4h + 2 q2, + 1), whose raw words
// are the first ones of `raw` (fetch_quarter_from).
template <int TYPE, bool QUARTER = false>
__device__ __forceinline__ void expand_kstep(const Raw<TYPE> &raw, int ks, int h, uint8_t *tile,
                                             int r, bool valid, int q2 = 0) {
  constexpr int NC = QUARTER ? 2 : 4;  // chunks of 8 weights this thread writes
  const int cbase = 4 * h + (QUARTER ? 2 * q2 : 0);
  if (!valid) {
#pragma unroll
    for (int c4 = 0; c4 < NC; c4++) store_chunk(tile, r, cbase + c4, make_uint4(0, 0, 0, 0));
    return;
  }
  const int j = ks & 3;
  if constexpr (TYPE == kIQ4_NL) {
    // w = d * table[q] (dequant.cr IQ4_NL): element i is the low nibble of byte i, element 16 + i
    // the high one.  Three byte permutes look four nibbles up (the table's halves by the low three
    // bits, then a choice by the fourth); two more sort the results into element order.
    const float d = __half2float(__ushort_as_half((unsigned short)raw.d));
    const uint64_t d_2 = f2_pack(d, d), unbias2 = f2_pack(-8388736.f, -8388736.f);
    auto lut4 = [](uint32_t hq) {
      const uint32_t s7 = hq & 0x7777u;
      const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, s7);
      const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, s7);
      return __byte_perm(lo, hi, 0x3210u | ((hq >> 1) & 0x4444u));
    };
    uint32_t lows[4], highs[4];  // elements 4i .. 4i+3 and 16+4i .. 16+4i+3 as int8
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const uint32_t a = lut4(raw.q[i]), b = lut4(raw.q[i] >> 16);
      lows[i] = __byte_perm(a, b, 0x6420);
      highs[i] = __byte_perm(a, b, 0x7531);
    }
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
      uint32_t out[4];
#pragma unroll
      for (int w2 = 0; w2 < 2; w2++) {
        const uint32_t q = (c4 < 2 ? lows[2 * c4 + w2] : highs[2 * (c4 - 2) + w2]) ^ 0x80808080u;
        out[2 * w2] = f2_to_bf16x2(f2_mul(d_2, f2_add(bytes2_biased(q, 0), unbias2)));
        out[2 * w2 + 1] = f2_to_bf16x2(f2_mul(d_2, f2_add(bytes2_biased(q, 2), unbias2)));
      }
      store_chunk(tile, r, 4 * h + c4, make_uint4(out[0], out[1], out[2], out[3]));
    }
  } else if constexpr (TYPE == kQ8_0) {
    // w = d * q (dequant.cr Q8_0): int8 b as the float 2^23 + (b ^ 0x80), minus 2^23 + 128
    const float d = __half2float(__ushort_as_half((unsigned short)raw.d));
    const uint64_t d_2 = f2_pack(d, d), unbias2 = f2_pack(-8388736.f, -8388736.f);
#pragma unroll
    for (int c4 = 0; c4 < 4; c4++) {
      uint32_t out[4];
#pragma unroll
      for (int w2 = 0; w2 < 2; w2++) {
        const uint32_t q = raw.q[2 * c4 + w2] ^ 0x80808080u;
        out[2 * w2] = f2_to_bf16x2(f2_mul(d_2, f2_add(bytes2_biased(q, 0), unbias2)));
        out[2 * w2 + 1] = f2_to_bf16x2(f2_mul(d_2, f2_add(bytes2_biased(q, 2), unbias2)));
      }
      store_chunk(tile, r, 4 * h + c4, make_uint4(out[0], out[1], out[2], out[3]));
    }
  } else if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
    // low nibbles (h = 0): sub-block 2j, high nibbles (h = 1): sub-block 2j+1
    const __half2 dd = *reinterpret_cast<const __half2 *>(&raw.hdr.x);
    const float d = __low2float(dd), dmin = __high2float(dd);
    const uint32_t qw[8] = {raw.q0.x, raw.q0.y, raw.q0.z, raw.q0.w,
                            raw.q1.x, raw.q1.y, raw.q1.z, raw.q1.w};
    uint32_t hw[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if constexpr (TYPE == kQ5_K) {
      hw[0] = raw.h0.x; hw[1] = raw.h0.y; hw[2] = raw.h0.z; hw[3] = raw.h0.w;
      hw[4] = raw.h1.x; hw[5] = raw.h1.y; hw[6] = raw.h1.z; hw[7] = raw.h1.w;
    }
    float sc, mn;
    scale_min_regs(raw.hdr, 2 * j + h, sc, mn);
    const float d1 = __fmul_rn(d, sc), m1 = __fmul_rn(dmin, mn);
    const uint64_t d1_2 = f2_pack(d1, d1), nm1_2 = f2_pack(-m1, -m1);
    const uint64_t unbias2 = f2_pack(-8388608.f, -8388608.f);
#pragma unroll
    for (int c4 = 0; c4 < NC; c4++) {          // 8 elements: bytes 8*c4 .. 8*c4+7 (of the quarter)
      uint32_t out[4];
#pragma unroll
      for (int w2 = 0; w2 < 2; w2++) {
        uint32_t q = (qw[2 * c4 + w2] >> (4 * h)) & 0x0f0f0f0fu;
        if constexpr (TYPE == kQ5_K)
          q |= ((hw[2 * c4 + w2] >> (2 * j + h)) & 0x01010101u) << 4;
        // d1 * q - m1, fused, on pairs: (2^23 + b) - 2^23 is exact
        out[2 * w2] = f2_to_bf16x2(f2_fma(d1_2, f2_add(bytes2_biased(q, 0), unbias2), nm1_2));
        out[2 * w2 + 1] = f2_to_bf16x2(f2_fma(d1_2, f2_add(bytes2_biased(q, 2), unbias2), nm1_2));
      }
      store_chunk(tile, r, cbase + c4, make_uint4(out[0], out[1], out[2], out[3]));
    }
  } else {
    // the k-step is elements 64*hi .. 64*hi+63 of the superblock's half n = j >> 1: two runs of 32,
    // kk = 2*hi + h is this thread's; its quants are nibble hi of ql bytes 32*h .. 32*h+31 of the
    // half and bits 2*kk, 2*kk+1 of the half's 32 qh bytes; scales l/16 + 2*kk of the half
    const float d = __half2float(__ushort_as_half((unsigned short)raw.d));
    const int hi = j & 1, kk = 2 * hi + h;
#pragma unroll
    for (int c4 = 0; c4 < NC; c4++) {
      const int scb = (int)(int8_t)((raw.sc >> (8 * ((QUARTER ? q2 : (c4 >> 1)) + 2 * h))) & 0xff);
      const float dsc = __fmul_rn(d, (float)scb);
      const uint64_t dsc_2 = f2_pack(dsc, dsc), unbias2 = f2_pack(-8388640.f, -8388640.f);
      uint32_t out[4];
#pragma unroll
      for (int w2 = 0; w2 < 2; w2++) {
        const uint32_t qlw = raw.ql[2 * c4 + w2];
        const uint32_t qhw = raw.qh[2 * c4 + w2];
        const uint32_t q = ((qlw >> (4 * hi)) & 0x0f0f0f0fu) | (((qhw >> (2 * kk)) & 0x03030303u) << 4);
        // dsc * (q - 32) on pairs: (2^23 + b) - (2^23 + 32) is exact
        out[2 * w2] = f2_to_bf16x2(f2_mul(dsc_2, f2_add(bytes2_biased(q, 0), unbias2)));
        out[2 * w2 + 1] = f2_to_bf16x2(f2_mul(dsc_2, f2_add(bytes2_biased(q, 2), unbias2)));
      }
      store_chunk(tile, r, cbase + c4, make_uint4(out[0], out[1], out[2], out[3]));
    }
  }
}

// Ordered split along K.  Four CTAs of a tile take a quarter of K each and add their partial tiles
// into y (the first part of every group is stored, so y is not zeroed).  Float addition does not commute over four addends, so the order is fixed: the
// tile's columns form four groups, split z adds its part of group (z + t) mod 4 at step t, and a
// turn counter per (tile, group) admits the steps in order; in every step the four splits work on
// different groups.  The order depends on the group only, so every launch gives the same bits.
// The four CTAs of a tile must run at the same time: the host uses this only for grids of at most
// one CTA per SM.  The wait is bounded like every wait.
__device__ unsigned g_prefill_turns[8][64 * 4];  // [stream slot][tile][group], zero between launches

__device__ __forceinline__ void wait_turn(const unsigned *turn, unsigned want) {
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 0;; spin++) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(turn) : "memory");
    if (v == want) return;
    __nanosleep(64);
    if ((spin & 63u) == 63u) {
      if (pipe_broken()) return;
      if (global_ns() - t0 > kPipeWaitLimitNs) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        return;
      }
    }
  }
}

// ---------------------------------------------------------------------------- the kernel
template <int TYPE, int BN, bool STAGED>
__global__ void __launch_bounds__(threads_for(TYPE, STAGED, BN), 1)
    gemm_prefill_kernel(const __grid_constant__ CUtensorMap tmap_x,
                        const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
  constexpr int kRawStage = raw_stage_bytes(TYPE);
  constexpr int kStages = stages_for(BN, raw_bytes(TYPE, STAGED));
  static_assert(kStages >= 2, "at least two stages");
  constexpr int kDequantWarps = dequant_warps(TYPE, STAGED);
  constexpr int kHalves = kDequantWarps >= 8 ? 1 : 2;   // halves of a k-step per thread
  constexpr bool kQuarter = kDequantWarps == 16;        // a thread expands one quarter of a k-step
  constexpr int kBTile = BN * kBK * 2;
  constexpr int kStageBytes = kATile + kBTile;
  // UMMA N is at most 256: a 512-token tile is two accumulators of 256 TMEM columns, fed by the
  // two 256-row halves of the stage's B tile
  constexpr int kNMma = BN > 256 ? 256 : BN, kNSub = BN / kNMma;
  extern __shared__ uint8_t smem_raw[];
  // stage tiles must sit on 1024-byte boundaries (the swizzle pattern repeats every 1024 bytes)
  uint8_t *smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint8_t *raw_win = smem + kStages * kStageBytes;  // STAGED: two raw stages of two boxes each
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_win + raw_bytes(TYPE, STAGED));
  // bars: full_a[S] | full_b[S][kNSub] | empty_a[S] | empty_b[S][kNSub] | acc_full | raw_full[2] |
  // raw_empty[2]; then the TMEM base address slot.  The B tile of a stage is kNSub boxes of 256
  // tokens, each with its own full / empty barrier: a box is reloaded as soon as the MMAs that read
  // it are done, half a k-step before the stage's other box, which is what lets a 32 KB load hide
  // behind the MMAs with only two stages.
  constexpr int kFullB = kStages, kEmptyA = kFullB + kStages * kNSub, kEmptyB = kEmptyA + kStages;
  constexpr int kAccBar = kEmptyB + kStages * kNSub;
  static_assert((kAccBar + 5) * 8 + 4 <= 256, "barriers fit their 256 bytes");
  uint64_t *raw_bars = bars + kAccBar + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raw_bars + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * kBM, m0 = blockIdx.y * BN;
  // STAGED: the raw boxes of the last row tile start early enough to lie inside the matrix (the
  // host stages only matrices of at least 128 rows); the tile's rows are then further down the box
  const int raw_n0 = STAGED ? min(n0, p.n_out - kBM) : n0;
  // this CTA's k-steps: ks0 .. ks0 + nks - 1 (all of them unless the launch is split along K)
  const int ks0 = blockIdx.z * p.ks_per_split;
  const int nks = min(p.ks_per_split, p.k_in / kBK - ks0);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; s++) {
      mbar_init(smem_u32(&bars[s]), kDequantWarps);        // full_a: one arrive per dequant warp
      mbar_init(smem_u32(&bars[kEmptyA + s]), 1);          // empty_a: tcgen05.commit
      for (int h = 0; h < kNSub; h++) {
        mbar_init(smem_u32(&bars[kFullB + s * kNSub + h]), 1);   // full_b: the TMA thread + bytes
        mbar_init(smem_u32(&bars[kEmptyB + s * kNSub + h]), 1);  // empty_b: tcgen05.commit
      }
    }
    mbar_init(smem_u32(&bars[kAccBar]), 1);                // accumulator complete
    if constexpr (STAGED) {
      mbar_init(smem_u32(&raw_bars[0]), 1);                // raw_full: the issuing thread + bytes
      mbar_init(smem_u32(&raw_bars[1]), 1);
      mbar_init(smem_u32(&raw_bars[2]), kDequantWarps);    // raw_empty: one arrive per dequant warp
      mbar_init(smem_u32(&raw_bars[3]), kDequantWarps);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  using R = Roles<isolate_mma_warp(TYPE, STAGED, BN)>;
  if (warp == R::tma_warp) {
    // ---------------------------------------------------------------- activations via TMA
    if (lane == 0) {
      // STAGED: the same thread keeps the next superblock column's raw windows in flight.
      // Superblock sb of a row starts Sb bytes * sb into it (rows are multiples of 16 bytes here);
      // the Q6_K window: see q6_window_start.
      const int sb0 = ks0 >> 2, nsb = (nks + 3) >> 2;
      auto issue_raw = [&](int sbl) {
        const uint32_t full = smem_u32(&raw_bars[sbl & 1]);
        mbar_arrive_expect_tx(full, kRawStage);
        if constexpr (TYPE == kQ6_K) {
          const int x0 = q6_window_start(sb0 + sbl, (int)p.row_bytes);
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage), &tmap_w, x0, raw_n0, full);
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage + kRawBox), &tmap_w, x0 + 128, raw_n0, full);
        } else {  // 144- and 176-byte blocks start on 16-byte boundaries
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage), &tmap_w,
                      Sb<TYPE>::bytes * (sb0 + sbl), raw_n0, full);
        }
      };
      {
      if constexpr (STAGED) issue_raw(0);
      }
      for (int ks = 0; ks < nks; ks++) {
        const int s = ks % kStages;
        if constexpr (STAGED) {
          const int sbl = ks >> 2;
          if ((ks & 3) == 0 && sbl + 1 < nsb) {
            // the other buffer was last used by superblock sbl - 1: released by the dequant warps
            // well before the MMAs free this k-step's stage
            if (sbl >= 1) mbar_wait(smem_u32(&raw_bars[2 + ((sbl & 1) ^ 1)]), ((sbl - 1) >> 1) & 1);
            issue_raw(sbl + 1);
          }
        }
#pragma unroll
        for (int h = 0; h < kNSub; h++) {
          mbar_wait(smem_u32(&bars[kEmptyB + s * kNSub + h]), ((ks / kStages) & 1) ^ 1);
          const uint32_t full = smem_u32(&bars[kFullB + s * kNSub + h]);
          mbar_arrive_expect_tx(full, kBTile / kNSub);
          tma_load_2d(smem_u32(smem + s * kStageBytes + kATile + h * kNMma * kBK * 2), &tmap_x,
                      (ks0 + ks) * kBK, m0 + h * kNMma, full);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = idesc_bf16(kBM, kNMma);
      const uint32_t bar0 = smem_u32(&bars[0]);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem));
      uint32_t s = 0, ph = 0;
      for (int ks = 0; ks < nks; ks++) {
        mbar_wait(bar0 + 8 * s, ph);
        const uint32_t a_lo = a_lo0 + s * (kStageBytes >> 4);
#pragma unroll
        for (int h = 0; h < kNSub; h++) {
          mbar_wait(bar0 + 8 * (kFullB + s * kNSub + h), ph);
          tc_fence_after();
          umma4_bf16(tmem_base + h * kNMma, a_lo, a_lo + ((kATile + h * kNMma * kBK * 2) >> 4), idesc, ks != 0);
          umma_commit(bar0 + 8 * (kEmptyB + s * kNSub + h));  // frees this box of tokens
        }
        umma_commit(bar0 + 8 * (kEmptyA + s));             // frees the weight tile when the MMAs are done
        if (++s == kStages) {
          s = 0;
          ph ^= 1;
        }
      }
      umma_commit(smem_u32(&bars[kAccBar]));               // accumulator ready
    }
  } else if (R::is_dequant(warp)) {
    // ---------------------------------------------------------------- dequant producers
    const int dt = R::dequant_index(warp) * 32 + lane;
    const int r = dt & 127;                                // tile row 0..127
    const int part = dt >> 7;
    const int h0 = kQuarter ? part >> 1 : part;            // first (or only) half of every k-step
    const int q2 = kQuarter ? part & 1 : 0;                // the half's quarter
    const bool valid = n0 + r < p.n_out;
    const uint8_t *row = p.w + (long long)(valid ? n0 + r : 0) * p.row_bytes;
    Raw<TYPE> cur[kHalves], nxt[kHalves];
    auto fetch_all = [&](int ks, Raw<TYPE>(&dst)[kHalves]) {
      fetch_raw<TYPE>(row, ks0 + ks, h0, dst[0]);
      if constexpr (kHalves == 2) {
        if constexpr (TYPE == kQ6_K) {
          fetch_raw<TYPE, false>(row, ks0 + ks, 1, dst[1]);
#pragma unroll
          for (int w = 0; w < 8; w++) dst[1].qh[w] = dst[0].qh[w];
          dst[1].sc = dst[0].sc;
          dst[1].d = dst[0].d;
        } else {
          dst[1] = dst[0];  // Q4_K / Q5_K: both halves read the same bytes
        }
      }
    };
    if constexpr (STAGED) {
      const int sb0 = ks0 >> 2;
      const int rr = min(r + n0 - raw_n0, kBM - 1);  // this thread's row of the raw box
      for (int ks = 0; ks < nks; ks++) {
        const int s = ks % kStages;
        const int sbl = ks >> 2, buf = sbl & 1;
        if ((ks & 3) == 0) mbar_wait(smem_u32(&raw_bars[buf]), (sbl >> 1) & 1);
        if constexpr (kQuarter)
          fetch_quarter_from<TYPE>(raw_win + buf * kRawStage + rr * Sb<TYPE>::bytes, (ks0 + ks) & 3, q2, cur[0]);
        else if constexpr (TYPE == kQ6_K)
          fetch_staged_q6<kHalves>(raw_win + buf * kRawStage, rr,
                                   210 * (sb0 + sbl) - q6_window_start(sb0 + sbl, (int)p.row_bytes),
                                   (ks0 + ks) & 3, h0, cur);
        else  // the block of row r sits at r * block bytes: the global fetch code reads it as it is
          fetch_raw_from<TYPE>(raw_win + buf * kRawStage + rr * Sb<TYPE>::bytes, (ks0 + ks) & 3, h0, cur[0]);
        if ((ks & 3) == 3 || ks == nks - 1) {  // this warp has read all it needs of the window
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&raw_bars[2 + buf]));
        }
        mbar_wait(smem_u32(&bars[kEmptyA + s]), ((ks / kStages) & 1) ^ 1);
#pragma unroll
        for (int i = 0; i < kHalves; i++)
          expand_kstep<TYPE, kQuarter>(cur[i], ks0 + ks, h0 + i, smem + s * kStageBytes, r, valid, q2);
        fence_async_smem();                                   // generic-proxy writes -> tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[s]));
      }
    } else {
      fetch_all(0, cur);
      for (int ks = 0; ks < nks; ks++) {
        const int s = ks % kStages;
        if (ks + 1 < nks) fetch_all(ks + 1, nxt);             // in flight while this k-step expands
        mbar_wait(smem_u32(&bars[kEmptyA + s]), ((ks / kStages) & 1) ^ 1);
#pragma unroll
        for (int i = 0; i < kHalves; i++)
          expand_kstep<TYPE>(cur[i], ks0 + ks, h0 + i, smem + s * kStageBytes, r, valid);
        fence_async_smem();                                   // generic-proxy writes -> tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bars[s]));
#pragma unroll
        for (int i = 0; i < kHalves; i++) cur[i] = nxt[i];
      }
    }
  }
  // ---------------------------------------------------------------- epilogue
  if (R::in_epilogue(warp)) {
    mbar_wait(smem_u32(&bars[kAccBar]), 0);
    tc_fence_after();
    const int q = warp & 3;                                // TMEM lane quarter this warp may read
    const int n = n0 + 32 * q + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16);
    // the warps of a lane quarter take an equal share of the token columns each
    constexpr int kCols = BN / (isolate_mma_warp(TYPE, STAGED, BN) ? 4 : kDequantWarps / 4);
    const int cbeg = R::epilogue_chunk(warp) * kCols;
    if constexpr ((kCols / 4) % 32 == 0) {
      if (p.turns) {  // four splits: the groups of this warp's columns in the order of the turns
        constexpr int kEpiThreads = 32 * (isolate_mma_warp(TYPE, STAGED, BN) ? 16 : kDequantWarps);
        constexpr int kG = kCols / 4;
        unsigned *turn = p.turns + (size_t)(blockIdx.y * gridDim.x + blockIdx.x) * 4;
        const bool leader = threadIdx.x == (isolate_mma_warp(TYPE, STAGED, BN) ? 0 : 64);
#pragma unroll 1
        for (int t = 0; t < 4; t++) {
          const int g = ((int)blockIdx.z + t) & 3;
          if (leader) wait_turn(turn + g, (unsigned)t);
          asm volatile("bar.sync 2, %0;" ::"n"(kEpiThreads) : "memory");
#pragma unroll 1
          for (int c0 = cbeg + g * kG; c0 < cbeg + (g + 1) * kG; c0 += 32) {
            uint32_t v[32];
            tmem_ld32(taddr + c0, v);
            tmem_ld_wait();
            if (n < p.n_out) {
#pragma unroll
              for (int jj = 0; jj < 32; jj++) {
                const int m = m0 + c0 + jj;
                if (m < p.m_rows) {
                  float *dst = reinterpret_cast<float *>(p.y) + (long long)m * p.n_out + n;
                  if (t == 0) *dst = __uint_as_float(v[jj]);  // the group's first part: y needs no zeroing
                  else atomicAdd(dst, __uint_as_float(v[jj]));
                }
              }
            }
          }
          // the additions of all threads happen before the leader's release below (barrier, then a
          // cumulative gpu-scope release), and the next split's after its leader's acquire
          asm volatile("bar.sync 2, %0;" ::"n"(kEpiThreads) : "memory");
          if (leader)
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(turn + g), "r"(t == 3 ? 0u : (unsigned)(t + 1))
                         : "memory");
        }
      }
    }
    const bool plain_epilogue = !((kCols / 4) % 32 == 0 && p.turns);
#pragma unroll 1
    for (int c0 = cbeg; plain_epilogue && c0 < cbeg + kCols; c0 += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c0, v);
      tmem_ld_wait();
      if (n < p.n_out) {
#pragma unroll
        for (int jj = 0; jj < 32; jj++) {
          const int m = m0 + c0 + jj;
          if (m < p.m_rows) {
            const float f = __uint_as_float(v[jj]);
            if (p.splits > 1)  // two partial tiles onto zeros: the sum does not depend on their order
              atomicAdd(reinterpret_cast<float *>(p.y) + (long long)m * p.n_out + n, f);
            else if (p.out_bf16)
              reinterpret_cast<__nv_bfloat16 *>(p.y)[(long long)m * p.n_out + n] = __float2bfloat16_rn(f);
            else
              reinterpret_cast<float *>(p.y)[(long long)m * p.n_out + n] = f;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, BN);
}

// ---------------------------------------------------------------------------- the 2-CTA kernel
// A pair of CTAs (a cluster of two SMs) computes 256 weight rows x 512 tokens with
// tcgen05.mma.cta_group::2: each CTA dequantises its own 128 rows (the A operand of its half of
// M = 256) and loads only 128 of the 256 tokens of every B box; the tensor cores of both SMs read
// both halves.  Per k-step a CTA's shared memory then takes 32 KB of activations instead of 64 KB
// (half the L2 -> SM traffic of the one-CTA tile), which leaves room for five weight stages and
// three token stages where the one-CTA tile has two stages of 80 KB.
//   * CTA 0 of the pair issues the MMAs.  Its full barriers collect the arrivals of both CTAs'
//     dequant warps (remote mbarrier arrives) and the bytes of both CTAs' TMA loads (the loads name
//     CTA 0's barrier); the empty and accumulator barriers exist in both CTAs and are signalled by
//     one tcgen05.commit each.
//   * No load of this kernel is multicast.
//   * The accumulation order is the one-CTA kernel's: the results are equal bit for bit.
__device__ __forceinline__ uint32_t cluster_cta_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address of `addr` (shared memory of this CTA) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_in_cluster(uint32_t cluster_addr) {
  // default semantics (release at CTA scope): what the arrive has to order is this warp's
  // fence.proxy.async before it; a cluster-scope release costs a memory barrier per k-step and
  // warp (measured: the leading stall of the kernel)
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier at `cluster_addr` (any CTA of the pair) once every MMA issued so far
// by this thread has completed in both CTAs.
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_addr)
               : "memory");
}
// 2-D TMA tile load into this CTA's shared memory whose bytes are counted on a barrier of either
// CTA of the pair (cluster address).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *tmap, int c0, int c1,
                                                 uint32_t bar_cluster_addr) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], "
      "[%1, {%2, %3}], [%4];" ::"r"(dst),
      "l"(tmap), "r"(c0), "r"(c1), "r"(bar_cluster_addr)
      : "memory");
}

constexpr int kPairBN = 512;                 // tokens per pair tile: two accumulators of 256 columns
constexpr int kPairThreads = 32 * kIsoWarps;
constexpr int kPairBHalf = 128 * kBK * 2;    // this CTA's 128 tokens of a 256-token box: 16 KB
// Two rings: the dequantised weight tiles (16 KB per k-step) and the token boxes (2 x 16 KB per
// k-step and CTA).  They are decoupled because what a weight tile costs is latency, not work:
// from the commit that frees a slot over the expansion, the proxy fence and the (remote) arrive to
// the MMA thread's wake-up is more than two k-steps of MMAs, so the weight ring has to be deeper
// than the three token stages that fit.
constexpr int kPairBStages = 3;
constexpr int kPairBStage = 2 * kPairBHalf;  // 32 KB
__host__ __device__ constexpr int pair_a_stages(int type) {
  const int fit = (227 * 1024 - 1024 - 256 - raw_bytes(type, true) - kPairBStages * kPairBStage) / kATile;
  return fit < 6 ? fit : 6;
}

template <int TYPE>
__global__ void __launch_bounds__(kPairThreads, 1)
    gemm_prefill_pair_kernel(const __grid_constant__ CUtensorMap tmap_x,
                             const __grid_constant__ CUtensorMap tmap_w, const GemmParams p) {
  constexpr int kRawStage = raw_stage_bytes(TYPE);
  constexpr int kSA = pair_a_stages(TYPE), kSB = kPairBStages;
  static_assert(kSA >= 2, "at least two weight stages");
  constexpr int kDequantWarps = dequant_warps(TYPE, true);
  constexpr int kHalves = kDequantWarps >= 8 ? 1 : 2;
  static_assert(kDequantWarps == 16, "the warp roles below assume sixteen dequant warps");
  constexpr bool kQuarter = kDequantWarps == 16;
  constexpr int kNSub = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint8_t *smem_b = smem + kSA * kATile;
  uint8_t *raw_win = smem_b + kSB * kPairBStage;
  uint64_t *bars = reinterpret_cast<uint64_t *>(raw_win + raw_bytes(TYPE, true));
  // bars: full_a[SA] | full_b[SB][2] | empty_a[SA] | empty_b[SB][2] | acc_full | raw_full[2] |
  // raw_empty[2]; the full barriers are used in CTA 0 only
  constexpr int kFullB = kSA, kEmptyA = kFullB + kSB * kNSub, kEmptyB = kEmptyA + kSA;
  constexpr int kAccBar = kEmptyB + kSB * kNSub;
  static_assert((kAccBar + 5) * 8 + 4 <= 256, "barriers fit their 256 bytes");
  uint64_t *raw_bars = bars + kAccBar + 1;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(raw_bars + 4);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_cta_rank();  // 0 issues the MMAs
  const int n0 = blockIdx.x * kBM, m0 = blockIdx.y * kPairBN;
  const int raw_n0 = min(n0, p.n_out - kBM);
  const int nks = p.k_in / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kSA; s++) {
      mbar_init(smem_u32(&bars[s]), 2 * kDequantWarps);    // full_a: the dequant warps of both CTAs
      mbar_init(smem_u32(&bars[kEmptyA + s]), 1);          // empty_a: tcgen05.commit
    }
    for (int s = 0; s < kSB; s++) {
      for (int h = 0; h < kNSub; h++) {
        mbar_init(smem_u32(&bars[kFullB + s * kNSub + h]), 1);   // full_b: CTA 0's TMA thread + both CTAs' bytes
        mbar_init(smem_u32(&bars[kEmptyB + s * kNSub + h]), 1);  // empty_b: tcgen05.commit
      }
    }
    mbar_init(smem_u32(&bars[kAccBar]), 1);                // accumulator complete
    mbar_init(smem_u32(&raw_bars[0]), 1);
    mbar_init(smem_u32(&raw_bars[1]), 1);
    mbar_init(smem_u32(&raw_bars[2]), kDequantWarps);
    mbar_init(smem_u32(&raw_bars[3]), kDequantWarps);
    mbar_fence_init();
  }
  if (warp == 1) {  // the same warp of both CTAs takes part in the pair's allocation
    tmem_alloc_pair(smem_u32(tmem_slot), kPairBN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();  // barriers initialised and TMEM allocated in both CTAs
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  using R = Roles<true>;
  if (warp == R::tma_warp) {
    // ---------------------------------------------------------------- activations and raw weights via TMA
    if (lane == 0) {
      const int nsb = (nks + 3) >> 2;
      auto issue_raw = [&](int sbl) {
        const uint32_t full = smem_u32(&raw_bars[sbl & 1]);
        mbar_arrive_expect_tx(full, kRawStage);
        if constexpr (TYPE == kQ6_K) {
          const int x0 = q6_window_start(sbl, (int)p.row_bytes);
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage), &tmap_w, x0, raw_n0, full);
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage + kRawBox), &tmap_w, x0 + 128, raw_n0, full);
        } else {
          tma_load_2d(smem_u32(raw_win + (sbl & 1) * kRawStage), &tmap_w, Sb<TYPE>::bytes * sbl, raw_n0, full);
        }
      };
      issue_raw(0);
      for (int ks = 0; ks < nks; ks++) {
        const int s = ks % kSB;
        const int sbl = ks >> 2;
        if ((ks & 3) == 0 && sbl + 1 < nsb) {
          if (sbl >= 1) mbar_wait(smem_u32(&raw_bars[2 + ((sbl & 1) ^ 1)]), ((sbl - 1) >> 1) & 1);
          issue_raw(sbl + 1);
        }
#pragma unroll
        for (int h = 0; h < kNSub; h++) {
          mbar_wait(smem_u32(&bars[kEmptyB + s * kNSub + h]), ((ks / kSB) & 1) ^ 1);
          const uint32_t full = smem_u32(&bars[kFullB + s * kNSub + h]);
          if (rank == 0) mbar_arrive_expect_tx(full, 2 * kPairBHalf);  // both CTAs' halves of the box
          tma_load_2d_pair(smem_u32(smem_b + s * kPairBStage + h * kPairBHalf), &tmap_x, ks * kBK,
                           m0 + h * 256 + (int)rank * 128, map_to_cta(full, 0));
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issue (CTA 0)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = idesc_bf16(256, 256);
      // the barriers' addresses in both CTAs, as cluster addresses (linear in the barrier index)
      const uint32_t bars0 = map_to_cta(smem_u32(&bars[0]), 0), bars1 = map_to_cta(smem_u32(&bars[0]), 1);
      const uint32_t bar0 = smem_u32(&bars[0]);
      const uint32_t a_lo0 = smem_desc_lo(smem_u32(smem)), b_lo0 = smem_desc_lo(smem_u32(smem_b));
      uint32_t sa = 0, pa = 0, s = 0, ph = 0;
      for (int ks = 0; ks < nks; ks++) {
        mbar_wait(bar0 + 8 * sa, pa);
#pragma unroll
        for (int h = 0; h < kNSub; h++) {
          mbar_wait(bar0 + 8 * (kFullB + s * kNSub + h), ph);
          tc_fence_after();
          umma4_bf16_pair(tmem_base + h * 256, a_lo0 + sa * (kATile >> 4),
                          b_lo0 + ((s * kPairBStage + h * kPairBHalf) >> 4), idesc, ks != 0);
          umma_commit_pair(bars0 + 8 * (kEmptyB + s * kNSub + h));
          umma_commit_pair(bars1 + 8 * (kEmptyB + s * kNSub + h));
        }
        umma_commit_pair(bars0 + 8 * (kEmptyA + sa));
        umma_commit_pair(bars1 + 8 * (kEmptyA + sa));
        if (++sa == kSA) {
          sa = 0;
          pa ^= 1;
        }
        if (++s == kSB) {
          s = 0;
          ph ^= 1;
        }
      }
      umma_commit_pair(bars0 + 8 * kAccBar);
      umma_commit_pair(bars1 + 8 * kAccBar);
    }
  } else if (R::is_dequant(warp)) {
    // ---------------------------------------------------------------- dequant producers
    const int dt = R::dequant_index(warp) * 32 + lane;
    const int r = dt & 127;
    const int part = dt >> 7;
    const int h0 = kQuarter ? part >> 1 : part;
    const int q2 = kQuarter ? part & 1 : 0;
    const bool valid = n0 + r < p.n_out;
    Raw<TYPE> cur[kHalves];
    const int rr = max(0, min(r + n0 - raw_n0, kBM - 1));  // this thread's row of the raw box
    for (int ks = 0; ks < nks; ks++) {
      const int s = ks % kSA;
      const int sbl = ks >> 2, buf = sbl & 1;
      if ((ks & 3) == 0) mbar_wait(smem_u32(&raw_bars[buf]), (sbl >> 1) & 1);
      if constexpr (kQuarter)
        fetch_quarter_from<TYPE>(raw_win + buf * kRawStage + rr * Sb<TYPE>::bytes, ks & 3, q2, cur[0]);
      else if constexpr (TYPE == kQ6_K)
        fetch_staged_q6<kHalves>(raw_win + buf * kRawStage, rr,
                                 210 * sbl - q6_window_start(sbl, (int)p.row_bytes), ks & 3, h0, cur);
      else
        fetch_raw_from<TYPE>(raw_win + buf * kRawStage + rr * Sb<TYPE>::bytes, ks & 3, h0, cur[0]);
      if ((ks & 3) == 3 || ks == nks - 1) {
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&raw_bars[2 + buf]));
      }
      mbar_wait(smem_u32(&bars[kEmptyA + s]), ((ks / kSA) & 1) ^ 1);
#pragma unroll
      for (int i = 0; i < kHalves; i++)
        expand_kstep<TYPE, kQuarter>(cur[i], ks, h0 + i, smem + s * kATile, r, valid, q2);
      fence_async_smem();  // generic-proxy writes -> tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive_in_cluster(map_to_cta(smem_u32(&bars[s]), 0));
    }
  }
  // ---------------------------------------------------------------- epilogue (own 128 rows)
  if (R::in_epilogue(warp)) {
    mbar_wait(smem_u32(&bars[kAccBar]), 0);
    tc_fence_after();
    const int q = warp & 3;
    const int n = n0 + 32 * q + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(32 * q) << 16);
    constexpr int kCols = kPairBN / 4;
    const int cbeg = R::epilogue_chunk(warp) * kCols;
#pragma unroll 1
    for (int c0 = cbeg; c0 < cbeg + kCols; c0 += 32) {
      uint32_t v[32];
      tmem_ld32(taddr + c0, v);
      tmem_ld_wait();
      if (n < p.n_out) {
#pragma unroll
        for (int jj = 0; jj < 32; jj++) {
          const int m = m0 + c0 + jj;
          if (m < p.m_rows) {
            const float f = __uint_as_float(v[jj]);
            if (p.out_bf16)
              reinterpret_cast<__nv_bfloat16 *>(p.y)[(long long)m * p.n_out + n] = __float2bfloat16_rn(f);
            else
              reinterpret_cast<float *>(p.y)[(long long)m * p.n_out + n] = f;
          }
        }
      }
    }
  }

  tc_fence_before();
  cluster_sync_all();  // both epilogues done: neither CTA's TMEM or shared memory is in use any more
  if (warp == 1) tmem_dealloc_pair(tmem_base, kPairBN);
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// The turn counters of the ordered four-way split: one region of the static device array per
// (device, stream) that has used it, so that launches on different streams do not share counters.
constexpr int kTurnSlots = 8, kTurnTiles = 64;
std::mutex g_turn_mutex;
unsigned *g_turn_base[64] = {nullptr};
cudaStream_t g_turn_streams[64][kTurnSlots];
int g_turn_nstreams[64] = {0};
unsigned *turn_region(cudaStream_t s) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_turn_mutex);
  if (!g_turn_base[dev]) {
    void *a = nullptr;
    if (cudaGetSymbolAddress(&a, g_prefill_turns) != cudaSuccess || !a) return nullptr;
    g_turn_base[dev] = static_cast<unsigned *>(a);
  }
  int slot = -1;
  for (int i = 0; i < g_turn_nstreams[dev]; i++)
    if (g_turn_streams[dev][i] == s) slot = i;
  if (slot < 0) {
    if (g_turn_nstreams[dev] == kTurnSlots) return nullptr;
    slot = g_turn_nstreams[dev]++;
    g_turn_streams[dev][slot] = s;
  }
  return g_turn_base[dev] + (size_t)slot * kTurnTiles * 4;
}

int g_prefill_force_bn = 0;  // diagnostics: 0 = automatic, else the token-tile width to use
int g_prefill_stage_raw = 1;    // diagnostics: 0 = dequant threads read global memory directly
int g_prefill_force_split = 0;  // diagnostics: 0 = automatic, 1 = never split along K, 2 = two splits where allowed, 3 = four

template <int TYPE, int BN, bool STAGED>
int launch(const void *d_w, const void *d_x, void *d_y, int out_type, int m_rows, int n_out,
           int k_in, int splits, cudaStream_t s) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return COGNI_QMM_ERR_DEVICE;
  const long long row_bytes = (long long)(k_in / 256) * Sb<TYPE>::bytes;
  CUtensorMap tmap, tmap_w;
  if (STAGED) {
    // the weights as a byte matrix [n_out, row_bytes]: boxes of 128 rows x 128 bytes
    const cuuint64_t wdims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_out};
    const cuuint64_t wstrides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t wbox[2] = {TYPE == kQ6_K ? 128u : (cuuint32_t)Sb<TYPE>::bytes, 128};
    const cuuint32_t westr[2] = {1, 1};
    CUresult wr = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d_w), wdims,
                         wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         TYPE == kQ6_K ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (wr != CUDA_SUCCESS) return (int)wr;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k_in, (cuuint64_t)m_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k_in * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)(BN > 256 ? 256 : BN)};
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(d_x), dims,
                       strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return (int)cr;
  constexpr int smem = stages_for(BN, raw_bytes(TYPE, STAGED)) * (kATile + BN * kBK * 2) +
                       raw_bytes(TYPE, STAGED) + 1024 /*alignment*/ + 256 /*barriers*/;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_prefill_kernel<TYPE, BN, STAGED>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  GemmParams p;
  p.w = static_cast<const uint8_t *>(d_w);
  p.y = d_y;
  p.m_rows = m_rows; p.n_out = n_out; p.k_in = k_in;
  p.out_bf16 = out_type == COGNI_QMM_OUT_BF16;
  p.row_bytes = row_bytes;
  if (!STAGED) tmap_w = tmap;  // unused by the kernel
  const int nks = k_in / kBK;
  p.splits = splits;
  p.ks_per_split = splits > 1 ? ((nks + splits - 1) / splits + 3) / 4 * 4 : nks;  // whole superblocks
  p.turns = nullptr;
  if (splits == 4) {  // the caller has checked that the tiles fit the region and the SMs
    p.turns = turn_region(s);
    if (!p.turns) return COGNI_QMM_ERR_LIMIT;
  }
  if (splits == 2) {  // (four ordered splits store their first part)
    cudaError_t e = cudaMemsetAsync(d_y, 0, (size_t)m_rows * n_out * sizeof(float), s);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((n_out + kBM - 1) / kBM, (m_rows + BN - 1) / BN, splits);
  gemm_prefill_kernel<TYPE, BN, STAGED><<<grid, threads_for(TYPE, STAGED, BN), smem, s>>>(tmap, tmap_w, p);
  return (int)cudaGetLastError();
}

int g_prefill_pair = 1;  // diagnostics: 0 = the one-CTA kernel for 512-token tiles too

// The 2-CTA kernel: 256 weight rows x 512 tokens per cluster of two CTAs.
template <int TYPE>
int launch_pair(const void *d_w, const void *d_x, void *d_y, int out_type, int m_rows, int n_out,
                int k_in, cudaStream_t s) {
  EncodeTiledFn encode = encode_tiled_fn();
  if (!encode) return COGNI_QMM_ERR_DEVICE;
  const long long row_bytes = (long long)(k_in / 256) * Sb<TYPE>::bytes;
  CUtensorMap tmap, tmap_w;
  {
    const cuuint64_t wdims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)n_out};
    const cuuint64_t wstrides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t wbox[2] = {TYPE == kQ6_K ? 128u : (cuuint32_t)Sb<TYPE>::bytes, 128};
    const cuuint32_t westr[2] = {1, 1};
    CUresult wr = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(d_w), wdims,
                         wstrides, wbox, westr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         TYPE == kQ6_K ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (wr != CUDA_SUCCESS) return (int)wr;
  }
  const cuuint64_t dims[2] = {(cuuint64_t)k_in, (cuuint64_t)m_rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k_in * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, 128};  // a CTA's 128 tokens of a 256-token box
  const cuuint32_t estr[2] = {1, 1};
  CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(d_x), dims,
                       strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return (int)cr;
  constexpr int smem = pair_a_stages(TYPE) * kATile + kPairBStages * kPairBStage + raw_bytes(TYPE, true) +
                       1024 /*alignment*/ + 256 /*barriers*/;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemm_prefill_pair_kernel<TYPE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  GemmParams p;
  p.w = static_cast<const uint8_t *>(d_w);
  p.y = d_y;
  p.m_rows = m_rows; p.n_out = n_out; p.k_in = k_in;
  p.out_bf16 = out_type == COGNI_QMM_OUT_BF16;
  p.row_bytes = row_bytes;
  p.splits = 1;
  p.ks_per_split = k_in / kBK;
  p.turns = nullptr;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * ((n_out + 2 * kBM - 1) / (2 * kBM)), (m_rows + kPairBN - 1) / kPairBN, 1);
  cfg.blockDim = dim3(kPairThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_prefill_pair_kernel<TYPE>, tmap, tmap_w, p);
}

template <int TYPE>
int launch_typed(const void *d_w, const void *d_x, void *d_y, int out_type, int m_rows, int n_out,
                 int k_in, cudaStream_t s) {
  // Token-tile width: wider tiles do less dequant work per flop, narrower ones fill the SMs in
  // fewer, fuller waves.  Measured time of a tile of 128 / 256 / 512 tokens (in_dim 4096, one wave,
  // us): Q4_K 39 / 45 / 61 (the 512-token tile on a CTA pair; 63 on one CTA), Q5_K 40 / 45 / 60,
  // IQ4_NL 49 / 52 / 66, Q6_K 53 / 59 / 69, Q8_0 58 / 67 / 81.  Pick the width with the least
  // waves x tile time.
  static int sms_of[64] = {0};  // per device: a process may drive GPUs of different sizes
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = dev >= 0 && dev < 64 ? sms_of[dev] : 0;
  if (!sms) {
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    if (dev >= 0 && dev < 64) sms_of[dev] = sms;
  }
  const long long row_tiles = (n_out + kBM - 1) / kBM;
  const double rel256 = TYPE == kQ4_K || TYPE == kQ5_K || TYPE == kQ8_0 ? 1.15 : 1.10;
  const double rel512 = TYPE == kQ4_K || TYPE == kQ5_K ? 1.55 : TYPE == kIQ4_NL ? 1.37 : TYPE == kQ8_0 ? 1.41 : 1.31;
  // Few row tiles against many SMs (a down projection at a short prompt): two CTAs per tile take
  // half of K each and add their partial tiles onto a zeroed f32 y.  Two addends commute, so the
  // result stays independent of the order; more splits would not.  The price is the memset of y
  // and read-modify-write instead of plain stores: about 12 bytes of HBM traffic per output
  // element, weighed here against the measured time of a 128-token tile's k-step (microseconds).
  const bool may_split = out_type == COGNI_QMM_OUT_F32 && k_in / kBK >= 16 && g_prefill_force_split != 1;
  const double us_per_kstep = TYPE == kQ4_K || TYPE == kQ5_K ? 0.61 : TYPE == kIQ4_NL ? 0.76 : TYPE == kQ6_K ? 0.83 : 0.92;
  const double tile_us = us_per_kstep * (k_in / kBK);
  const double split_us = 12.0 * (double)m_rows * (double)n_out / 6.0e6;
  auto cost = [&](int bn, double rel, int splits) {
    const long long tiles = row_tiles * ((m_rows + bn - 1) / bn) * splits;
    return (double)((tiles + sms - 1) / sms) * rel * tile_us / splits + (splits > 1 ? split_us : 0.0);
  };
  const int widths[3] = {128, 256, 512};
  const double rels[3] = {1.0, rel256, rel512};
  int bn = 0, splits = 1;
  double best = 1e30;
  for (int i = 0; i < 3; i++) {
    if (g_prefill_force_bn && g_prefill_force_bn != widths[i]) continue;
    for (int sp = 1; sp <= (may_split ? 2 : 1); sp++) {
      if (g_prefill_force_split >= 2 && may_split && sp != 2) continue;
      const double c = cost(widths[i], rels[i], sp);
      if (c <= best) { best = c; bn = widths[i]; splits = sp; }
    }
  }
  // Four splits in a fixed order of addition (see wait_turn): 512-token tiles only (the groups of
  // the epilogue), all CTAs resident at once, a quarter of K of at least 16 k-steps each; costs
  // the two-split price plus four rounds of turn-taking (about 3 us).
  {
    const long long tiles4 = row_tiles * ((m_rows + 511) / 512);
    const bool can4 = may_split && k_in / kBK >= 64 && tiles4 * 4 <= sms && tiles4 <= kTurnTiles &&
                      (!g_prefill_force_bn || g_prefill_force_bn == 512);
    if (can4 && g_prefill_force_split != 2) {
      const double c4 = rel512 * tile_us / 4 + split_us + 3.0;
      if (c4 < best || g_prefill_force_split == 3) { best = c4; bn = 512; splits = 4; }
    }
  }
  // Rows that are multiples of 16 bytes (always for Q4_K / Q5_K; Q6_K: in_dim a multiple of 2048)
  // of a matrix with at least one full row tile can be fetched by TMA: the raw superblocks of the
  // tile's rows are then staged through shared memory
  {
    const long long row_bytes = (long long)(k_in / 256) * Sb<TYPE>::bytes;
    if (TYPE != kQ8_0 && row_bytes % 16 == 0 && n_out >= kBM && g_prefill_stage_raw) {
      if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        if (bn == 512 && splits == 1 && g_prefill_pair)
          return launch_pair<TYPE>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, s);
      }
      if (bn == 512) return launch<TYPE, 512, true>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
      if (bn == 256) return launch<TYPE, 256, true>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
      return launch<TYPE, 128, true>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
    }
  }
  if (bn == 512) return launch<TYPE, 512, false>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
  if (bn == 256) return launch<TYPE, 256, false>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
  return launch<TYPE, 128, false>(d_w, d_x, d_y, out_type, m_rows, n_out, k_in, splits, s);
}

}  // namespace

int launch_gemm_prefill(int type, const void *d_w, const void *d_x_bf16, void *d_y, int out_type,
                        int m_rows, int n_out, int k_in, cudaStream_t s) {
  switch (type) {
    case kQ4_K: return launch_typed<kQ4_K>(d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in, s);
    case kQ5_K: return launch_typed<kQ5_K>(d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in, s);
    case kQ6_K: return launch_typed<kQ6_K>(d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in, s);
    case kQ8_0: return launch_typed<kQ8_0>(d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in, s);
    case kIQ4_NL: return launch_typed<kIQ4_NL>(d_w, d_x_bf16, d_y, out_type, m_rows, n_out, k_in, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

void gemm_prefill_set_tile(int bn) { g_prefill_force_bn = bn; }
void gemm_prefill_set_split(int mode) { g_prefill_force_split = mode; }
void gemm_prefill_set_stage_raw(int on) { g_prefill_stage_raw = on; }
void gemm_prefill_set_pair(int on) { g_prefill_pair = on; }

unsigned gemm_prefill_timeouts() {
  unsigned v = 0;
  cudaMemcpyFromSymbol(&v, g_pipe_wait_timeouts, sizeof(v));
  return v;
}

int gemm_prefill_reset_timeouts() {
  const unsigned zero = 0;
  cudaError_t e = cudaMemcpyToSymbol(g_pipe_wait_timeouts, &zero, sizeof(zero));
  if (e != cudaSuccess) return (int)e;
  void *turns = nullptr;  // an expired wait can leave turn counters of the ordered split non-zero
  e = cudaGetSymbolAddress(&turns, g_prefill_turns);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(turns, 0, sizeof(unsigned) * 8 * 64 * 4);
}

}  // namespace cogni
