// Decode GEMV for Q4_K / Q5_K / Q6_K / Q8_0 straight from the raw GGUF blocks (sm_100a):
// bulk-async staging + integer tensor-core MMAs on the raw quants.  The description below is the
// batch 1-2 arrangement; batches 3-8 per launch use the dense column sets described further down.
//
// The kernel is HBM-bound; at 6.5 TB/s an SM has about three issue slots per weight, and the
// integer (ALU) pipe runs at half rate, so the design removes every per-weight instruction it can:
//
//  * A persistent CTA per SM walks row tiles of 16 output rows.  One producer warp streams the
//    tiles' rows with 1-D bulk async copies (cp.async.bulk, completion on an mbarrier) into a ring
//    of shared-memory stages, KB superblocks of every row per stage.  The consumer warps take
//    work items (one superblock of a 16-row tile, or the fold of a finished tile) in order from a
//    shared counter: every warp stays busy until the CTA runs dry and the warps of a scheduler
//    are always in different phases (waiting for data, decoding scales, issuing MMAs, folding),
//    which is what hides the long dependent chains of this kernel.  Rows that are only 2/8-byte
//    aligned (Q6_K) are fetched from the 16-byte boundary below their start.
//  * Activations are quantised once per CTA to 15-bit block floating point: per scale group
//    (32 elements for Q4_K/Q5_K, 16 for Q6_K) x = sx * n with |n| <= 16256, n = 128*hi + lo, hi
//    and lo int8 (hi = n >> 7, lo = n & 127).  The rounding step is 2^-14 of the group maximum,
//    i.e. ~4e-5 relative rms.  The warps do this on the way, superblock by superblock, while they
//    work through the CTA's first tile.
//  * The quants feed mma.sync.m16n8k32 (u8 x s8 -> s32) as they are.  One MMA covers two scale
//    groups at once: the hi and lo planes of group A occupy columns 0-1 with zeros in group B's
//    k-slots, group B's planes columns 2-3 with zeros in A's slots, so each lane ends up with the
//    exact integer dot product of one (row, group) pair.  It is combined (128*hi + lo), converted
//    once and multiplied by d*sc*sx in fp32; accumulation across groups is fp32.
//    Q4_K does not even separate its nibbles: a byte b = lo + 16*hi goes in whole (k-slots 0..15)
//    next to H = b & 0xF0 (k-slots 16..31).  Group A's columns hold x in the first half and -x in
//    the second, so the MMA yields sum((b - H) * x) = sum(lo * x); group B's columns hold x only in
//    the second half and yield 16 * sum(hi * x), the 1/16 being folded into that group's scale.
//    That is one AND per eight weights.
//  * Terms that do not depend on the quants (Q4_K/Q5_K -dmin*m, Q6_K's -32) are folded into one
//    correction per (row, superblock) from the per-group sums of the quantised activations.
//  * Each superblock's partial sums go to a per-tile buffer indexed by superblock; a later work
//    item adds them in superblock order, adds the addend (bias or residual) and stores y.  The
//    result does not depend on which warp computed what.
//
// The kernel is launched with programmatic stream serialisation: it lets its successor start
// launching at once and itself waits for its predecessor only before it touches x or y.  With
// `resident` weights the producer starts fetching weights before that wait.
#include <climits>
#include <mutex>
#include <type_traits>

#include "qmm_common.cuh"
#include "tma_pipe.cuh"

// Timing diagnostics (stream only / decode only / no copies / sleeping items) give invalid results
// and exist only in builds made with -DCOGNI_QMM_DIAG_TIMING; the shipped kernels carry none.
#ifdef COGNI_QMM_DIAG_TIMING
#define COGNI_DIAG(x) (x)
#else
#define COGNI_DIAG(x) 0
#endif

namespace cogni {
namespace {

// Consumer warps per CTA.  Every warp holds the stage bytes of its item until it is done, so
// more warps leave fewer stages for the copies in flight; 16 (20 for single-superblock items of
// the 210-byte Q6_K blocks) measured best for batches 1-2.  The 4- and 8-row instances are bound
// by their consumer warps' latencies and take 20 (batch 8: Q4_K 65536 x 4096 55.4 -> 51.5 us,
// 4096 x 16384 32.6 -> 27.2, Q5_K 65536 x 4096 69.6 -> 60.5; 24 warps: Q4_K 53.2), except Q6_K,
// whose slab launches need the stages (4096 x 12288 with 20: 29.3 -> 31.4 us, the 151936 x 5120
// head 262 -> 278).
__host__ __device__ constexpr int consumer_warps(int type, int pair, int nb = 1) {
  if (nb > 2) return type == kQ6_K ? 16 : 20;
  return type == kQ6_K && pair == 1 ? 20 : 16;
}
// tiles whose partial sums can be pending (power of 2)
__host__ __device__ constexpr int fold_bufs(int nb) { return nb > 2 ? 2 : 4; }
// One warp issues bulk copies at roughly one per 70-90 cycles however many of its lanes take
// part; the copy unit itself accepts several times that, so the rows of a stage are split over
// kPW producer warps.
constexpr int kPW = 4;                       // producer warps
constexpr int kR = 16;                       // rows per tile
constexpr size_t kDynSmemMax = 227 * 1024 - 1024;
constexpr int kNMax = 16256;                 // |n| bound: 127 * 128
static_assert(kR == 4 * kPW, "each producer warp issues four rows of a stage");

constexpr int stage_row_stride(int bb, int kb, bool unaligned_rows) {
  int rs = (bb * kb + (unaligned_rows ? 16 : 0) + 15) / 16 * 16;
  for (;; rs += 16) {
    const int m = rs % 128;
    if (unaligned_rows ? ((m / 16) % 2 == 1) : (m == 32 || m == 96)) return rs;
  }
}

template <int TYPE> struct Cfg;
template <> struct Cfg<kQ4_K> {
  static constexpr int BB = 144, KB = 16, NG = 8, GROUP = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr bool HAS_MIN = true;
};
template <> struct Cfg<kQ5_K> {
  static constexpr int BB = 176, KB = 16, NG = 8, GROUP = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr bool HAS_MIN = true;
};
// Q8_0: eight 34-byte blocks (fp16 d + 32 int8) are treated as one 272-byte superblock of eight
// scale groups; rows and superblocks are 16-byte aligned, the quants of a block 2 bytes off.
template <> struct Cfg<kQ8_0> {
  static constexpr int BB = 272, KB = 8, NG = 8, GROUP = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr bool HAS_MIN = false;
};
// IQ4_NL: eight 18-byte blocks (fp16 d + 16 bytes of nibble pairs: element i in the low nibble of
// byte i, element 16 + i in the high one; values through a 16-entry table) form a 144-byte
// superblock of eight scale groups.  Only the 4- and 8-row instances of the kernel exist for it.
template <> struct Cfg<kIQ4_NL> {
  static constexpr int BB = 144, KB = 16, NG = 8, GROUP = 32;
  static constexpr int RS = stage_row_stride(BB, KB, false);
  static constexpr bool HAS_MIN = false;
};
template <> struct Cfg<kQ6_K> {
  static constexpr int BB = 210, KB = 8, NG = 16, GROUP = 16;
  static constexpr int RS = stage_row_stride(BB, KB, true);
  static constexpr bool HAS_MIN = false;
};

constexpr int kMaxJobs = 32;  // weight matrices one launch can take (they share x)
constexpr int kMaxRanks = 8;   // GPUs of one box
constexpr int kMaxItems = 128;  // work items (superblocks or pairs) per row tile: in_dim <= 32768

struct Job {
  const uint8_t *w;
  const float *addend;
  float *y;
  int out_dim;
};

struct Exchange {
  int world, rank;                  // world <= 1: no exchange
  long long peer_delta[kMaxRanks];  // bytes from an address in this GPU's buffer to the same place in GPU g's, as mapped here ([rank]: 0)
  unsigned *epoch;                  // exchanges this GPU has completed on this buffer set
  unsigned *ticket;                 // CTA arrivals of the running launch, zero between launches
};

// Where a kernel's activations come from: plain f32, or the 8-byte (value, epoch) words an
// exchanging launch leaves in the gather buffer of every GPU.  Such a word is written by ONE
// 8-byte store, so value and epoch arrive together: the reader polls the word until it carries the
// epoch it expects and needs no fence, flag or barrier (the "LL" scheme of collective libraries).
struct XSrc {
  int ll;
  unsigned epoch;
};
// Four consecutive activations from element `off` on.  LL is a template parameter so that the
// plain path stays a bare load: a run-time branch in front of every load would keep the compiler
// from issuing a lane's loads together (measured: +2 us per launch).
template <bool LL>
__device__ __forceinline__ float4 ld4x(const float *x, long long off, const XSrc &src) {
  if constexpr (!LL) return __ldg(reinterpret_cast<const float4 *>(x + off));
  const uint2 *w = reinterpret_cast<const uint2 *>(x) + off;  // 16-byte aligned: off is a multiple of 4
  uint4 a, b;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 0;; spin++) {
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(w) : "memory");
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(w + 2) : "memory");
    if (a.y == src.epoch && a.w == src.epoch && b.y == src.epoch && b.w == src.epoch) break;
    if ((spin & 255u) == 255u) {  // bounded like every wait: count the expiry and carry on
      if (pipe_broken()) break;
      if (global_ns() - t0 > kPipeWaitLimitNs) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        break;
      }
    }
  }
  return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}
// One output value: plain, or as a (value, epoch) word here and at the same place on every peer.
__device__ __forceinline__ void store_y(float *y, long long idx, float v, const Exchange &ex, unsigned e_out) {
  if (ex.world <= 1) {
    y[idx] = v;
    return;
  }
  char *w = reinterpret_cast<char *>(reinterpret_cast<uint2 *>(y) + idx);
  for (int gpu = 0; gpu < ex.world; gpu++)
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(w + ex.peer_delta[gpu]),
                 "r"(__float_as_uint(v)), "r"(e_out) : "memory");
}

struct Params {
  const float *x;
  const float *x_up;  // non-null: the activations are silu(x) * x_up (SwiGLU), formed while quantising
  const float *norm_w;  // non-null: the activations are RMSNorm(x) * norm_w, normalised while quantising
  const float *norm_x;  // the rows the norm is taken over: norm_dim elements each (a launch may cover a column range of them)
  int norm_dim;
  int x_pitch;          // floats between the batch rows of x / x_up
  float norm_eps;
  long long addend_stride;  // floats between the batch rows of an addend; -1: the job's out_dim
  int in_dim;
  int batch;     // rows of x (batches above 2: may be below the kernel's NB)
  int nblk, nchunks, stages;
  int njobs;
  int tcum[kMaxJobs + 1];  // tcum[j] = first global tile of job j; tcum[njobs] = all tiles
  Job jobs[kMaxJobs];
  long long row_bytes;
  int off_flags, off_red, off_area, off_sx, off_xx, off_xq, off_stage, stage_bytes;
  int pair;      // superblocks per work item (1 or 2)
  int nflags;    // words of the per-item flags of x
  int resident;  // weights were complete before the preceding kernel started
  int debug;     // diagnostics: bits 0-1: 1 = no work on the stages, 2 = decode only; bit 2: no copies; bit 3: items sleep
  // K slabs: nslabs CTAs share a row tile, each takes nblk superblocks of the row (slab s: the
  // superblocks s*nblk ..); their partial sums meet in ws, the CTA that arrives last adds them up
  int nslabs;            // 1: every CTA takes whole rows
  float *ws;             // [tile][slab][batch row][16] partial sums
  unsigned *ws_tickets;  // [tile] arrival counters, zero between launches
  // Exchange of the outputs with the other GPUs of the box, fused into the kernel: every y value
  // goes, as a (value, epoch) word, into this GPU's gather buffer and into the same place of each
  // peer's (peer-mapped memory, ordinary 8-byte stores over NVLink).
  Exchange ex;
  int ex_wait;           // the activations are the (value, epoch) words of the exchange before this launch
  long long y_pitch;     // elements between the batch rows of y; 0: the job's out_dim
  long long *part_keys;  // fused top-1 (nullptr: plain GEMV)
  unsigned *counter;
  int32_t *top_idx;
  float *top_val;
  long long *top_key;
  int index_base;
};


template <int NW>
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(NW * 32) : "memory");
}
__device__ __forceinline__ void imma_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// s8 x s8 variants (Q8_0 quants are signed)
__device__ __forceinline__ void imma_s8_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                             uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}
__device__ __forceinline__ void imma_s8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 x 8 x 16 variants: one 16-element scale group per MMA (Q6_K with batches above 2)
__device__ __forceinline__ void imma16_zero(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
      "{%7,%7,%7,%7};"
      : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
      : "r"(a0), "r"(a1), "r"(b0), "r"(0));
}
// scale * (byte i of v), exactly rounded once: 0x4B0000bb is the float 2^23 + b, and
// fma(2^23 + b, scale, -2^23 * scale) = b * scale (the product 2^23 * scale is exact).
__device__ __forceinline__ float byte_times(uint32_t v, int i, float scale, float scale_2p23) {
  return fmaf(__uint_as_float(__byte_perm(v, 0x4B000000u, 0x7650 + i)), scale, -scale_2p23);
}

// Shared-memory layout of the quantised activations, in MMA B-fragment order.  A "unit" is 64
// consecutive-in-layout elements that one warp turns into two MMAs:
//   Q4_K/Q5_K  unit = (superblock, pair g4): elements 64*g4 .. 64*g4+63 (sub-blocks 2g4, 2g4+1)
//   Q6_K       unit = (superblock, half n, h): elements 128n + 32k + 16h + (0..15), k = 0..3
// Per unit: NCX = 4*NB columns (batch b, group slot sub, plane pl -> column 4b + 2sub + pl), per
// column 4 lanes t, per lane 16 bytes = (MMA0.b0, MMA0.b1, MMA1.b0, MMA1.b1).  A column of group
// slot `sub` only fills the b`sub` words; the other words stay zero.
template <int TYPE>
__device__ __forceinline__ int xq_word_offset(int e_in /*element within superblock*/, int ncx,
                                              int col_base /*4b + plane*/, int &sub) {
  int unit, t, m;
  if (TYPE == kQ6_K) {
    const int n = e_in >> 7, k = (e_in & 127) >> 5, h = (e_in & 31) >> 4;
    unit = 2 * n + h;
    m = k >> 1;
    sub = k & 1;
    t = (e_in & 15) >> 2;
  } else {
    const int g4 = e_in >> 6;
    unit = g4;
    sub = (e_in >> 5) & 1;
    t = (e_in & 31) >> 3;
    m = (e_in & 7) >> 2;
  }
  return ((unit * ncx + col_base + 2 * sub) * 4 + t) * 16 + m * 8 + sub * 4;
}

// ---------------------------------------------------------------------------- per-block work
// Area of one warp: per batch row 16 tile rows of AREA_ROW floats.  Row r holds d*sc*sx of the
// superblock's scale groups, ordered so that an MMA lane fetches the ones of its group slot `sub`
// with vector loads, then the row's correction term at index NG:
//   Q4_K/Q5_K/Q8_0  index 4*sub + g4           group 2*g4 + sub
//   Q6_K       index 8*sub + 4*n + 2*h + m     group 8*n + h + 2*sub + 4*m
template <int TYPE> struct Area {
  static constexpr int ROW = Cfg<TYPE>::NG + 4;  // 12 / 20 floats: rows stay 16-byte aligned
  static constexpr int BATCH = 16 * ROW;         // floats per batch row
};

// An item covers two neighbouring superblocks of a tile.  Lane (r = lane & 15, which = lane >> 4)
// decodes all scale groups of row r of superblock `which` of the pair into that superblock's half
// of the warp's area.
template <int TYPE, int NB>
__device__ __forceinline__ void decode_scales(const uint8_t *blk_row, int lane, int kblk,
                                              const float *SX, const float *XX, float *area) {
  using C = Cfg<TYPE>;
  using A = Area<TYPE>;
  constexpr int NH = C::NG / 2;  // groups per pass
  const int r = lane & 15;
  float *rows = area + (lane >> 4) * NB * A::BATCH + r * A::ROW;
  float corr[NB];
#pragma unroll
  for (int b = 0; b < NB; b++) corr[b] = 0.f;
  uint32_t u0 = 0, u1 = 0, u2 = 0;
  float d = 0.f, dmin = 0.f;
  if constexpr (C::HAS_MIN) {
    const uint4 h = *reinterpret_cast<const uint4 *>(blk_row);
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    d = __low2float(dd);
    dmin = __high2float(dd);
    u0 = h.y; u1 = h.z; u2 = h.w;
  } else if constexpr (TYPE == kQ6_K) {
    d = load_half_as_float(blk_row + 208);
  }
#pragma unroll
  for (int half = 0; half < 2; half++) {
    float dsc[NH], kk[NH];
    if constexpr (TYPE == kQ8_0) {  // the eight blocks' own fp16 scales; no minimum, no offset
#pragma unroll
      for (int i = 0; i < 4; i++) {
        dsc[i] = load_half_as_float(blk_row + 34 * (4 * half + i));
        kk[i] = 0.f;
      }
    } else if constexpr (C::HAS_MIN) {
      // four 6-bit scales / mins of this half as bytes (dequant.cr:240-249, four at a time)
      const uint32_t scw = half ? ((u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u)) : (u0 & 0x3f3f3f3fu);
      const uint32_t mnw = half ? (((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u)) : (u1 & 0x3f3f3f3fu);
      const float d23 = d * 8388608.f, ndmin = -dmin, ndmin23 = ndmin * 8388608.f;
      // Q4_K: the odd groups' integer sums arrive multiplied by 16 (see mma_block)
      const float dodd = TYPE == kQ4_K ? d * 0.0625f : d, dodd23 = dodd * 8388608.f;
#pragma unroll
      for (int i = 0; i < 4; i++) {
        dsc[i] = (i & 1) ? byte_times(scw, i, dodd, dodd23) : byte_times(scw, i, d, d23);
        kk[i] = byte_times(mnw, i, ndmin, ndmin23);
      }
    } else {
      const int8_t *sc = reinterpret_cast<const int8_t *>(blk_row + 192 + 8 * half);
#pragma unroll
      for (int i = 0; i < 8; i++) {
        dsc[i] = d * (float)sc[i];
        kk[i] = dsc[i];  // times -32 once, at the end
      }
    }
    // the half's groups are consecutive in the tables: NH * NB floats each, 16-byte aligned
    const int grp0 = kblk * C::NG + NH * half;
    float sxv[NH * NB], xxv[NH * NB];
#pragma unroll
    for (int i = 0; i < NH * NB / 4; i++) {
      const float4 a = reinterpret_cast<const float4 *>(SX + grp0 * NB)[i];
      const float4 c = reinterpret_cast<const float4 *>(XX + grp0 * NB)[i];
      sxv[4 * i] = a.x; sxv[4 * i + 1] = a.y; sxv[4 * i + 2] = a.z; sxv[4 * i + 3] = a.w;
      xxv[4 * i] = c.x; xxv[4 * i + 1] = c.y; xxv[4 * i + 2] = c.z; xxv[4 * i + 3] = c.w;
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      float *row = rows + b * A::BATCH;
      float v[NH];
#pragma unroll
      for (int i = 0; i < NH; i++) {
        v[i] = dsc[i] * sxv[i * NB + b];
        corr[b] = fmaf(kk[i], xxv[i * NB + b], corr[b]);
      }
      if constexpr (C::NG == 8) {  // groups 4*half + i: g4 = 2*half + (i >> 1), sub = i & 1
        *reinterpret_cast<float2 *>(row + 2 * half) = make_float2(v[0], v[2]);
        *reinterpret_cast<float2 *>(row + 4 + 2 * half) = make_float2(v[1], v[3]);
      } else {  // groups 8*half + i: n = half, h = i & 1, sub = (i >> 1) & 1, m = i >> 2
        *reinterpret_cast<float4 *>(row + 4 * half) = make_float4(v[0], v[4], v[1], v[5]);
        *reinterpret_cast<float4 *>(row + 8 + 4 * half) = make_float4(v[2], v[6], v[3], v[7]);
      }
    }
  }
#pragma unroll
  for (int b = 0; b < NB; b++) rows[b * A::BATCH + C::NG] = TYPE == kQ6_K ? -32.f * corr[b] : corr[b];
}

// Single-superblock items: lanes (r = lane & 15, half = lane >> 4) decode one half of the scale
// groups of row r; the two halves' corrections are combined with one shuffle.
// d*sc (Q4_K's odd groups: d*sc/16, see mma_block) and the offset factors of one half (NG/2
// groups) of a row's superblock.
template <int TYPE>
__device__ __forceinline__ void half_scales(const uint8_t *blk_row, int half,
                                            float (&dsc)[Cfg<TYPE>::NG / 2],
                                            float (&kk)[Cfg<TYPE>::NG / 2]) {
  using C = Cfg<TYPE>;
  if constexpr (TYPE == kQ8_0 || TYPE == kIQ4_NL) {  // the blocks' own fp16 scales; no minimum, no offset
    constexpr int BLK = TYPE == kQ8_0 ? 34 : 18;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      dsc[i] = load_half_as_float(blk_row + BLK * (4 * half + i));
      kk[i] = 0.f;
    }
  } else if constexpr (C::HAS_MIN) {
    const uint4 h = *reinterpret_cast<const uint4 *>(blk_row);
    const __half2 dd = *reinterpret_cast<const __half2 *>(&h.x);
    const float d = __low2float(dd), dmin = __high2float(dd);
    const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
    // four 6-bit scales / mins of this half as bytes (dequant.cr:240-249, four at a time)
    const uint32_t scw = half ? ((u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u)) : (u0 & 0x3f3f3f3fu);
    const uint32_t mnw = half ? (((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u)) : (u1 & 0x3f3f3f3fu);
    const float d23 = d * 8388608.f, ndmin = -dmin, ndmin23 = ndmin * 8388608.f;
    // Q4_K: the odd groups' integer sums arrive multiplied by 16 (see mma_block)
    const float dodd = TYPE == kQ4_K ? d * 0.0625f : d, dodd23 = dodd * 8388608.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
      dsc[i] = (i & 1) ? byte_times(scw, i, dodd, dodd23) : byte_times(scw, i, d, d23);
      kk[i] = byte_times(mnw, i, ndmin, ndmin23);
    }
  } else {
    const float d = load_half_as_float(blk_row + 208);
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk_row + 192 + 8 * half);
#pragma unroll
    for (int i = 0; i < 8; i++) {
      dsc[i] = d * (float)sc[i];
      kk[i] = dsc[i];  // times -32 once, at the end
    }
  }
}

template <int TYPE, int NB>
__device__ __forceinline__ void decode_scales_half(const uint8_t *blk_row, int lane, int kblk,
                                              const float *SX, const float *XX, float *area) {
  using C = Cfg<TYPE>;
  using A = Area<TYPE>;
  constexpr int NH = C::NG / 2;  // groups per lane
  const int r = lane & 15, half = lane >> 4;
  float dsc[NH], kk[NH];
  half_scales<TYPE>(blk_row, half, dsc, kk);
  // this lane's groups are consecutive in the tables: NH * NB floats each, 16-byte aligned
  const int grp0 = kblk * C::NG + NH * half;
  float sxv[NH * NB], xxv[NH * NB];
#pragma unroll
  for (int i = 0; i < NH * NB / 4; i++) {
    const float4 a = reinterpret_cast<const float4 *>(SX + grp0 * NB)[i];
    const float4 c = reinterpret_cast<const float4 *>(XX + grp0 * NB)[i];
    sxv[4 * i] = a.x; sxv[4 * i + 1] = a.y; sxv[4 * i + 2] = a.z; sxv[4 * i + 3] = a.w;
    xxv[4 * i] = c.x; xxv[4 * i + 1] = c.y; xxv[4 * i + 2] = c.z; xxv[4 * i + 3] = c.w;
  }
#pragma unroll
  for (int b = 0; b < NB; b++) {
    float *row = area + b * A::BATCH + r * A::ROW;
    float v[NH], corr = 0.f;
#pragma unroll
    for (int i = 0; i < NH; i++) {
      v[i] = dsc[i] * sxv[i * NB + b];
      corr = fmaf(kk[i], xxv[i * NB + b], corr);
    }
    if constexpr (C::NG == 8) {  // lane's groups 4*half + i: g4 = 2*half + (i >> 1), sub = i & 1
      *reinterpret_cast<float2 *>(row + 2 * half) = make_float2(v[0], v[2]);
      *reinterpret_cast<float2 *>(row + 4 + 2 * half) = make_float2(v[1], v[3]);
    } else {  // lane's groups 8*half + i: n = half, h = i & 1, sub = (i >> 1) & 1, m = i >> 2
      *reinterpret_cast<float4 *>(row + 4 * half) = make_float4(v[0], v[4], v[1], v[5]);
      *reinterpret_cast<float4 *>(row + 8 + 4 * half) = make_float4(v[2], v[6], v[3], v[7]);
    }
    corr += __shfl_xor_sync(0xffffffffu, corr, 16);
    if (half == 0) row[C::NG] = TYPE == kQ6_K ? -32.f * corr : corr;
  }
}

// Q6_K part of mma_block: aa / ab8 are the addresses of this lane's first ql bytes in rows g and
// g+8 (4 * t into the superblock).
template <int UNIT_BYTES, bool ALIGNED>
__device__ __forceinline__ void mma_q6(uintptr_t aa, uintptr_t ab8, const uint8_t *xu,
                                       const float *rowa, const float *rowb, int sub, float &acc0,
                                       float &acc1) {
  constexpr uint32_t M4 = 0x0f0f0f0fu, M2 = 0x30303030u;
  const uint8_t *base[2] = {reinterpret_cast<const uint8_t *>(aa & ~(uintptr_t)3),
                            reinterpret_cast<const uint8_t *>(ab8 & ~(uintptr_t)3)};
  const uint32_t sh[2] = {(uint32_t)(aa & 2) * 8, (uint32_t)(ab8 & 2) * 8};
#pragma unroll
  for (int n = 0; n < 2; n++) {
    const float4 sa4 = *reinterpret_cast<const float4 *>(rowa + 8 * sub + 4 * n);
    const float4 sb4 = *reinterpret_cast<const float4 *>(rowb + 8 * sub + 4 * n);
    const float sa[4] = {sa4.x, sa4.y, sa4.z, sa4.w}, sb[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
#pragma unroll
    for (int h = 0; h < 2; h++) {
      const uint4 bv = *reinterpret_cast<const uint4 *>(xu + (2 * n + h) * UNIT_BYTES);
      uint32_t q[2][4];
#pragma unroll
      for (int r = 0; r < 2; r++) {
        auto ld = [&](int off) {
          const uint32_t *w32 = reinterpret_cast<const uint32_t *>(base[r] + off);
          if constexpr (ALIGNED) return w32[0];
          else return __funnelshift_r(w32[0], w32[1], sh[r]);
        };
        const uint32_t ql0 = ld(64 * n + 16 * h), ql1 = ld(64 * n + 32 + 16 * h);
        const uint32_t qhw = ld(128 + 32 * n + 16 * h);
        q[r][0] = (ql0 & M4) | ((qhw << 4) & M2);
        q[r][1] = (ql1 & M4) | ((qhw << 2) & M2);
        q[r][2] = ((ql0 >> 4) & M4) | (qhw & M2);
        q[r][3] = ((ql1 >> 4) & M4) | ((qhw >> 2) & M2);
      }
#pragma unroll
      for (int m = 0; m < 2; m++) {
        int cc[4];
        // k-slots 0..15: run k = 2m, 16..31: run k = 2m+1 (scale group 8n + h + 2k)
        imma_zero(cc, q[0][2 * m], q[1][2 * m], q[0][2 * m + 1], q[1][2 * m + 1],
                  m ? bv.z : bv.x, m ? bv.w : bv.y);
        acc0 = fmaf(sa[2 * h + m], (float)(cc[0] * 128 + cc[1]), acc0);
        acc1 = fmaf(sb[2 * h + m], (float)(cc[2] * 128 + cc[3]), acc1);
      }
    }
  }
}

// MMAs of one superblock (16 rows x 256 columns) for this lane's (group slot sub, batch row).
// blk: the superblock of row 0 of the tile inside the stage; xu: this lane's B fragments of the
// superblock's first unit; ab: this lane's batch row of the superblock's area.  Adds the partial
// sums of rows g and g+8 (the correction included in the sub == 0 lanes) to acc0 / acc1.
template <int TYPE, int UNIT_BYTES>
__device__ __forceinline__ void mma_block(const uint8_t *blk, int pad_a, int pad_b,
                                          const uint8_t *xu, const float *ab, int g, int t,
                                          int sub, float &acc0, float &acc1) {
  using C = Cfg<TYPE>;
  using A = Area<TYPE>;
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const float *rowa = ab + g * A::ROW, *rowb = ab + (g + 8) * A::ROW;
  if (sub == 0) {
    acc0 += rowa[C::NG];
    acc1 += rowb[C::NG];
  }
  if constexpr (TYPE == kQ8_0) {
    // ra / rb are 8-byte aligned (superblocks and the stage's rows are 16-byte aligned).  The quants
    // of block j start at 34*j + 2: 2 bytes past a word for even j (three words and two funnel
    // shifts give this lane's 8 bytes), on a word for odd j.
    const uint8_t *ra = blk + g * C::RS + 8 * t, *rb = blk + (g + 8) * C::RS + 8 * t;
    const float4 sa4 = *reinterpret_cast<const float4 *>(rowa + 4 * sub);
    const float4 sb4 = *reinterpret_cast<const float4 *>(rowb + 4 * sub);
    const float sa[4] = {sa4.x, sa4.y, sa4.z, sa4.w}, sb[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
    auto even_block = [](const uint8_t *p, uint32_t &w0, uint32_t &w1) {  // p: the block's d
      const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
      const uint32_t a = q[0], b = q[1], c = q[2];
      w0 = __funnelshift_r(a, b, 16);
      w1 = __funnelshift_r(b, c, 16);
    };
    auto odd_block = [](const uint8_t *p, uint32_t &w0, uint32_t &w1) {  // p: the block's quants
      const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
      w0 = q[0];
      w1 = q[1];
    };
#pragma unroll
    for (int g4 = 0; g4 < 4; g4++) {
      const uint4 bv = *reinterpret_cast<const uint4 *>(xu + g4 * UNIT_BYTES);
      uint32_t la0, la1, ha0, ha1, lb0, lb1, hb0, hb1;
      even_block(ra + 68 * g4, la0, la1);
      odd_block(ra + 68 * g4 + 36, ha0, ha1);
      even_block(rb + 68 * g4, lb0, lb1);
      odd_block(rb + 68 * g4 + 36, hb0, hb1);
      int cc[4];
      // k-slots 0..15: block 2*g4, 16..31: block 2*g4+1
      imma_s8_zero(cc, la0, lb0, ha0, hb0, bv.x, bv.y);
      imma_s8_acc(cc, la1, lb1, ha1, hb1, bv.z, bv.w);
      acc0 = fmaf(sa[g4], (float)(cc[0] * 128 + cc[1]), acc0);
      acc1 = fmaf(sb[g4], (float)(cc[2] * 128 + cc[3]), acc1);
    }
  } else if constexpr (C::HAS_MIN) {
    constexpr bool Q5 = TYPE == kQ5_K;
    constexpr int QOFF = Q5 ? 48 : 16;
    constexpr uint32_t M1 = 0x10101010u;
    const uint8_t *ra = blk + g * C::RS + pad_a + 8 * t, *rb = blk + (g + 8) * C::RS + pad_b + 8 * t;
    const float4 sa4 = *reinterpret_cast<const float4 *>(rowa + 4 * sub);
    const float4 sb4 = *reinterpret_cast<const float4 *>(rowb + 4 * sub);
    const float sa[4] = {sa4.x, sa4.y, sa4.z, sa4.w}, sb[4] = {sb4.x, sb4.y, sb4.z, sb4.w};
    uint2 qha = make_uint2(0, 0), qhb = make_uint2(0, 0);
    if constexpr (Q5) {
      qha = *reinterpret_cast<const uint2 *>(ra + 16);
      qhb = *reinterpret_cast<const uint2 *>(rb + 16);
    }
#pragma unroll
    for (int g4 = 0; g4 < 4; g4++) {
      const uint4 bv = *reinterpret_cast<const uint4 *>(xu + g4 * UNIT_BYTES);
      const uint2 qa = *reinterpret_cast<const uint2 *>(ra + QOFF + 32 * g4);
      const uint2 qb = *reinterpret_cast<const uint2 *>(rb + QOFF + 32 * g4);
      int cc[4];
      if constexpr (!Q5) {
        constexpr uint32_t MH = 0xf0f0f0f0u;
        imma_zero(cc, qa.x, qb.x, qa.x & MH, qb.x & MH, bv.x, bv.y);
        imma_acc(cc, qa.y, qb.y, qa.y & MH, qb.y & MH, bv.z, bv.w);
      } else {
        uint32_t la0 = qa.x & M4, la1 = qa.y & M4, lb0 = qb.x & M4, lb1 = qb.y & M4;
        uint32_t ha0 = (qa.x >> 4) & M4, ha1 = (qa.y >> 4) & M4;
        uint32_t hb0 = (qb.x >> 4) & M4, hb1 = (qb.y >> 4) & M4;
        // fifth bit: bit 2*g4 of qh for the low-nibble elements, bit 2*g4+1 for the high ones
        auto bit = [&](uint32_t q, int b) { return b <= 4 ? ((q << (4 - b)) & M1) : ((q >> (b - 4)) & M1); };
        la0 |= bit(qha.x, 2 * g4);     la1 |= bit(qha.y, 2 * g4);
        lb0 |= bit(qhb.x, 2 * g4);     lb1 |= bit(qhb.y, 2 * g4);
        ha0 |= bit(qha.x, 2 * g4 + 1); ha1 |= bit(qha.y, 2 * g4 + 1);
        hb0 |= bit(qhb.x, 2 * g4 + 1); hb1 |= bit(qhb.y, 2 * g4 + 1);
        // k-slots 0..15: sub-block 2*g4 (low nibbles), 16..31: sub-block 2*g4+1 (high)
        imma_zero(cc, la0, lb0, ha0, hb0, bv.x, bv.y);
        imma_acc(cc, la1, lb1, ha1, hb1, bv.z, bv.w);
      }
      acc0 = fmaf(sa[g4], (float)(cc[0] * 128 + cc[1]), acc0);
      acc1 = fmaf(sb[g4], (float)(cc[2] * 128 + cc[3]), acc1);
    }
  } else {
    const uintptr_t aa = reinterpret_cast<uintptr_t>(blk + g * C::RS + pad_a + 4 * t);
    const uintptr_t ab8 = reinterpret_cast<uintptr_t>(blk + (g + 8) * C::RS + pad_b + 4 * t);
    // Superblocks are 210 bytes: every other one starts 2 bytes off a word boundary.  When the
    // whole warp reads word-aligned rows, one load per word does; otherwise two loads and a
    // funnel shift.
    if (__all_sync(0xffffffffu, ((aa | ab8) & 2) == 0))
      mma_q6<UNIT_BYTES, true>(aa, ab8, xu, rowa, rowb, sub, acc0, acc1);
    else
      mma_q6<UNIT_BYTES, false>(aa, ab8, xu, rowa, rowb, sub, acc0, acc1);
  }
}

// Quantises NBLK consecutive superblocks of x, starting at kblk (256 elements per batch row
// each), into the fragment-ordered layout: per scale group sx = max|x| / 16256,
// n = rint(x / sx) = 128*hi + lo with hi = n >> 7 in [-127, 127] and lo = n & 127.  One warp,
// lane = 8 consecutive elements.  The superblocks' areas are zeroed first: their unused words are
// the structural zeros of the layout.  All loads are issued before the first use.
template <int TYPE, int NB, int NBLK, bool LL>
__device__ __forceinline__ void quantise_superblocks(const float *x, const float *x_up,
                                                     const float *norm_w, const float *inv_rms,
                                                     int K, int kblk, int lane, uint8_t *xq,
                                                     float *SX, float *XX, const XSrc &src) {
  using C = Cfg<TYPE>;
  constexpr int NCX = 4 * NB, UNIT_BYTES = NCX * 64;
  constexpr int LPG = C::GROUP / 8;  // lanes per scale group
  uint8_t *base0 = xq + (size_t)kblk * 4 * UNIT_BYTES;
#pragma unroll
  for (int i = 0; i < NBLK * 4 * UNIT_BYTES / 512; i++)
    reinterpret_cast<uint4 *>(base0)[i * 32 + lane] = make_uint4(0, 0, 0, 0);
  const int e_in = lane * 8;
  float4 v0[NBLK][NB], v1[NBLK][NB];
#pragma unroll
  for (int q = 0; q < NBLK; q++)
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const long long off = (long long)b * K + (kblk + q) * 256 + e_in;
      v0[q][b] = ld4x<LL>(x, off, src);
      v1[q][b] = ld4x<LL>(x, off + 4, src);
      if (x_up) {  // SwiGLU: silu(gate) * up in f32, silu(v) = v / (1 + exp(-v)) (qwen35_cpu.cr:512-519, 1716-1717)
        const float4 u0 = ld4x<LL>(x_up, off, src);
        const float4 u1 = ld4x<LL>(x_up, off + 4, src);
        auto sw = [](float gte, float up) { return gte / (1.f + expf(-gte)) * up; };
        v0[q][b] = make_float4(sw(v0[q][b].x, u0.x), sw(v0[q][b].y, u0.y), sw(v0[q][b].z, u0.z), sw(v0[q][b].w, u0.w));
        v1[q][b] = make_float4(sw(v1[q][b].x, u1.x), sw(v1[q][b].y, u1.y), sw(v1[q][b].z, u1.z), sw(v1[q][b].w, u1.w));
      }
      if (norm_w) {  // RMSNorm: x * inv_rms * w in f32, left to right (qwen35_cpu.cr:484-490)
        const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + (kblk + q) * 256 + e_in));
        const float4 w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + (kblk + q) * 256 + e_in + 4));
        const float r = inv_rms[b];
        v0[q][b] = make_float4(v0[q][b].x * r * w0.x, v0[q][b].y * r * w0.y, v0[q][b].z * r * w0.z, v0[q][b].w * r * w0.w);
        v1[q][b] = make_float4(v1[q][b].x * r * w1.x, v1[q][b].y * r * w1.y, v1[q][b].z * r * w1.z, v1[q][b].w * r * w1.w);
      }
    }
  __syncwarp();
#pragma unroll
  for (int q = 0; q < NBLK; q++) {
    uint8_t *blk_base = base0 + q * 4 * UNIT_BYTES;
    const int k = (kblk + q) * 256 + e_in;
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const float v[8] = {v0[q][b].x, v0[q][b].y, v0[q][b].z, v0[q][b].w,
                          v1[q][b].x, v1[q][b].y, v1[q][b].z, v1[q][b].w};
      float mx = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) mx = fmaxf(mx, fabsf(v[e]));
#pragma unroll
      for (int off = 1; off < LPG; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      // groups below 1e-30 contribute nothing (their scale would underflow anyway)
      const bool live = mx > 1e-30f;
      const float sx = live ? mx * (1.f / kNMax) : 1.f;
      const float inv = live ? (float)kNMax / mx : 0.f;
      // round to nearest through the 1.5 * 2^23 bias (|x * inv| <= 16256 * (1 + 2^-21)): the low
      // bits of the sum are n in two's complement; bits 0-6 are lo, bits 7-14 the byte hi
      uint32_t bits[8], up[8];
      int nsum = 0;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        bits[e] = __float_as_uint(fmaf(v[e], inv, 12582912.f));
        up[e] = bits[e] << 1;
        nsum += (int)(bits[e] - 0x4B400000u);
      }
#pragma unroll
      for (int off = 1; off < LPG; off <<= 1) nsum += __shfl_xor_sync(0xffffffffu, nsum, off);
      if ((lane & (LPG - 1)) == 0) {
        const int grp = k / C::GROUP;
        SX[grp * NB + b] = sx;
        XX[grp * NB + b] = sx * (float)nsum;
      }
#pragma unroll
      for (int w4 = 0; w4 < 2; w4++) {  // the two 4-element words of this lane's 8 elements
        int sub;
        const int off = xq_word_offset<TYPE>(e_in + 4 * w4, NCX, 4 * b, sub);
        const uint32_t lw = __byte_perm(__byte_perm(bits[4 * w4], bits[4 * w4 + 1], 0x0040),
                                        __byte_perm(bits[4 * w4 + 2], bits[4 * w4 + 3], 0x0040),
                                        0x5410) & 0x7f7f7f7fu;
        const uint32_t hw = __byte_perm(__byte_perm(up[4 * w4], up[4 * w4 + 1], 0x0051),
                                        __byte_perm(up[4 * w4 + 2], up[4 * w4 + 3], 0x0051), 0x5410);
        *reinterpret_cast<uint32_t *>(blk_base + off) = hw;       // hi plane: column + 0
        *reinterpret_cast<uint32_t *>(blk_base + off + 64) = lw;  // lo plane: column + 1
        if (TYPE == kQ4_K && sub == 0) {  // the even group's second half: -x against H
          *reinterpret_cast<uint32_t *>(blk_base + off + 4) = __vneg4(hw);
          *reinterpret_cast<uint32_t *>(blk_base + off + 68) = __vneg4(lw);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------- batches 3 .. 8
// With more than two batch rows the MMA columns are (batch row b' of a set of four, plane):
// column 2b' + plane, one MMA per scale group and set (m16n8k32 for the 32-element groups,
// m16n8k16 for Q6_K's 16-element groups), no structural zeros.  Lane (g, t) of the result holds
// the hi and lo sums of batch row 4j + t for weight rows g and g+8 of set j.  The warp's area holds
// d*sc per (row, group) in group order, without the activation scale, which the lane multiplies in
// per (group, batch row); the row's corrections follow at index NG + b.
template <int TYPE> struct Dense {
  static constexpr int W = TYPE == kQ6_K ? 4 : 8;  // bytes of a lane's B fragment per (group, set)
  static constexpr int GB = 32 * W;                // bytes of a (group, set)
};
// floats per area row: NG scales + NB corrections, padded so that the 8 rows a warp reads with
// 16-byte loads fall into distinct banks
__host__ __device__ constexpr int dense_area_row(int ng, int nb) {
  return nb <= 4 ? ng + 4 : (ng == 8 ? 20 : 28);
}

// Quantises superblock kblk of x for NB batch rows (rows beyond `batch` repeat the last one) into
// the dense fragment order: byte offset ((group * J + set) * 32 + column * 4 + t) * W.
// SB: one scale per superblock and batch row (SX[kblk * NB + b]) and the groups' integer sums of n
// in XX, for the integer-domain loop of the K-quants; otherwise one scale per group.
template <int TYPE, int NB, bool LL, bool SB>
__device__ __forceinline__ void quantise_dense(const float *x, const float *x_up,
                                               const float *norm_w, const float *inv_rms, int K,
                                               int batch, int kblk, int lane, uint8_t *xq,
                                               float *SX, float *XX, const XSrc &src) {
  using C = Cfg<TYPE>;
  constexpr int J = NB / 4, W = Dense<TYPE>::W;
  constexpr int LPG = C::GROUP / 8;  // lanes per scale group
  const int k = kblk * 256 + lane * 8;
  const int grp = k / C::GROUP;
  // this lane's 8 bytes inside a column's 4 * W: lanes t of the MMA take W bytes each
  const int tpos = (lane & (LPG - 1)) * 8;
  float4 w0 = make_float4(1.f, 1.f, 1.f, 1.f), w1 = w0;
  if (norm_w) {
    w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + k));
    w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + k + 4));
  }
#pragma unroll
  for (int b4 = 0; b4 < NB; b4 += 4) {
    float4 v0[4], v1[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int br = min(b4 + i, batch - 1);
      const long long off = (long long)br * K + k;
      v0[i] = ld4x<LL>(x, off, src);
      v1[i] = ld4x<LL>(x, off + 4, src);
      if (x_up) {  // SwiGLU: silu(gate) * up in f32, silu(v) = v / (1 + exp(-v)) (qwen35_cpu.cr:512-519, 1716-1717)
        const float4 u0 = ld4x<LL>(x_up, off, src);
        const float4 u1 = ld4x<LL>(x_up, off + 4, src);
        auto sw = [](float gte, float up) { return gte / (1.f + expf(-gte)) * up; };
        v0[i] = make_float4(sw(v0[i].x, u0.x), sw(v0[i].y, u0.y), sw(v0[i].z, u0.z), sw(v0[i].w, u0.w));
        v1[i] = make_float4(sw(v1[i].x, u1.x), sw(v1[i].y, u1.y), sw(v1[i].z, u1.z), sw(v1[i].w, u1.w));
      }
      if (norm_w) {  // RMSNorm: x * inv_rms * w in f32, left to right (qwen35_cpu.cr:484-490)
        const float r = inv_rms[br];
        v0[i] = make_float4(v0[i].x * r * w0.x, v0[i].y * r * w0.y, v0[i].z * r * w0.z, v0[i].w * r * w0.w);
        v1[i] = make_float4(v1[i].x * r * w1.x, v1[i].y * r * w1.y, v1[i].z * r * w1.z, v1[i].w * r * w1.w);
      }
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
      const int b = b4 + i;
      const float v[8] = {v0[i].x, v0[i].y, v0[i].z, v0[i].w, v1[i].x, v1[i].y, v1[i].z, v1[i].w};
      float mx = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) mx = fmaxf(mx, fabsf(v[e]));
#pragma unroll
      for (int off = 1; off < (SB ? 32 : LPG); off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const bool live = mx > 1e-30f;  // as in quantise_superblocks
      const float sx = live ? mx * (1.f / kNMax) : 1.f;
      const float inv = live ? (float)kNMax / mx : 0.f;
      uint32_t bits[8], up[8];
      int nsum = 0;
#pragma unroll
      for (int e = 0; e < 8; e++) {
        bits[e] = __float_as_uint(fmaf(v[e], inv, 12582912.f));
        up[e] = bits[e] << 1;
        nsum += (int)(bits[e] - 0x4B400000u);
      }
#pragma unroll
      for (int off = 1; off < LPG; off <<= 1) nsum += __shfl_xor_sync(0xffffffffu, nsum, off);
      if constexpr (SB) {
        if (lane == 0) SX[kblk * NB + b] = sx;
        if ((lane & (LPG - 1)) == 0) reinterpret_cast<int *>(XX)[grp * NB + b] = nsum;
      } else if ((lane & (LPG - 1)) == 0) {
        SX[grp * NB + b] = sx;
        XX[grp * NB + b] = sx * (float)nsum;
      }
      uint32_t lw[2], hw[2];
#pragma unroll
      for (int w4 = 0; w4 < 2; w4++) {
        lw[w4] = __byte_perm(__byte_perm(bits[4 * w4], bits[4 * w4 + 1], 0x0040),
                             __byte_perm(bits[4 * w4 + 2], bits[4 * w4 + 3], 0x0040), 0x5410) & 0x7f7f7f7fu;
        hw[w4] = __byte_perm(__byte_perm(up[4 * w4], up[4 * w4 + 1], 0x0051),
                             __byte_perm(up[4 * w4 + 2], up[4 * w4 + 3], 0x0051), 0x5410);
      }
      uint8_t *dst = xq + ((size_t)(grp * J + (b >> 2)) * 32 + 2 * (b & 3) * 4) * W + tpos;
      if constexpr (TYPE == kIQ4_NL) {
        // The A fragments come out of the nibble table in the order (element i, element 16 + i,
        // element i + 1, element 17 + i) per pair of weight bytes, so the activations are laid out
        // to match: element e of the block (byte be = e & 15 of its 16, nibble e >> 4) goes to
        // MMA lane t = be >> 2, word m = (be >> 1) & 1, byte 2 * (be & 1) + (e >> 4).
        const int c = lane & 3;  // this lane holds elements 8c .. 8c + 7
        uint8_t *col = dst - tpos;
#pragma unroll
        for (int i = 0; i < 8; i++) {
          const int off = (2 * (c & 1) + (i >> 2)) * 8 + ((i >> 1) & 1) * 4 + 2 * (i & 1) + (c >> 1);
          col[off] = (uint8_t)(hw[i >> 2] >> (8 * (i & 3)));
          col[off + 4 * W] = (uint8_t)(lw[i >> 2] >> (8 * (i & 3)));
        }
      } else {
        *reinterpret_cast<uint2 *>(dst) = make_uint2(hw[0], hw[1]);          // hi plane: column 2b'
        *reinterpret_cast<uint2 *>(dst + 4 * W) = make_uint2(lw[0], lw[1]);  // lo plane: column 2b' + 1
      }
    }
  }
}

// Lanes (r = lane & 15, half = lane >> 4) decode one half of the scale groups of row r into the
// warp's area; the corrections of the NB batch rows are combined across the halves by shuffles.
template <int TYPE, int NB>
__device__ __forceinline__ void decode_dense(const uint8_t *blk_row, int lane, int kblk,
                                             const float *XX, float *area) {
  using C = Cfg<TYPE>;
  constexpr int NH = C::NG / 2, ROW = dense_area_row(C::NG, NB);
  const int r = lane & 15, half = lane >> 4;
  float dsc[NH], kk[NH];
  half_scales<TYPE>(blk_row, half, dsc, kk);
  float *row = area + r * ROW;
#pragma unroll
  for (int i = 0; i < NH; i += 4)
    *reinterpret_cast<float4 *>(row + NH * half + i) = make_float4(dsc[i], dsc[i + 1], dsc[i + 2], dsc[i + 3]);
  if constexpr (C::HAS_MIN || TYPE == kQ6_K) {
    float corr[NB];
#pragma unroll
    for (int b = 0; b < NB; b++) corr[b] = 0.f;
    const float4 *xx = reinterpret_cast<const float4 *>(XX + (size_t)(kblk * C::NG + NH * half) * NB);
#pragma unroll
    for (int i = 0; i < NH; i++)
#pragma unroll
      for (int b4 = 0; b4 < NB / 4; b4++) {
        const float4 c = xx[i * (NB / 4) + b4];
        corr[4 * b4] = fmaf(kk[i], c.x, corr[4 * b4]);
        corr[4 * b4 + 1] = fmaf(kk[i], c.y, corr[4 * b4 + 1]);
        corr[4 * b4 + 2] = fmaf(kk[i], c.z, corr[4 * b4 + 2]);
        corr[4 * b4 + 3] = fmaf(kk[i], c.w, corr[4 * b4 + 3]);
      }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      corr[b] += __shfl_xor_sync(0xffffffffu, corr[b], 16);
      if (TYPE == kQ6_K) corr[b] *= -32.f;
    }
    // the halves store alternate fours of the batch rows
#pragma unroll
    for (int b4 = 0; b4 < NB / 4; b4++)
      if (half == (b4 & 1))
        *reinterpret_cast<float4 *>(row + C::NG + 4 * b4) =
            make_float4(corr[4 * b4], corr[4 * b4 + 1], corr[4 * b4 + 2], corr[4 * b4 + 3]);
  } else {
#pragma unroll
    for (int b4 = 0; b4 < NB / 4; b4++)
      if (half == (b4 & 1))
        *reinterpret_cast<float4 *>(row + C::NG + 4 * b4) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// MMAs of one superblock for all NB batch rows.  xg: this lane's B fragment of the superblock's
// first (group, set); sxg: SX of the superblock's first group at batch row t.
template <int TYPE, int NB>
__device__ __forceinline__ void mma_dense(const uint8_t *blk, int pad_a, int pad_b,
                                          const uint8_t *xg, const float *area, const float *sxg,
                                          int g, int t, float (&acc0)[NB / 4], float (&acc1)[NB / 4]) {
  using C = Cfg<TYPE>;
  constexpr int J = NB / 4, GB = Dense<TYPE>::GB, ROW = dense_area_row(C::NG, NB);
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const float *rowa = area + g * ROW, *rowb = area + (g + 8) * ROW;
#pragma unroll
  for (int j = 0; j < J; j++) {
    acc0[j] = rowa[C::NG + 4 * j + t];
    acc1[j] = rowb[C::NG + 4 * j + t];
  }
  // scale group gi with A fragments (a0, a1, a2, a3): rows g / g+8, first / second eight elements
  auto group32 = [&](int gi, float fa, float fb, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
#pragma unroll
    for (int j = 0; j < J; j++) {
      const uint2 bv = *reinterpret_cast<const uint2 *>(xg + (gi * J + j) * GB);
      int cc[4];
      if constexpr (TYPE == kQ8_0 || TYPE == kIQ4_NL) imma_s8_zero(cc, a0, a1, a2, a3, bv.x, bv.y);
      else imma_zero(cc, a0, a1, a2, a3, bv.x, bv.y);
      const float sx = sxg[gi * NB + 4 * j];
      acc0[j] = fmaf(fa * sx, (float)(cc[0] * 128 + cc[1]), acc0[j]);
      acc1[j] = fmaf(fb * sx, (float)(cc[2] * 128 + cc[3]), acc1[j]);
    }
  };
  if constexpr (TYPE == kIQ4_NL) {
    // this lane's four nibble-pair bytes 4t .. 4t+3 of every block, rows g and g+8; the quants of
    // block j start 18j + 2 bytes into the superblock: on a word for odd j, 2 bytes off for even j
    const uint8_t *ra = blk + g * C::RS + 4 * t, *rb = blk + (g + 8) * C::RS + 4 * t;
    auto lut4 = [](uint32_t h) {  // nibbles 0 .. 3 of h -> the four table values as bytes
      const uint32_t s7 = h & 0x7777u;
      const uint32_t lo = __byte_perm(0xBFAD9881u, 0xF6EADDCFu, s7);   // entries 0 .. 7
      const uint32_t hi = __byte_perm(0x26190D01u, 0x71594535u, s7);   // entries 8 .. 15
      return __byte_perm(lo, hi, 0x3210u | ((h >> 1) & 0x4444u));
    };
#pragma unroll 1  // rolled: the unrolled body of eight groups x two sets overflowed the instruction cache
    for (int g4 = 0; g4 < 4; g4++) {
      const float2 sa = *reinterpret_cast<const float2 *>(rowa + 2 * g4);
      const float2 sb = *reinterpret_cast<const float2 *>(rowb + 2 * g4);
      const uint32_t *ea = reinterpret_cast<const uint32_t *>(ra + 36 * g4);
      const uint32_t *eb = reinterpret_cast<const uint32_t *>(rb + 36 * g4);
      const uint32_t wa0 = __funnelshift_r(ea[0], ea[1], 16), wb0 = __funnelshift_r(eb[0], eb[1], 16);
      const uint32_t wa1 = ea[5], wb1 = eb[5];  // block 2*g4 + 1: 36*g4 + 18 + 2
      group32(2 * g4, sa.x, sb.x, lut4(wa0), lut4(wb0), lut4(wa0 >> 16), lut4(wb0 >> 16));
      group32(2 * g4 + 1, sa.y, sb.y, lut4(wa1), lut4(wb1), lut4(wa1 >> 16), lut4(wb1 >> 16));
    }
  } else if constexpr (TYPE == kQ8_0) {
    const uint8_t *ra = blk + g * C::RS + 8 * t, *rb = blk + (g + 8) * C::RS + 8 * t;
    auto even_block = [](const uint8_t *p, uint32_t &w0, uint32_t &w1) {  // p: the block's d
      const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
      const uint32_t a = q[0], b = q[1], c = q[2];
      w0 = __funnelshift_r(a, b, 16);
      w1 = __funnelshift_r(b, c, 16);
    };
#pragma unroll 1  // rolled: the unrolled body of eight groups x two sets overflowed the instruction cache
    for (int g4 = 0; g4 < 4; g4++) {
      const float2 sa = *reinterpret_cast<const float2 *>(rowa + 2 * g4);
      const float2 sb = *reinterpret_cast<const float2 *>(rowb + 2 * g4);
      uint32_t la0, la1, lb0, lb1;
      even_block(ra + 68 * g4, la0, la1);
      even_block(rb + 68 * g4, lb0, lb1);
      // the odd block's quants sit on a word, not on a double word
      const uint32_t *ha = reinterpret_cast<const uint32_t *>(ra + 68 * g4 + 36);
      const uint32_t *hb = reinterpret_cast<const uint32_t *>(rb + 68 * g4 + 36);
      group32(2 * g4, sa.x, sb.x, la0, lb0, la1, lb1);
      group32(2 * g4 + 1, sa.y, sb.y, ha[0], hb[0], ha[1], hb[1]);
    }
  } else if constexpr (C::HAS_MIN) {
    constexpr bool Q5 = TYPE == kQ5_K;
    constexpr int QOFF = Q5 ? 48 : 16;
    constexpr uint32_t M1 = 0x10101010u, MH = 0xf0f0f0f0u;
    const uint8_t *ra = blk + g * C::RS + pad_a + 8 * t, *rb = blk + (g + 8) * C::RS + pad_b + 8 * t;
    uint2 qha = make_uint2(0, 0), qhb = make_uint2(0, 0);
    if constexpr (Q5) {
      qha = *reinterpret_cast<const uint2 *>(ra + 16);
      qhb = *reinterpret_cast<const uint2 *>(rb + 16);
    }
#pragma unroll 1  // rolled: the unrolled body of eight groups x two sets overflowed the instruction cache
    for (int g4 = 0; g4 < 4; g4++) {
      const float2 sa = *reinterpret_cast<const float2 *>(rowa + 2 * g4);
      const float2 sb = *reinterpret_cast<const float2 *>(rowb + 2 * g4);
      const uint2 qa = *reinterpret_cast<const uint2 *>(ra + QOFF + 32 * g4);
      const uint2 qb = *reinterpret_cast<const uint2 *>(rb + QOFF + 32 * g4);
      uint32_t la0 = qa.x & M4, la1 = qa.y & M4, lb0 = qb.x & M4, lb1 = qb.y & M4;
      uint32_t ha0, ha1, hb0, hb1;
      if constexpr (!Q5) {  // high nibbles stay in place: 16 * q, the 1/16 is in the group's scale
        ha0 = qa.x & MH; ha1 = qa.y & MH; hb0 = qb.x & MH; hb1 = qb.y & MH;
      } else {
        ha0 = (qa.x >> 4) & M4; ha1 = (qa.y >> 4) & M4; hb0 = (qb.x >> 4) & M4; hb1 = (qb.y >> 4) & M4;
        // fifth bit: bit 2*g4 of qh for the low-nibble elements, bit 2*g4+1 for the high ones
        auto bit = [&](uint32_t q, int b) { return b <= 4 ? ((q << (4 - b)) & M1) : ((q >> (b - 4)) & M1); };
        la0 |= bit(qha.x, 2 * g4);     la1 |= bit(qha.y, 2 * g4);
        lb0 |= bit(qhb.x, 2 * g4);     lb1 |= bit(qhb.y, 2 * g4);
        ha0 |= bit(qha.x, 2 * g4 + 1); ha1 |= bit(qha.y, 2 * g4 + 1);
        hb0 |= bit(qhb.x, 2 * g4 + 1); hb1 |= bit(qhb.y, 2 * g4 + 1);
      }
      group32(2 * g4, sa.x, sb.x, la0, lb0, la1, lb1);
      group32(2 * g4 + 1, sa.y, sb.y, ha0, hb0, ha1, hb1);
    }
  } else {
    constexpr uint32_t M2 = 0x30303030u;
    const uintptr_t aa = reinterpret_cast<uintptr_t>(blk + g * C::RS + pad_a + 4 * t);
    const uintptr_t ab8 = reinterpret_cast<uintptr_t>(blk + (g + 8) * C::RS + pad_b + 4 * t);
    const uint8_t *base[2] = {reinterpret_cast<const uint8_t *>(aa & ~(uintptr_t)3),
                              reinterpret_cast<const uint8_t *>(ab8 & ~(uintptr_t)3)};
    const uint32_t sh[2] = {(uint32_t)(aa & 2) * 8, (uint32_t)(ab8 & 2) * 8};
#pragma unroll
    for (int n = 0; n < 2; n++) {
      const float4 sa0 = *reinterpret_cast<const float4 *>(rowa + 8 * n), sa1 = *reinterpret_cast<const float4 *>(rowa + 8 * n + 4);
      const float4 sb0 = *reinterpret_cast<const float4 *>(rowb + 8 * n), sb1 = *reinterpret_cast<const float4 *>(rowb + 8 * n + 4);
      const float sa[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
      const float sb[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint32_t q[2][4];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          auto ld = [&](int off) {  // rows may start 2 bytes off a word: two loads and a funnel shift
            const uint32_t *w32 = reinterpret_cast<const uint32_t *>(base[r] + off);
            return __funnelshift_r(w32[0], w32[1], sh[r]);
          };
          const uint32_t ql0 = ld(64 * n + 16 * h), ql1 = ld(64 * n + 32 + 16 * h);
          const uint32_t qhw = ld(128 + 32 * n + 16 * h);
          q[r][0] = (ql0 & M4) | ((qhw << 4) & M2);
          q[r][1] = (ql1 & M4) | ((qhw << 2) & M2);
          q[r][2] = ((ql0 >> 4) & M4) | (qhw & M2);
          q[r][3] = ((ql1 >> 4) & M4) | ((qhw >> 2) & M2);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {  // elements 128n + 32k + 16h + (0..15): scale group 8n + 2k + h
          const int gi = 8 * n + 2 * k + h;
          const float fa = sa[2 * k + h], fb = sb[2 * k + h];
#pragma unroll
          for (int j = 0; j < J; j++) {
            const uint32_t bw = *reinterpret_cast<const uint32_t *>(xg + (gi * J + j) * GB);
            int cc[4];
            imma16_zero(cc, q[0][k], q[1][k], bw);
            const float sx = sxg[gi * NB + 4 * j];
            acc0[j] = fmaf(fa * sx, (float)(cc[0] * 128 + cc[1]), acc0[j]);
            acc1[j] = fmaf(fb * sx, (float)(cc[2] * 128 + cc[3]), acc1[j]);
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------- batches 3 .. 8, K-quants
// Q4_K, Q5_K and Q6_K keep a superblock in the integer domain, like Q6_K at batch 1-2: one
// activation scale per superblock and batch row, the weights' 6-bit (int8) group scales multiplied
// onto the integer group sums, one conversion per (row, batch row) and superblock.  Per (group, set
// of four batch rows) a lane issues one B-fragment load, one MMA and four integer multiply-adds
// (rows g / g+8 x planes hi / lo).  The planes stay apart until the conversion (hi * 128 + lo in
// float), which keeps the sums in range: per group |sum| <= 32 * 240 * 127 (Q4_K's high nibbles in
// place), times a scale <= 63 (the low-nibble groups' scales come times 16 instead), eight groups:
// below 5e8; Q5_K 32 * 31 * 127 * 63 * 8 < 7e7; Q6_K 16 * 63 * 127 * 128 * 16 < 2.7e8.  The
// offsets (-dmin * m, -32) are integer sums of (min or scale) x (group sum of n), below 5.4e8.
template <int TYPE> constexpr bool kDenseInt = TYPE == kQ4_K || TYPE == kQ5_K || TYPE == kQ6_K;

// Lanes (r = lane & 15, half = lane >> 4) write the integer scales of one half of row r's groups
// into the warp's area; the offsets of the NB batch rows follow at index NG + b as floats.
template <int TYPE, int NB>
__device__ __forceinline__ void decode_dense_int(const uint8_t *blk_row, int lane, int kblk,
                                                 const float *SX, const int *XN, float *area) {
  using C = Cfg<TYPE>;
  constexpr int NH = C::NG / 2, ROW = dense_area_row(C::NG, NB);
  const int r = lane & 15, half = lane >> 4;
  int sc[NH], mn[NH];
  float dneg;  // the factor of the offset sum: -dmin, or -32 d
  if constexpr (C::HAS_MIN) {
    const uint4 h = *reinterpret_cast<const uint4 *>(blk_row);
    dneg = -__high2float(*reinterpret_cast<const __half2 *>(&h.x));
    const uint32_t u0 = h.y, u1 = h.z, u2 = h.w;
    // four 6-bit scales / mins of this half as bytes (dequant.cr:240-249, four at a time)
    const uint32_t scw = half ? ((u2 & 0x0f0f0f0fu) | ((u0 >> 2) & 0x30303030u)) : (u0 & 0x3f3f3f3fu);
    const uint32_t mnw = half ? (((u2 >> 4) & 0x0f0f0f0fu) | ((u1 >> 2) & 0x30303030u)) : (u1 & 0x3f3f3f3fu);
#pragma unroll
    for (int i = 0; i < 4; i++) {
      sc[i] = (int)((scw >> (8 * i)) & 0xffu);
      // Q4_K: the odd groups' sums arrive times 16 (nibbles in place), so the even ones' scales do
      if (TYPE == kQ4_K && !(i & 1)) sc[i] <<= 4;
      mn[i] = (int)((mnw >> (8 * i)) & 0xffu);
    }
  } else {
    dneg = -32.f * load_half_as_float(blk_row + 208);
    const int8_t *s8 = reinterpret_cast<const int8_t *>(blk_row + 192 + 8 * half);
#pragma unroll
    for (int i = 0; i < 8; i++) sc[i] = mn[i] = (int)s8[i];
  }
  int *row = reinterpret_cast<int *>(area + r * ROW);
#pragma unroll
  for (int i = 0; i < NH; i += 4)
    *reinterpret_cast<int4 *>(row + NH * half + i) = make_int4(sc[i], sc[i + 1], sc[i + 2], sc[i + 3]);
  int cs[NB];
#pragma unroll
  for (int b = 0; b < NB; b++) cs[b] = 0;
  const int4 *xn = reinterpret_cast<const int4 *>(XN + (size_t)(kblk * C::NG + NH * half) * NB);
#pragma unroll
  for (int i = 0; i < NH; i++)
#pragma unroll
    for (int b4 = 0; b4 < NB / 4; b4++) {
      const int4 c = xn[i * (NB / 4) + b4];
      cs[4 * b4] += mn[i] * c.x;
      cs[4 * b4 + 1] += mn[i] * c.y;
      cs[4 * b4 + 2] += mn[i] * c.z;
      cs[4 * b4 + 3] += mn[i] * c.w;
    }
#pragma unroll
  for (int b = 0; b < NB; b++) cs[b] += __shfl_xor_sync(0xffffffffu, cs[b], 16);
  // the halves store alternate fours of the batch rows
#pragma unroll
  for (int b4 = 0; b4 < NB / 4; b4++)
    if (half == (b4 & 1)) {
      const float4 sx = *reinterpret_cast<const float4 *>(SX + (size_t)kblk * NB + 4 * b4);
      *reinterpret_cast<float4 *>(area + r * ROW + C::NG + 4 * b4) =
          make_float4(dneg * sx.x * (float)cs[4 * b4], dneg * sx.y * (float)cs[4 * b4 + 1],
                      dneg * sx.z * (float)cs[4 * b4 + 2], dneg * sx.w * (float)cs[4 * b4 + 3]);
    }
}

// MMAs of one superblock for all NB batch rows.  xg: this lane's B fragment of the superblock's
// first (group, set); sxb: the superblock's activation scales (one per batch row).
template <int TYPE, int NB>
__device__ __forceinline__ void mma_dense_int(const uint8_t *blk, int pad_a, int pad_b,
                                              const uint8_t *xg, const float *area, const float *sxb,
                                              int g, int t, float (&acc0)[NB / 4], float (&acc1)[NB / 4]) {
  using C = Cfg<TYPE>;
  constexpr int J = NB / 4, GB = Dense<TYPE>::GB, ROW = dense_area_row(C::NG, NB);
  constexpr uint32_t M4 = 0x0f0f0f0fu;
  const int *rowa = reinterpret_cast<const int *>(area + g * ROW);
  const int *rowb = reinterpret_cast<const int *>(area + (g + 8) * ROW);
  int h0[J], l0[J], h1[J], l1[J];  // rows g / g+8, planes hi / lo, batch row 4j + t
#pragma unroll
  for (int j = 0; j < J; j++) h0[j] = l0[j] = h1[j] = l1[j] = 0;
  float da, db;
  if constexpr (C::HAS_MIN) {
    constexpr bool Q5 = TYPE == kQ5_K;
    constexpr int QOFF = Q5 ? 48 : 16;
    constexpr uint32_t M1 = 0x10101010u, MH = 0xf0f0f0f0u;
    const uint8_t *ra = blk + g * C::RS + pad_a, *rb = blk + (g + 8) * C::RS + pad_b;
    da = load_half_as_float(ra) * (Q5 ? 1.f : 0.0625f);
    db = load_half_as_float(rb) * (Q5 ? 1.f : 0.0625f);
    ra += 8 * t;
    rb += 8 * t;
    uint2 qha = make_uint2(0, 0), qhb = make_uint2(0, 0);
    if constexpr (Q5) {
      qha = *reinterpret_cast<const uint2 *>(ra + 16);
      qhb = *reinterpret_cast<const uint2 *>(rb + 16);
    }
    auto group32 = [&](int gi, int sa, int sb, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3) {
#pragma unroll
      for (int j = 0; j < J; j++) {
        const uint2 bv = *reinterpret_cast<const uint2 *>(xg + (gi * J + j) * GB);
        int cc[4];
        imma_zero(cc, a0, a1, a2, a3, bv.x, bv.y);
        h0[j] += sa * cc[0];
        l0[j] += sa * cc[1];
        h1[j] += sb * cc[2];
        l1[j] += sb * cc[3];
      }
    };
#pragma unroll 1  // unrolling by 2 or 4 measured the same
    for (int g4 = 0; g4 < 4; g4++) {
      const int2 sa = *reinterpret_cast<const int2 *>(rowa + 2 * g4);
      const int2 sb = *reinterpret_cast<const int2 *>(rowb + 2 * g4);
      const uint2 qa = *reinterpret_cast<const uint2 *>(ra + QOFF + 32 * g4);
      const uint2 qb = *reinterpret_cast<const uint2 *>(rb + QOFF + 32 * g4);
      uint32_t la0 = qa.x & M4, la1 = qa.y & M4, lb0 = qb.x & M4, lb1 = qb.y & M4;
      uint32_t ha0, ha1, hb0, hb1;
      if constexpr (!Q5) {  // high nibbles stay in place: 16 * q
        ha0 = qa.x & MH; ha1 = qa.y & MH; hb0 = qb.x & MH; hb1 = qb.y & MH;
      } else {
        ha0 = (qa.x >> 4) & M4; ha1 = (qa.y >> 4) & M4; hb0 = (qb.x >> 4) & M4; hb1 = (qb.y >> 4) & M4;
        // fifth bit: bit 2*g4 of qh for the low-nibble elements, bit 2*g4+1 for the high ones
        auto bit = [&](uint32_t q, int b) { return b <= 4 ? ((q << (4 - b)) & M1) : ((q >> (b - 4)) & M1); };
        la0 |= bit(qha.x, 2 * g4);     la1 |= bit(qha.y, 2 * g4);
        lb0 |= bit(qhb.x, 2 * g4);     lb1 |= bit(qhb.y, 2 * g4);
        ha0 |= bit(qha.x, 2 * g4 + 1); ha1 |= bit(qha.y, 2 * g4 + 1);
        hb0 |= bit(qhb.x, 2 * g4 + 1); hb1 |= bit(qhb.y, 2 * g4 + 1);
      }
      group32(2 * g4, sa.x, sb.x, la0, lb0, la1, lb1);
      group32(2 * g4 + 1, sa.y, sb.y, ha0, hb0, ha1, hb1);
    }
  } else {
    constexpr uint32_t M2 = 0x30303030u;
    da = load_half_as_float(blk + g * C::RS + pad_a + 208);
    db = load_half_as_float(blk + (g + 8) * C::RS + pad_b + 208);
    const uintptr_t aa = reinterpret_cast<uintptr_t>(blk + g * C::RS + pad_a + 4 * t);
    const uintptr_t ab8 = reinterpret_cast<uintptr_t>(blk + (g + 8) * C::RS + pad_b + 4 * t);
    const uint8_t *base[2] = {reinterpret_cast<const uint8_t *>(aa & ~(uintptr_t)3),
                              reinterpret_cast<const uint8_t *>(ab8 & ~(uintptr_t)3)};
    const uint32_t sh[2] = {(uint32_t)(aa & 2) * 8, (uint32_t)(ab8 & 2) * 8};
#pragma unroll
    for (int n = 0; n < 2; n++) {
      const int4 sa0 = *reinterpret_cast<const int4 *>(rowa + 8 * n), sa1 = *reinterpret_cast<const int4 *>(rowa + 8 * n + 4);
      const int4 sb0 = *reinterpret_cast<const int4 *>(rowb + 8 * n), sb1 = *reinterpret_cast<const int4 *>(rowb + 8 * n + 4);
      const int sa[8] = {sa0.x, sa0.y, sa0.z, sa0.w, sa1.x, sa1.y, sa1.z, sa1.w};
      const int sb[8] = {sb0.x, sb0.y, sb0.z, sb0.w, sb1.x, sb1.y, sb1.z, sb1.w};
#pragma unroll
      for (int h = 0; h < 2; h++) {
        uint32_t q[2][4];
#pragma unroll
        for (int r = 0; r < 2; r++) {
          auto ld = [&](int off) {  // rows may start 2 bytes off a word: two loads and a funnel shift
            const uint32_t *w32 = reinterpret_cast<const uint32_t *>(base[r] + off);
            return __funnelshift_r(w32[0], w32[1], sh[r]);
          };
          const uint32_t ql0 = ld(64 * n + 16 * h), ql1 = ld(64 * n + 32 + 16 * h);
          const uint32_t qhw = ld(128 + 32 * n + 16 * h);
          q[r][0] = (ql0 & M4) | ((qhw << 4) & M2);
          q[r][1] = (ql1 & M4) | ((qhw << 2) & M2);
          q[r][2] = ((ql0 >> 4) & M4) | (qhw & M2);
          q[r][3] = ((ql1 >> 4) & M4) | ((qhw >> 2) & M2);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {  // elements 128n + 32k + 16h + (0..15): scale group 8n + 2k + h
          const int gi = 8 * n + 2 * k + h;
#pragma unroll
          for (int j = 0; j < J; j++) {
            const uint32_t bw = *reinterpret_cast<const uint32_t *>(xg + (gi * J + j) * GB);
            int cc[4];
            imma16_zero(cc, q[0][k], q[1][k], bw);
            h0[j] += sa[2 * k + h] * cc[0];
            l0[j] += sa[2 * k + h] * cc[1];
            h1[j] += sb[2 * k + h] * cc[2];
            l1[j] += sb[2 * k + h] * cc[3];
          }
        }
      }
    }
  }
  const float *rowfa = area + g * ROW + C::NG, *rowfb = area + (g + 8) * ROW + C::NG;
#pragma unroll
  for (int j = 0; j < J; j++) {
    const float sx = sxb[4 * j + t];
    acc0[j] = fmaf(da * sx, fmaf((float)h0[j], 128.f, (float)l0[j]), rowfa[4 * j + t]);
    acc1[j] = fmaf(db * sx, fmaf((float)h1[j], 128.f, (float)l1[j]), rowfb[4 * j + t]);
  }
}

// ---------------------------------------------------------------------------- Q6_K, batch 1-2
// Q6_K at batch 1-2 keeps everything up to the end of a superblock in the integer domain.
//  * Activations: ONE scale per superblock and batch row (x = sxb * n, |n| <= 16256, n = 128*hi + lo
//    as above) instead of one per 16-element group, so the int8 group scales of the weights can be
//    applied to the integer group sums and a row converts to float once per superblock.
//  * The quants are never assembled.  ql bytes are split by two ANDs into L = b & 0x0F (elements
//    32k + l, k = 0 / 1) and H = b & 0xF0 (16 x elements 32k + l, k = 2 / 3); the qh byte by four
//    ANDs into its 2-bit fields in place (f0, 4*f1, 16*f2, 64*f3).  Per "unit" (half n of the
//    superblock, 16-element run h: 64 weights of 4 scale groups k = 0..3 per row) four MMAs
//        A = [L(ql run of k=0) | L(ql run of k=1)],  A = [H(k=2) | H(k=3)]   -> accumulator cq
//        A = [f0 | 4 f1],                            A = [16 f2 | 64 f3]     -> accumulator ch
//    whose eight columns are (group k, plane): column 2k + plane holds that group's activations in
//    the k-slots of its own run and zeros in the other run's.  Lane (g, t) thus receives the exact
//    sums of group k = t for rows g and g+8; 16 * sum(q * n) = mq * cq + mh * ch with
//    (mq, mh) = (16, 256), (16, 64), (1, 16), (1, 4) for k = 0..3.
//  * A lane keeps one activation word per unit (its column's 4 elements of its plane); the B
//    fragments are that word or zero, selected by the lane's k: 2 bytes of shared memory per
//    element and batch row.
//  * The -32 of every quant is one integer term per group from the sums of n.
// Integer ranges: |cq| <= 16 * 240 * 127, |ch| <= 16 * 192 * 127 per unit, times |sc| <= 128, four
// units per lane and superblock, times at most 16 resp. 256 at the end: below 1.1e9.
//
// Quantises NBLK superblocks of x from kblk on.  Lane = 8 consecutive elements:
// element 128 n + 32 k + 16 h + i  ->  unit u = 2 n + h, column 2 k + plane, MMA lane t = i / 4.
template <int NB, int NBLK, bool LL>
__device__ __forceinline__ void quantise_q6v2(const float *x, const float *x_up, const float *norm_w,
                                              const float *inv_rms, int K, int kblk, int lane,
                                              uint8_t *xq, float *SXB, int *NG, const XSrc &src) {
  const int e_in = lane * 8;
  float4 v0[NBLK][NB], v1[NBLK][NB];
#pragma unroll
  for (int q = 0; q < NBLK; q++)
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const long long off = (long long)b * K + (kblk + q) * 256 + e_in;
      v0[q][b] = ld4x<LL>(x, off, src);
      v1[q][b] = ld4x<LL>(x, off + 4, src);
      if (x_up) {  // SwiGLU: silu(gate) * up in f32 (qwen35_cpu.cr:512-519, 1716-1717)
        const float4 u0 = ld4x<LL>(x_up, off, src);
        const float4 u1 = ld4x<LL>(x_up, off + 4, src);
        auto sw = [](float gte, float up) { return gte / (1.f + expf(-gte)) * up; };
        v0[q][b] = make_float4(sw(v0[q][b].x, u0.x), sw(v0[q][b].y, u0.y), sw(v0[q][b].z, u0.z), sw(v0[q][b].w, u0.w));
        v1[q][b] = make_float4(sw(v1[q][b].x, u1.x), sw(v1[q][b].y, u1.y), sw(v1[q][b].z, u1.z), sw(v1[q][b].w, u1.w));
      }
      if (norm_w) {  // RMSNorm: x * inv_rms * w in f32, left to right (qwen35_cpu.cr:484-490)
        const float4 w0 = __ldg(reinterpret_cast<const float4 *>(norm_w + (kblk + q) * 256 + e_in));
        const float4 w1 = __ldg(reinterpret_cast<const float4 *>(norm_w + (kblk + q) * 256 + e_in + 4));
        const float r = inv_rms[b];
        v0[q][b] = make_float4(v0[q][b].x * r * w0.x, v0[q][b].y * r * w0.y, v0[q][b].z * r * w0.z, v0[q][b].w * r * w0.w);
        v1[q][b] = make_float4(v1[q][b].x * r * w1.x, v1[q][b].y * r * w1.y, v1[q][b].z * r * w1.z, v1[q][b].w * r * w1.w);
      }
    }
  const int n = lane >> 4, k = (lane >> 2) & 3, h = (lane >> 1) & 1;
  const int u = 2 * n + h, t0 = 2 * (lane & 1);
#pragma unroll
  for (int q = 0; q < NBLK; q++)
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const float v[8] = {v0[q][b].x, v0[q][b].y, v0[q][b].z, v0[q][b].w,
                          v1[q][b].x, v1[q][b].y, v1[q][b].z, v1[q][b].w};
      float mx = 0.f;
#pragma unroll
      for (int e = 0; e < 8; e++) mx = fmaxf(mx, fabsf(v[e]));
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      const bool live = mx > 1e-30f;  // a superblock below that contributes nothing
      const float sxb = live ? mx * (1.f / kNMax) : 1.f;
      const float inv = live ? (float)kNMax / mx : 0.f;
      uint32_t bits[8], up[8];
      int nsum = 0;
#pragma unroll
      for (int e = 0; e < 8; e++) {  // n in the low bits of x * inv + 1.5 * 2^23 (round to nearest)
        bits[e] = __float_as_uint(fmaf(v[e], inv, 12582912.f));
        up[e] = bits[e] << 1;
        nsum += (int)(bits[e] - 0x4B400000u);
      }
      nsum += __shfl_xor_sync(0xffffffffu, nsum, 1);  // the group's 16 elements: this lane and its neighbour
      const int sb = (kblk + q) * NB + b;
      if ((lane & 1) == 0) NG[(sb * 4 + k) * 4 + u] = nsum;
      if (lane == 0) SXB[sb] = sxb;
      uint32_t *dst = reinterpret_cast<uint32_t *>(xq) + (sb * 4 + u) * 32 + 8 * k + t0;
#pragma unroll
      for (int w4 = 0; w4 < 2; w4++) {
        const uint32_t lw = __byte_perm(__byte_perm(bits[4 * w4], bits[4 * w4 + 1], 0x0040),
                                        __byte_perm(bits[4 * w4 + 2], bits[4 * w4 + 3], 0x0040),
                                        0x5410) & 0x7f7f7f7fu;
        const uint32_t hw = __byte_perm(__byte_perm(up[4 * w4], up[4 * w4 + 1], 0x0051),
                                        __byte_perm(up[4 * w4 + 2], up[4 * w4 + 3], 0x0051), 0x5410);
        dst[w4] = hw;      // column 2k:     hi plane
        dst[4 + w4] = lw;  // column 2k + 1: lo plane
      }
    }
}

// One superblock of 16 rows against NB batch rows.  ra / rb: this superblock in rows g and g+8
// (2-byte aligned); xw: the lane's activation word of unit 0, batch row 0; ng: the lane's four
// group sums (units 0..3 of group k = t), batch row 0; sxb: the superblock's activation scales.
template <int NB, bool ALIGNED>
__device__ __forceinline__ void mma_q6v2(const uint8_t *ra, const uint8_t *rb, const uint32_t *xw,
                                         const int4 *ng, const float *sxb, int lane,
                                         float (&acc0)[NB], float (&acc1)[NB]) {
  constexpr uint32_t ML = 0x0f0f0f0fu, MH = 0xf0f0f0f0u;
  const int t = lane & 3, kcol = lane >> 3;
  const uintptr_t aa = reinterpret_cast<uintptr_t>(ra) + 4 * t, ab = reinterpret_cast<uintptr_t>(rb) + 4 * t;
  const uint8_t *base[2] = {reinterpret_cast<const uint8_t *>(aa & ~(uintptr_t)3),
                            reinterpret_cast<const uint8_t *>(ab & ~(uintptr_t)3)};
  const uint32_t sh[2] = {(uint32_t)(aa & 2) * 8, (uint32_t)(ab & 2) * 8};
  auto ld = [&](int r, int off) {
    const uint32_t *w32 = reinterpret_cast<const uint32_t *>(base[r] + off);
    if constexpr (ALIGNED) return w32[0];
    else return __funnelshift_r(w32[0], w32[1], sh[r]);
  };
  // the group scales of this lane's groups 8n + 2t + h, as (n, h) = unit order, rows g / g+8
  int sc[2][4];
#pragma unroll
  for (int r = 0; r < 2; r++) {
    const uint8_t *row = r ? rb : ra;
    const uint32_t s01 = *reinterpret_cast<const unsigned short *>(row + 192 + 2 * t);
    const uint32_t s23 = *reinterpret_cast<const unsigned short *>(row + 200 + 2 * t);
    sc[r][0] = (int)(signed char)(s01 & 0xffu);
    sc[r][1] = (int)(signed char)(s01 >> 8);
    sc[r][2] = (int)(signed char)(s23 & 0xffu);
    sc[r][3] = (int)(signed char)(s23 >> 8);
  }
  // B fragment selectors: the lane's word belongs to the k-slots of run k of its column's group
  const uint32_t m0 = kcol == 0 ? 0xffffffffu : 0u, m1 = kcol == 1 ? 0xffffffffu : 0u;
  const uint32_t m2 = kcol == 2 ? 0xffffffffu : 0u, m3 = kcol == 3 ? 0xffffffffu : 0u;
  int aq[NB][4], ah[NB][4], corr[NB][2];
#pragma unroll
  for (int b = 0; b < NB; b++) {
#pragma unroll
    for (int i = 0; i < 4; i++) aq[b][i] = ah[b][i] = 0;
    corr[b][0] = corr[b][1] = 0;
  }
  int4 ngv[NB];
#pragma unroll
  for (int b = 0; b < NB; b++) ngv[b] = ng[b * 4];
#pragma unroll
  for (int u = 0; u < 4; u++) {
    const int n = u >> 1, h = u & 1;
    uint32_t q0[2], q1[2], qh[2];
#pragma unroll
    for (int r = 0; r < 2; r++) {
      q0[r] = ld(r, 64 * n + 16 * h);
      q1[r] = ld(r, 64 * n + 32 + 16 * h);
      qh[r] = ld(r, 128 + 32 * n + 16 * h);
    }
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const uint32_t w = xw[(b * 4 + u) * 32];
      const uint32_t b0 = w & m0, b1 = w & m1, b2 = w & m2, b3 = w & m3;
      int cq[4], ch[4];
      imma_zero(cq, q0[0] & ML, q0[1] & ML, q1[0] & ML, q1[1] & ML, b0, b1);
      imma_acc(cq, q0[0] & MH, q0[1] & MH, q1[0] & MH, q1[1] & MH, b2, b3);
      imma_zero(ch, qh[0] & 0x03030303u, qh[1] & 0x03030303u, qh[0] & 0x0c0c0c0cu, qh[1] & 0x0c0c0c0cu, b0, b1);
      imma_acc(ch, qh[0] & 0x30303030u, qh[1] & 0x30303030u, qh[0] & 0xc0c0c0c0u, qh[1] & 0xc0c0c0c0u, b2, b3);
      const int ngu = u == 0 ? ngv[b].x : u == 1 ? ngv[b].y : u == 2 ? ngv[b].z : ngv[b].w;
      aq[b][0] += sc[0][u] * cq[0];  aq[b][1] += sc[0][u] * cq[1];
      aq[b][2] += sc[1][u] * cq[2];  aq[b][3] += sc[1][u] * cq[3];
      ah[b][0] += sc[0][u] * ch[0];  ah[b][1] += sc[0][u] * ch[1];
      ah[b][2] += sc[1][u] * ch[2];  ah[b][3] += sc[1][u] * ch[3];
      corr[b][0] += sc[0][u] * ngu;
      corr[b][1] += sc[1][u] * ngu;
    }
  }
  const int mq = t < 2 ? 16 : 1, mh = 256 >> (2 * t);
  const float da = load_half_as_float(ra + 208), db = load_half_as_float(rb + 208);
#pragma unroll
  for (int b = 0; b < NB; b++) {
    const float s16 = sxb[b] * 0.0625f;  // the integer sums are 16 x the true ones
    const float fa = fmaf(-512.f, (float)corr[b][0],
                          fmaf(128.f, (float)(mq * aq[b][0] + mh * ah[b][0]), (float)(mq * aq[b][1] + mh * ah[b][1])));
    const float fb = fmaf(-512.f, (float)corr[b][1],
                          fmaf(128.f, (float)(mq * aq[b][2] + mh * ah[b][2]), (float)(mq * aq[b][3] + mh * ah[b][3])));
    acc0[b] = fmaf(da * s16, fa, acc0[b]);
    acc1[b] = fmaf(db * s16, fb, acc1[b]);
  }
}

// ---------------------------------------------------------------------------- the kernel
// VAR picks how much the instance carries: 0 the plain GEMV; 1 adds the fused prologues (RMSNorm,
// SwiGLU) to the activation quantisers; 2 also splits row tiles over K slabs, exchanges its outputs
// with the other GPUs and reads activations that come out of an exchange; 3 is the plain GEMV that
// only sends its outputs (whole rows, plain activations).  The plain instance carries none of
// that code.
template <int TYPE, int NB, int PAIR, int VAR>
__global__ void __launch_bounds__((consumer_warps(TYPE, PAIR, NB) + kPW) * 32, 1)
    gemv_imma_kernel(const Params p) {
  // XT: K slabs and exchanged activations; XO: outputs go to the other GPUs
  constexpr bool XT = VAR == 2, XO = VAR >= 2, PRO = VAR == 1 || VAR == 2;
  constexpr int kNW = consumer_warps(TYPE, PAIR, NB), kThreads = (kNW + kPW) * 32;
  using C = Cfg<TYPE>;
  using A = Area<TYPE>;
  constexpr bool DENSE = NB > 2;                 // batches 3 .. 8: one MMA column set per 4 batch rows
  constexpr bool V2 = TYPE == kQ6_K && !DENSE;   // integer-domain group scales, no decode pass
  static_assert(!DENSE || (PAIR == 1 && NB % 4 == 0), "dense items are single superblocks");
  constexpr int kFoldBufs = fold_bufs(NB);
  constexpr int NCX = 4 * NB;                    // columns of the quantised-x layout
  constexpr int UNIT_BYTES = NCX * 64;
  constexpr int AREA_FLOATS = V2 ? 0 : DENSE ? 16 * dense_area_row(C::NG, NB) : PAIR * NB * A::BATCH;  // PAIR superblocks per item
  extern __shared__ __align__(128) uint8_t smem[];
  // mbarriers full[S] | empty[S] in the first 128 bytes; monotone counters from byte 192:
  // chunks armed by the producer | partial sums stored per tile buffer | folds done per tile buffer
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem);
  int *issued = reinterpret_cast<int *>(smem + 192);
  int *arrivals = issued + 1, *folded = arrivals + kFoldBufs;
  int *xready = reinterpret_cast<int *>(smem + p.off_flags);  // per superblock pair of x: quantised
  const int S = p.stages;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();

  uint8_t *stages = smem + p.off_stage;
  // The jobs' 16-row tiles form one global sequence (job-major).  The grid is G row groups x
  // nslabs K slabs: this CTA takes slab `slab` of the tiles rg + i * G, i < ntl.
  const int nslabs = XT ? p.nslabs : 1;
  const int slab = nslabs > 1 ? (int)blockIdx.x % nslabs : 0;
  const int rg = nslabs > 1 ? (int)blockIdx.x / nslabs : (int)blockIdx.x;
  const int G = nslabs > 1 ? (int)gridDim.x / nslabs : (int)gridDim.x;
  const long long slab_bytes = (long long)slab * p.nblk * C::BB;  // the slab's offset into a row
  const int ntl = (p.tcum[p.njobs] - rg + G - 1) / G;
  auto locate = [&](int gt, int &j) {  // job of global tile gt, searched from the hint j
    while (gt >= p.tcum[j + 1]) j++;
    while (gt < p.tcum[j]) j--;
  };

  if (warp >= kNW) {
    // ------------------------------------------------------------------ producer warps
    // The first producer warp initialises the mbarriers, so that streaming starts without
    // waiting for the consumers' set-up; the consumers meet the producers at named barrier 3.
    const int pw = warp - kNW;
    if (pw == 0) {
      if (lane < S) mbar_init(smem_u32(&bars[lane]), kPW);
      else if (lane < 2 * S) mbar_init(smem_u32(&bars[lane]), C::KB);
      else if (lane < 2 * S + 1 + 2 * kFoldBufs) issued[lane - 2 * S] = 0;
      for (int i = lane; i < p.nflags; i += 32) xready[i] = 0;
      mbar_fence_init();
    }
    asm volatile("bar.sync 2, %0;" ::"n"(kPW * 32) : "memory");
    asm volatile("bar.arrive 3, %0;" ::"n"(kThreads) : "memory");
    if (!p.resident) pdl_wait_prior_grid();
    // every producer warp walks the same chunk sequence; warp pw issues rows 4*pw .. 4*pw+3 and
    // arrives once per chunk with the byte count of its own rows
    int s = 0, par = 1, pj = 0, cc = 0;  // stage, parity of its empty barrier, chunk number
    for (int li = 0; li < ntl; li++) {
      const int gt = rg + li * G;
      locate(gt, pj);
      const int row = (gt - p.tcum[pj]) * kR + lane;
      const bool rvalid = lane < kR && row < p.jobs[pj].out_dim;
      const uint8_t *rsrc = p.jobs[pj].w + (long long)row * p.row_bytes + slab_bytes;
      for (int c = 0; c < p.nchunks; c++) {
        if (!mbar_wait(smem_u32(&bars[S + s]), par)) {  // broken pipeline: stop, let copies land
          drain_copies_in_flight();
          return;
        }
        const int nb = min(C::KB, p.nblk - c * C::KB);
        const uint8_t *src = rsrc + (long long)c * C::KB * C::BB;
        const uint32_t padb = (uint32_t)(reinterpret_cast<uintptr_t>(src) & 15);
        const uint32_t bytes = rvalid ? ((padb + nb * C::BB + 15u) & ~15u) : 0u;
        const uint32_t full = smem_u32(&bars[s]);
        const bool mine = rvalid && (lane >> 2) == pw;
        const uint32_t my_bytes = __reduce_add_sync(0xffffffffu, mine ? bytes : 0u);
        if (COGNI_DIAG(p.debug & 4)) {  // the stage is declared full without any copy
          if (lane == 0) mbar_arrive(full);
        } else {
          if (lane == 0) mbar_arrive_expect_tx(full, my_bytes);
          __syncwarp();
          if (mine)
            bulk_g2s(smem_u32(stages + (size_t)s * p.stage_bytes + lane * C::RS), src - padb,
                     bytes, full);
        }
        // Consumers test the full barrier of chunk cc by phase parity only once this says that
        // the barrier is in (or past) that chunk's phase: a warp whose items lie far apart could
        // otherwise mistake the stage's previous fill for it.
        cc++;
        if (pw == 0 && lane == 0) st_release_shared(issued, cc);
        if (++s == S) { s = 0; par ^= 1; }
      }
    }
    if (pipe_broken()) drain_copies_in_flight();  // the consumers may not have waited for the copies
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int ctid = threadIdx.x;  // 0 .. kNW*32-1
  uint8_t *xq = smem + p.off_xq;
  float *SX = reinterpret_cast<float *>(smem + p.off_sx);
  float *XX = reinterpret_cast<float *>(smem + p.off_xx);
  const int K = p.x_pitch;  // the quantisers only use it as the pitch of the batch rows
  const int slab_el = slab * p.nblk * 256;  // the slab's first element of a row of x
  const float *xs = p.x + slab_el;
  const float *xs_up = PRO && p.x_up ? p.x_up + slab_el : nullptr;
  const float *norm_ws = PRO && p.norm_w ? p.norm_w + slab_el : nullptr;

  asm volatile("bar.sync 3, %0;" ::"n"(kThreads) : "memory");  // mbarriers and counters ready
  pdl_wait_prior_grid();  // x (and y / the addend) may be produced by the preceding kernel
  // exchanges completed on this GPU before this launch: the epoch its inputs carry (if they come
  // out of an exchange) and, plus one, the epoch its outputs get
  unsigned ex_epoch = 0;
  if (XO && p.ex.epoch) {
    // (acquire: the ticket below must not be drawn before this load has been performed)
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(ex_epoch) : "l"(p.ex.epoch) : "memory");
    // The exchange is counted by the CTA that draws the last ticket: by then every CTA of this
    // launch has read the epoch, and the next launch reads it only after this grid has completed.
    // Drawn here, at the start, the atomic's round trip hides behind the launch's work.
    if (p.ex.world > 1 && ctid == 0) {
      const unsigned ticket = atomicAdd(p.ex.ticket, 1u);
      if (ticket == gridDim.x - 1u) {
        *p.ex.ticket = 0u;
        *reinterpret_cast<volatile unsigned *>(p.ex.epoch) = ex_epoch + 1u;
      }
    }
  }
  const XSrc xsrc{XT ? p.ex_wait : 0, ex_epoch};

  // RMSNorm prologue: 1 / sqrt(mean(x^2) + eps) per batch row, the sum of squares in f64 as the
  // reference has it (qwen35_cpu.cr:484-490); per-warp partial sums are added in warp order, so
  // every warp (and every CTA) arrives at the same value.
  __shared__ double s_ss2[24 * 2];
  __shared__ float s_inv_rms[DENSE ? NB : 2];
  if (PRO && p.norm_w) {
    // batches above 2 borrow the (still unused) partial-sum buffer for the warps' sums
    constexpr int NBS = DENSE ? NB : 2;
    double *s_ss = DENSE ? reinterpret_cast<double *>(smem + p.off_red) : s_ss2;
#pragma unroll
    for (int b = 0; b < NB; b++) {
      const int br = DENSE ? min(b, p.batch - 1) : b;
      double ss = 0.0;
      for (int k = ctid * 4; k < p.norm_dim; k += kNW * 32 * 4) {
        const float4 v = XT && xsrc.ll ? ld4x<true>(p.norm_x, (long long)br * K + k, xsrc)
                                       : ld4x<false>(p.norm_x, (long long)br * K + k, xsrc);
        ss += (double)v.x * v.x + (double)v.y * v.y + (double)v.z * v.z + (double)v.w * v.w;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
      if (lane == 0) s_ss[warp * NBS + b] = ss;
    }
    consumer_sync<kNW>();
    if (ctid < NB) {
      double ss = 0.0;
      for (int w = 0; w < kNW; w++) ss += s_ss[w * NBS + ctid];
      s_inv_rms[ctid] = (float)(1.0 / sqrt(ss / (double)p.norm_dim + (double)p.norm_eps));
    }
    consumer_sync<kNW>();
  }

  const int g = lane >> 2, t = lane & 3;
  const int sub = t & 1, bt = DENSE ? 0 : (t >> 1) & (NB - 1);  // this lane's group slot and batch row
  float *area = reinterpret_cast<float *>(smem + p.off_area) + warp * AREA_FLOATS;
  const float *area_b = area + bt * A::BATCH;
  // partial sums: [tile buffer][superblock pair of the row][g][batch row] float2 (rows g, g+8)
  float2 *red = reinterpret_cast<float2 *>(smem + p.off_red);
  const int npairs = (p.nblk + PAIR - 1) / PAIR;  // items per tile
  const int red_tile = npairs * 8 * NB;
  // this lane's 16 bytes of a unit's B fragments
  const uint8_t *xlane = DENSE ? xq + lane * Dense<TYPE>::W : xq + ((g & (NCX - 1)) * 4 + t) * 16;
  const uint32_t bar0 = smem_u32(bars);

  long long best = LLONG_MIN, best_b1 = LLONG_MIN;  // fused top-1: running maxima (batch row 0 / 1)
  long long bestd[DENSE ? NB / 2 : 1];              // batches above 2: rows 2i + (lane >> 4)
#pragma unroll
  for (int i = 0; i < (DENSE ? NB / 2 : 1); i++) bestd[i] = LLONG_MIN;

  // The CTA's work is one ordered sequence of items: per tile one item per PAIR neighbouring
  // superblocks of the row (scale decode + MMAs of 16 rows x PAIR*256 columns, partial sums to the
  // tile buffer) followed by one item that folds the PREVIOUS tile (its partials are complete by
  // then); after the last tile one more fold.  Warp w takes items w, w + kNW, ...: items only ever
  // wait for items earlier in the sequence (and for the producer), so the order is deadlock-free,
  // and the warps of a scheduler are always in different phases of their items.
  const int per_tile = npairs + 1;
  int li = warp / per_tile, e = warp - li * per_tile;  // this warp's item: entry e of tile li
  const int step_li = kNW / per_tile, step_e = kNW - step_li * per_tile;  // to its next item
  const uint32_t s_inv = 0xffffffffu / (uint32_t)S + 1u;  // cc / S == umulhi(cc, s_inv), cc < 2^32 / S
  const int tail_missing = p.nchunks * C::KB - p.nblk;     // superblocks the last chunk lacks
  int cj = 0, pad_a = 0, pad_b = 0, pad_d = 0, pad_li = -1;
  for (;;) {
    if (li > ntl || (li == ntl && e > 0)) break;
    if (e < npairs && li < ntl) {
      // ------------------------------------------------ superblocks 2e, 2e+1 of tile li
      const int e0 = PAIR * e, n2 = min(PAIR, p.nblk - e0);
      const int c = e0 / C::KB, bi = e0 - c * C::KB;  // KB is even: a pair lies in one chunk
      const int cc = li * p.nchunks + c;                // chunk number, its stage and parity
      const int fill = (int)__umulhi((uint32_t)cc, s_inv), s = cc - fill * S, par = fill & 1;
      if (TYPE == kQ6_K && pad_li != li) {  // only Q6_K rows can start off a 16-byte boundary
        pad_li = li;
        const int gt = rg + li * G;
        locate(gt, cj);
        const int tile = gt - p.tcum[cj];
        const uint32_t wlow = (uint32_t)reinterpret_cast<uintptr_t>(p.jobs[cj].w) + (uint32_t)slab_bytes;
        const uint32_t rb = (uint32_t)p.row_bytes;  // the low four bits are all that matter
        pad_a = (int)((wlow + (uint32_t)(tile * kR + g) * rb) & 15u);
        pad_b = (int)((wlow + (uint32_t)(tile * kR + g + 8) * rb) & 15u);
        pad_d = (int)((wlow + (uint32_t)(tile * kR + (lane & 15)) * rb) & 15u);
      }
      // The activations are quantised on the way: the warp that takes a superblock pair of the
      // CTA's first tile does x's two superblocks first; later tiles find them done.
      if (li == 0) {
        auto quantise = [&](auto ll_tag) {
          constexpr bool LL = decltype(ll_tag)::value;
          if constexpr (V2) {
            if (PAIR == 2 && n2 == 2) quantise_q6v2<NB, 2, LL>(xs, xs_up, norm_ws, s_inv_rms, K, e0, lane, xq, SX, reinterpret_cast<int *>(XX), xsrc);
            else quantise_q6v2<NB, 1, LL>(xs, xs_up, norm_ws, s_inv_rms, K, e0, lane, xq, SX, reinterpret_cast<int *>(XX), xsrc);
          } else if constexpr (DENSE) {
            quantise_dense<TYPE, NB, LL, kDenseInt<TYPE>>(xs, xs_up, norm_ws, s_inv_rms, K, p.batch, e0, lane, xq, SX, XX, xsrc);
          } else {
            if (PAIR == 2 && n2 == 2) quantise_superblocks<TYPE, NB, 2, LL>(xs, xs_up, norm_ws, s_inv_rms, K, e0, lane, xq, SX, XX, xsrc);
            else quantise_superblocks<TYPE, NB, 1, LL>(xs, xs_up, norm_ws, s_inv_rms, K, e0, lane, xq, SX, XX, xsrc);
          }
        };
        if constexpr (XT) {
          if (xsrc.ll) quantise(std::true_type{});
          else quantise(std::false_type{});
        } else {
          quantise(std::false_type{});
        }
        __syncwarp();
        if (lane == 0) st_release_shared(&xready[e], 1);
      } else {
        spin_until_ge(&xready[e], 1);
      }
      spin_until_ge(issued, cc + 1);
      mbar_wait(bar0 + 8 * s, par);
      const int tb = li & (kFoldBufs - 1);
      const uint8_t *blk = stages + (size_t)s * p.stage_bytes + bi * C::BB;
      if constexpr (DENSE) {
        constexpr int J = NB / 4;
        float acc0[J], acc1[J];  // rows g and g+8 of batch rows 4j + t
        if constexpr (kDenseInt<TYPE>) {
          decode_dense_int<TYPE, NB>(blk + (lane & 15) * C::RS + pad_d, lane, e0, SX,
                                     reinterpret_cast<const int *>(XX), area);
          __syncwarp();
          mma_dense_int<TYPE, NB>(blk, pad_a, pad_b, xlane + (size_t)e0 * C::NG * J * Dense<TYPE>::GB,
                                  area, SX + (size_t)e0 * NB, g, t, acc0, acc1);
        } else {
          decode_dense<TYPE, NB>(blk + (lane & 15) * C::RS + pad_d, lane, e0, XX, area);
          __syncwarp();
          mma_dense<TYPE, NB>(blk, pad_a, pad_b, xlane + (size_t)e0 * C::NG * J * Dense<TYPE>::GB, area,
                              SX + (size_t)e0 * C::NG * NB + t, g, t, acc0, acc1);
        }
        __syncwarp();  // the area is rewritten by this warp's next decode
        spin_until_ge(&folded[tb], li / kFoldBufs);  // the buffer's previous tile has been folded
#pragma unroll
        for (int j = 0; j < J; j++)
          red[tb * red_tile + (e * 8 + g) * NB + 4 * j + t] = make_float2(acc0[j], acc1[j]);
      } else if constexpr (V2) {
        float acc0[NB], acc1[NB];  // rows g and g+8, this lane's scale groups (k = t) of every unit
#pragma unroll
        for (int b = 0; b < NB; b++) acc0[b] = acc1[b] = 0.f;
#pragma unroll 1
        for (int q = 0; q < n2; q++) {
          const uint8_t *ra = blk + q * C::BB + g * C::RS + pad_a;
          const uint8_t *rb = blk + q * C::BB + (g + 8) * C::RS + pad_b;
          const uint32_t *xw = reinterpret_cast<const uint32_t *>(xq) + (size_t)(e0 + q) * NB * 128 + lane;
          const int4 *ng = reinterpret_cast<const int4 *>(XX) + ((size_t)(e0 + q) * NB * 4 + t);
          const float *sxb = SX + (size_t)(e0 + q) * NB;
          const uint32_t two = (uint32_t)((reinterpret_cast<uintptr_t>(ra) | reinterpret_cast<uintptr_t>(rb)) & 2);
          if (__all_sync(0xffffffffu, two == 0)) mma_q6v2<NB, true>(ra, rb, xw, ng, sxb, lane, acc0, acc1);
          else mma_q6v2<NB, false>(ra, rb, xw, ng, sxb, lane, acc0, acc1);
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {  // the four group lanes of a row pair
          acc0[b] += __shfl_xor_sync(0xffffffffu, acc0[b], 1);
          acc1[b] += __shfl_xor_sync(0xffffffffu, acc1[b], 1);
          acc0[b] += __shfl_xor_sync(0xffffffffu, acc0[b], 2);
          acc1[b] += __shfl_xor_sync(0xffffffffu, acc1[b], 2);
        }
        spin_until_ge(&folded[tb], li / kFoldBufs);  // the buffer's previous tile has been folded
        if (t == 0) {
#pragma unroll
          for (int b = 0; b < NB; b++) red[tb * red_tile + (e * 8 + g) * NB + b] = make_float2(acc0[b], acc1[b]);
        }
      } else {
      float acc0 = 0.f, acc1 = 0.f;  // rows g and g+8 of (group slot sub, batch row bt)
      if (COGNI_DIAG(p.debug & 8)) __nanosleep(1500);  // diagnostics: keep the consumers the bottleneck
      if (COGNI_DIAG(p.debug & 3) != 1) {
        const int which = lane >> 4;
        if constexpr (PAIR == 1) {
          decode_scales_half<TYPE, NB>(blk + (lane & 15) * C::RS + pad_d, lane, e0, SX, XX, area);
        } else if (which < n2) {
          decode_scales<TYPE, NB>(blk + (lane & 15) * C::RS + pad_d + which * C::BB, lane,
                                  e0 + which, SX, XX, area);
        }
        __syncwarp();
        if (COGNI_DIAG(p.debug & 3) != 2) {
          mma_block<TYPE, UNIT_BYTES>(blk, pad_a, pad_b, xlane + (size_t)e0 * 4 * UNIT_BYTES,
                                      area_b, g, t, sub, acc0, acc1);
          if (PAIR == 2 && n2 == 2)
            mma_block<TYPE, UNIT_BYTES>(blk + C::BB, pad_a, pad_b,
                                        xlane + (size_t)(e0 + 1) * 4 * UNIT_BYTES,
                                        area_b + NB * A::BATCH, g, t, sub, acc0, acc1);
        }
        __syncwarp();  // the area is rewritten by this warp's next decode
      }
      // the two group slots of a batch row sit in neighbouring lanes
      acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
      acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
      spin_until_ge(&folded[tb], li / kFoldBufs);  // the buffer's previous tile has been folded
      if (sub == 0 && (t >> 1) < NB)
        red[tb * red_tile + (e * 8 + g) * NB + (t >> 1)] = make_float2(acc0, acc1);
      }
      __syncwarp();
      if (lane == 0) {
        // release the stage (the tile's last item also arrives for the superblocks that a short
        // final chunk lacks) and count the partial sums in
        mbar_arrive_n(bar0 + 8 * (S + s), e == npairs - 1 ? n2 + tail_missing : n2);
        add_release_shared(&arrivals[tb], 1);
      }
    } else if (li > 0) {
      // ------------------------------------------------ fold tile li - 1
      const int fl = li - 1;
      const int tb = fl & (kFoldBufs - 1);
      spin_until_ge(&arrivals[tb], (fl / kFoldBufs + 1) * npairs);  // all partials of tile fl stored
      // lane = (batch row, row of the tile): a fixed-order sum over the superblock pairs
      const int r16 = lane & 15;
      const int gt = rg + fl * G;
      // K slabs: the tile's slabs leave their partial sums in ws; the one that draws the last
      // ticket adds them up in slab order (so the result does not depend on who was last) and
      // carries on as if it had summed the whole rows itself.
      bool last_slab = true;
      auto slab_ticket = [&]() {
        // one acq_rel atomic for the warp instead of fence + atomic (+ fence for the last slab; 3-4 %
        // of a slab launch): the lanes' stores are ordered before lane 0's release by the warp
        // barrier, which is cumulative, and their loads after its acquire by the shuffle below
        __syncwarp();
        unsigned ticket = 0;
        if (lane == 0)  // release: the warp's partial sums; acquire: the other slabs', for the last one
          asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;"
                       : "=r"(ticket)
                       : "l"(&p.ws_tickets[gt])
                       : "memory");
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        last_slab = ticket == (unsigned)nslabs - 1u;
      };
      if constexpr (DENSE) {
        float v[NB / 2];  // batch rows 2i + (lane >> 4)
#pragma unroll
        for (int i = 0; i < NB / 2; i++) {
          const int b = 2 * i + (lane >> 4);
          const float *src = reinterpret_cast<const float *>(red + tb * red_tile + (r16 & 7) * NB + b) + (r16 >> 3);
          float a = 0.f;
#pragma unroll 4
          for (int k = 0; k < npairs; k++) a += src[k * 16 * NB];
          v[i] = a;
        }
        __syncwarp();
        if (lane == 0) st_release_shared(&folded[tb], fl / kFoldBufs + 1);
        if (XT && nslabs > 1) {
          float *part = p.ws + (((long long)gt * nslabs + slab) * NB + (lane >> 4)) * 16 + r16;
#pragma unroll
          for (int i = 0; i < NB / 2; i++) part[2 * i * 16] = v[i];
          slab_ticket();
          if (last_slab) {
            const float *all = p.ws + ((long long)gt * nslabs * NB + (lane >> 4)) * 16 + r16;
#pragma unroll
            for (int i = 0; i < NB / 2; i++) {
              float a = 0.f;
              for (int sl = 0; sl < nslabs; sl++) a += __ldcg(all + (sl * NB + 2 * i) * 16);
              v[i] = a;
            }
            if (lane == 0) p.ws_tickets[gt] = 0u;  // ready for the next launch on this workspace
          }
        }
        locate(gt, cj);
        const Job &job = p.jobs[cj];
        const int row = (gt - p.tcum[cj]) * kR + r16;
#pragma unroll
        for (int i = 0; i < NB / 2; i++) {
          const int b = 2 * i + (lane >> 4);
          if (last_slab && b < p.batch && row < job.out_dim) {
            if (p.part_keys) {
              const long long key = top1_key(v[i], (uint32_t)(p.index_base + row));
              bestd[i] = key > bestd[i] ? key : bestd[i];
            } else {
              const long long as = p.addend_stride < 0 ? job.out_dim : p.addend_stride;
              const float a = job.addend ? job.addend[(long long)b * as + row] : 0.f;
              const long long idx = (long long)b * (XO && p.y_pitch ? p.y_pitch : job.out_dim) + row;
              if constexpr (XO) store_y(job.y, idx, a + v[i], p.ex, ex_epoch + 1u);
              else job.y[idx] = a + v[i];
            }
          }
        }
      } else {
      const int b = lane >> 4;
      const float *src = reinterpret_cast<const float *>(red + tb * red_tile + (r16 & 7) * NB + (b & (NB - 1))) + (r16 >> 3);
      float v = 0.f;
#pragma unroll 4
      for (int k = 0; k < npairs; k++) v += src[k * 16 * NB];
      __syncwarp();
      if (lane == 0) st_release_shared(&folded[tb], fl / kFoldBufs + 1);
      if (XT && nslabs > 1) {
        if (b < NB) p.ws[(((long long)gt * nslabs + slab) * NB + b) * 16 + r16] = v;
        slab_ticket();
        if (last_slab) {
          if (b < NB) {
            const float *all = p.ws + ((long long)gt * nslabs * NB + b) * 16 + r16;
            float a = 0.f;
            for (int sl = 0; sl < nslabs; sl++) a += __ldcg(all + sl * NB * 16);
            v = a;
          }
          if (lane == 0) p.ws_tickets[gt] = 0u;  // ready for the next launch on this workspace
        }
      }
      locate(gt, cj);
      const Job &job = p.jobs[cj];
      const int row = (gt - p.tcum[cj]) * kR + r16;
      if (last_slab && b < NB && row < job.out_dim) {
        if (p.part_keys) {
          const long long key = top1_key(v, (uint32_t)(p.index_base + row));
          if (b == 0) best = key > best ? key : best;
          else best_b1 = key > best_b1 ? key : best_b1;
        } else {
          const long long as = p.addend_stride < 0 ? job.out_dim : p.addend_stride;
          const float a = job.addend ? job.addend[(long long)b * as + row] : 0.f;
          const long long idx = (long long)b * (XO && p.y_pitch ? p.y_pitch : job.out_dim) + row;
          if constexpr (XO) store_y(job.y, idx, a + v, p.ex, ex_epoch + 1u);
          else job.y[idx] = a + v;
        }
      }
      }
    }
    // next item of this warp
    e += step_e;
    li += step_li;
    if (e >= per_tile) {
      e -= per_tile;
      li++;
    }
  }

  if (p.part_keys == nullptr) return;

  // ------------------------------------------------------------ fused top-1 epilogue
  // per-CTA maximum per batch row -> scratch slot; the CTA with the last ticket folds all slots
  __shared__ long long s_best[DENSE ? NB : 2];
  __shared__ bool s_last;
  if (ctid < (DENSE ? NB : 2)) s_best[ctid] = LLONG_MIN;
  consumer_sync<kNW>();
  if constexpr (DENSE) {
#pragma unroll
    for (int i = 0; i < NB / 2; i++) atomicMax(&s_best[2 * i + (lane >> 4)], bestd[i]);
  } else {
    atomicMax(&s_best[0], best);
    if (NB > 1) atomicMax(&s_best[1], best_b1);
  }
  consumer_sync<kNW>();
  const int nparts = gridDim.x;
  // rows at or beyond the batch have no slots in the caller's scratch (it is sized for `batch` rows)
  if (ctid < NB && ctid < p.batch) p.part_keys[(long long)ctid * nparts + blockIdx.x] = s_best[ctid];
  __threadfence();
  consumer_sync<kNW>();
  if (ctid == 0) {
    const unsigned ticket = atomicAdd(p.counter, 1u);
    s_last = ticket == (unsigned)nparts - 1u;
  }
  consumer_sync<kNW>();
  if (!s_last) return;
  __threadfence();
  if (warp < NB && warp < p.batch) {
    const int b = warp;
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
int g_imma_debug = 0;

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
  return cached[dev] > 0 ? cached[dev] : 148;
}

int g_imma_force_pair = 0;  // diagnostics: 0 = automatic, 1 / 2 = superblocks per item
int g_imma_min_splits = 1;  // diagnostics: at least this many column ranges per row

template <int TYPE>
bool make_plan_pair(int in_dim, int nb, int pair, Params &p, size_t &smem, bool thin = false) {
  using C = Cfg<TYPE>;
  const int nblk = in_dim / 256;
  const int ngroups = in_dim / C::GROUP;
  auto al = [](size_t v) { return (v + 127) & ~(size_t)127; };
  size_t off = 256;  // mbarriers and counters
  // one flag per work item of a row of x: 64 for rows of up to 16384 columns (more would cost the
  // Q4_K plan at 4096 columns its fifth stage, which fits to the byte), 128 beyond
  const int nflags = (nblk + pair - 1) / pair <= 64 ? 64 : kMaxItems;
  const size_t off_flags = off;  off += (size_t)nflags * 4;
  const bool dense = nb > 2;  // nb = 4 or 8 then: single-superblock items, 2 bytes of x per element and batch row
  const bool v2 = TYPE == kQ6_K && !dense;  // Q6_K batch 1-2: no decode areas, 2 bytes of x per element and batch row
  const size_t area_floats = v2 ? 0 : dense ? (size_t)16 * dense_area_row(C::NG, nb) : (size_t)pair * nb * Area<TYPE>::BATCH;
  const size_t off_red = off;    off = al(off + (size_t)fold_bufs(nb) * ((nblk + pair - 1) / pair) * 8 * nb * 8);  // [tile buffer][item][g][batch] float2
  const size_t off_area = off;   off = al(off + (size_t)consumer_warps(TYPE, pair, nb) * area_floats * 4);
  const size_t off_sx = off;     off = al(off + (size_t)ngroups * nb * 4);
  const size_t off_xx = off;     off = al(off + (size_t)ngroups * nb * 4);
  const size_t off_xq = off;     off = al(off + (dense || v2 ? (size_t)in_dim * 2 * nb : (size_t)(in_dim / 64) * (4 * nb) * 64));
  const size_t off_stage = off;
  const size_t stage_bytes = al((size_t)kR * C::RS);
  // Three stages, or for the 4- and 8-row instances two that still keep 64 KB in flight (Q5_K
  // at 8 rows: one launch over two 45 KB stages beat two column ranges, 30 against 37 us; Q4_K
  // 17408 x 5120 at 8 rows: two 37 KB stages 29.7 us against two column ranges 31.7 and two K
  // slabs 45.9; two 27 KB Q6_K stages did not: 340 against 279 us).  `thin`: two stages of any
  // size, for the fused top-1, which cannot use column ranges.
  const size_t room = kDynSmemMax > off_stage ? kDynSmemMax - off_stage : 0;
  const bool two_ok = nb > 2 && room >= 2 * stage_bytes && (thin || 2 * stage_bytes >= 64 * 1024);
  if (room < 3 * stage_bytes && !two_ok) return false;
  int stages = (int)((kDynSmemMax - off_stage) / stage_bytes);
  if (stages > 8) stages = 8;  // 2*stages mbarriers in the first 128 bytes of shared memory
  p.in_dim = in_dim;
  p.nblk = nblk; p.nchunks = (nblk + C::KB - 1) / C::KB;
  p.stages = stages; p.row_bytes = (long long)nblk * C::BB;
  p.off_flags = (int)off_flags; p.off_red = (int)off_red; p.off_area = (int)off_area; p.off_sx = (int)off_sx;
  p.off_xx = (int)off_xx; p.off_xq = (int)off_xq; p.off_stage = (int)off_stage;
  p.stage_bytes = (int)stage_bytes;
  p.pair = pair;
  p.nflags = nflags;
  smem = off_stage + (size_t)stages * stage_bytes;
  return true;
}

// Two superblocks per item halve the per-item bookkeeping and let every lane decode scales, but
// the items a CTA can hold in its stages halve too: pairs are used when the stages still hold
// enough of them to keep the warps busy.
template <int TYPE>
bool make_plan(int in_dim, int nb, Params &p, size_t &smem, bool thin = false) {
  if (nb > 2) return make_plan_pair<TYPE>(in_dim, nb, 1, p, smem, thin);
  if (g_imma_force_pair != 1 && make_plan_pair<TYPE>(in_dim, nb, 2, p, smem) &&
      (g_imma_force_pair == 2 || p.stages * Cfg<TYPE>::KB / 2 >= 20))
    return true;
  return make_plan_pair<TYPE>(in_dim, nb, 1, p, smem);
}

template <int TYPE, int NB, int PAIR, int VAR>
int launch_instance_x(const Params &p, size_t smem, int grid, cudaStream_t s) {
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gemv_imma_kernel<TYPE, NB, PAIR, VAR>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kDynSmemMax);
    if (e != cudaSuccess) return (int)e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3((consumer_warps(TYPE, PAIR, NB) + kPW) * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemv_imma_kernel<TYPE, NB, PAIR, VAR>, p);
}
template <int TYPE, int NB, int PAIR>
int launch_instance(const Params &p, size_t smem, int grid, cudaStream_t s) {
  if (p.nslabs > 1 || p.ex_wait || (p.ex.world > 1 && (p.x_up || p.norm_w)))
    return launch_instance_x<TYPE, NB, PAIR, 2>(p, smem, grid, s);
  if (p.ex.world > 1) return launch_instance_x<TYPE, NB, PAIR, 3>(p, smem, grid, s);
  if (p.x_up || p.norm_w) return launch_instance_x<TYPE, NB, PAIR, 1>(p, smem, grid, s);
  return launch_instance_x<TYPE, NB, PAIR, 0>(p, smem, grid, s);
}

// Batch rows of the kernel instance that takes `batch` (<= 8) rows: 1, 2, 4 or 8; IQ4_NL has only
// the 4- and 8-row instances (unused rows repeat the last one).
template <int TYPE>
int kernel_rows(int batch) {
  if (batch <= 2 && TYPE != kIQ4_NL) return batch;
  return batch <= 4 ? 4 : 8;
}

// Column ranges a launch covers when a whole row of activations does not fit into shared memory:
// the fewest equal ranges of whole superblocks whose plan fits.  Every weight byte is still read
// once; the later ranges add onto y.  0 = none fits.
template <int TYPE>
int column_splits(int in_dim, int batch, bool thin = false) {
  const int nb = kernel_rows<TYPE>(batch);
  const int nblk = in_dim / 256;
  for (int n = g_imma_min_splits < nblk ? g_imma_min_splits : nblk; n <= 8 && n <= nblk; n++) {
    Params p{};
    size_t smem = 0;
    if (make_plan<TYPE>((nblk + n - 1) / n * 256, nb, p, smem, thin)) return n;
  }
  return 0;
}

// Rows of x one launch takes when the batch is above 2: 8 (4 for batches 3 and 4); 0 = no plan.
// A tail of one or two rows runs on the batch 1-2 kernels.
template <int TYPE>
int batch_pass_width(int in_dim, int batch) {
  const int width = batch > 4 ? 8 : 4;
  if (column_splits<TYPE>(in_dim, width) == 0) return 0;
  const int tail = batch % width;
  if (tail > 4 && column_splits<TYPE>(in_dim, 8) == 0) return 0;
  if (tail > 2 && tail <= 4 && column_splits<TYPE>(in_dim, 4) == 0) return 0;
  if ((tail == 1 || tail == 2) && column_splits<TYPE>(in_dim, tail) == 0) return 0;
  return width;
}

// The same for the fused top-1, which needs whole rows in one launch: 8, else 4 rows where their
// activations fit without column ranges; 0 = the fused kernel cannot take the shape.
template <int TYPE>
int top1_pass_width(int in_dim, int batch) {
  if (batch <= 2) return column_splits<TYPE>(in_dim, batch, true) == 1 ? batch : 0;
  int width = 0;
  if (batch > 4 && column_splits<TYPE>(in_dim, 8, true) == 1) width = 8;
  else if (column_splits<TYPE>(in_dim, 4, true) == 1) width = 4;
  if (width == 0) return 0;
  const int tail = batch % width;
  if (tail > 4 && column_splits<TYPE>(in_dim, 8, true) != 1) return 0;
  if (tail > 2 && tail <= 4 && column_splits<TYPE>(in_dim, 4, true) != 1) return 0;
  if ((tail == 1 || tail == 2) && column_splits<TYPE>(in_dim, tail, true) != 1) return 0;
  return width;
}

// ---------------------------------------------------------------------------- K slabs
// When a matrix has few row tiles per SM (ffn_down 4096 x 12288: 256 tiles for 148 SMs, the k / v
// projections: 64), whole-row tiles leave SMs idle or give some of them twice the work of others.
// The launch then runs as G row groups x S slabs of the K dimension: every CTA takes nblk / S
// superblocks of its tiles' rows (and quantises only that part of x), the slabs' partial sums
// meet in a workspace and the CTA that arrives last at a tile adds them in slab order.
//
// The workspace is a fixed device array (nothing is ever allocated): kWsSlots regions, one per
// stream that has used the engine, so that launches which may overlap on the device (different
// streams) never share a region; launches of one stream are ordered by the stream (a dependent
// launch touches the workspace only after its predecessor has completed).  A seventeenth stream, or
// a shape whose partial sums do not fit a region, runs without slabs.
constexpr int kWsSlots = 16;
constexpr int kWsFloats = 1 << 19;  // 2 MB of partial sums per region
constexpr int kWsTickets = 4096;    // tiles per launch that can be split
static __device__ __align__(256) float g_slab_ws[kWsSlots][kWsFloats];
static __device__ unsigned g_slab_tickets[kWsSlots][kWsTickets];

struct SlabRegion {
  float *ws;
  unsigned *tickets;
};
std::mutex g_slab_mutex;
float *g_slab_ws_base[64];
unsigned *g_slab_tickets_base[64];
cudaStream_t g_slab_streams[64][kWsSlots];
int g_slab_nstreams[64];

bool slab_region(cudaStream_t s, SlabRegion &out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
  std::lock_guard<std::mutex> lock(g_slab_mutex);
  if (!g_slab_ws_base[dev]) {  // the arrays' device addresses, once per device, that device current
    void *a = nullptr, *b = nullptr;
    if (cudaGetSymbolAddress(&a, g_slab_ws) != cudaSuccess || !a) return false;
    if (cudaGetSymbolAddress(&b, g_slab_tickets) != cudaSuccess || !b) return false;
    g_slab_ws_base[dev] = static_cast<float *>(a);
    g_slab_tickets_base[dev] = static_cast<unsigned *>(b);
  }
  int slot = -1;
  for (int i = 0; i < g_slab_nstreams[dev]; i++)
    if (g_slab_streams[dev][i] == s) slot = i;
  if (slot < 0) {
    if (g_slab_nstreams[dev] == kWsSlots) return false;
    slot = g_slab_nstreams[dev]++;
    g_slab_streams[dev][slot] = s;
  }
  out.ws = g_slab_ws_base[dev] + (size_t)slot * kWsFloats;
  out.tickets = g_slab_tickets_base[dev] + (size_t)slot * kWsTickets;
  return true;
}

int g_imma_force_slabs = 0;  // diagnostics: 0 = automatic, n = n slabs wherever a plan allows it

// Slabs for a launch of `tiles` row tiles: the count that minimises the work of the busiest CTA,
//   tiles per CTA x (superblocks per slab + the fixed cost of a tile part) + the slab's share of
//   the activation pass,
// in units of one 16-row superblock.  0 = no single-launch plan fits (not even whole rows).
template <int TYPE>
int choose_slabs(int in_dim, int nbk, int tiles, bool thin, bool workspace_ok) {
  const int nblk = in_dim / 256, sms = sm_count();
  int best = 0;
  float best_cost = 0.f;
  // Where whole rows fit, slabs are correct but not faster: the fence and the ticket of every tile
  // part sit in a consumer warp's path (measured on the 9B FFN: 15.1 against 13.2 us for ffn_down
  // with four slabs), so such a launch only uses them when asked to.  Where a row of activations
  // does not fit shared memory, slabs replace the column ranges (one launch instead of several).
  Params whole{};
  size_t whole_smem = 0;
  const bool whole_fits = make_plan<TYPE>(in_dim, nbk, whole, whole_smem, thin);
  for (int S = 1; S <= 8; S++) {
    if (nblk % S != 0 || nblk / S < 4) continue;
    if (S != 1 && S != g_imma_force_slabs && (whole_fits || g_imma_force_slabs == 1)) continue;
    if (S > 1 && (!workspace_ok || tiles > kWsTickets || (long long)tiles * S * nbk * 16 > kWsFloats ||
                  sms / S < 1))
      continue;
    Params q{};
    size_t smem = 0;
    if (!make_plan<TYPE>(nblk / S * 256, nbk, q, smem, thin)) continue;
    const int G = tiles < sms / S ? tiles : sms / S;
    const int per_cta = (tiles + G - 1) / G, len = nblk / S;
    float cost = per_cta * (len + 1.5f) + 0.3f * (nbk > 2 ? nbk / 2 : 1) * len;
    if (g_imma_force_slabs > 0 && S == g_imma_force_slabs) cost = -1.f;
    if (best == 0 || cost < best_cost) {
      best = S;
      best_cost = cost;
    }
  }
  return best;
}

// One pass: up to kMaxJobs weight matrices against `batch` rows of x (1, 2, or 3 .. 8), as one
// launch per column range.
template <int TYPE>
int run_pass(int nj, const void *const *d_w, const float *d_x, const float *const *d_addend,
             int64_t addend_stride, float *const *d_y, const int *out_dims, int in_dim, int batch,
             int resident, const Params *top1, cudaStream_t s, const float *d_x_up,
             const float *d_norm_w, float norm_eps, const Exchange *ex = nullptr, int ex_wait = 0,
             long long y_pitch = 0) {
  using C = Cfg<TYPE>;
  const int nbk = kernel_rows<TYPE>(batch);
  const bool thin = top1 != nullptr;
  const int nblk = in_dim / 256;
  int tiles = 0;
  for (int j = 0; j < nj; j++) tiles += (out_dims[j] + kR - 1) / kR;
  // One launch over K slabs where a plan allows it; else (a row of activations too long for
  // shared memory and not divisible into equal slabs) one launch per column range.
  SlabRegion region{nullptr, nullptr};
  const bool have_ws = slab_region(s, region);
  int nslabs = choose_slabs<TYPE>(in_dim, nbk, tiles, thin, have_ws);
  int nsplit = nslabs > 0 && (nslabs == 1 || top1 || ex || g_imma_force_slabs > 0) ? 1
                                                                                 : column_splits<TYPE>(in_dim, nbk, thin);
  if (nslabs > 1 && nsplit > 1) {
    // Slabs or one launch per column range?  Every tile part of a slab launch pays a workspace
    // round trip, a fence and a ticket in the folding warp's path (about 1.4 us); a column range
    // pays a launch ramp and its activation pass.  With many tiles per SM the ranges are several
    // full waves each and win, with few the slabs do.  Measured at batch 8, ranges / slabs in us:
    // Q4_K 17408 x 5120 (1088 tiles) 31.7 / 45.9, Q4_K 12288 x 7168 (768) 30.9 / 57.7, Q4_K
    // 12288 x 8192 37.4 / 51.1; Q6_K 4096 x 12288 (256) 41.4 / 30.5, Q6_K 5120 x 17408 (320)
    // 84.6 / 54.8, Q4_K 4096 x 16384 (256) 42.8 / 33.7.  (On 256 tiles and two ranges the
    // picture is mixed: Q5_K / Q8_0 4096 x 8192 21.6 / 25.2, Q6_K 4096 x 12288 at batch 4
    // 26.2 / 21.3.)
    if (tiles >= 3 * sm_count()) nslabs = 0;
    else nsplit = 1;
  } else if (nslabs > 0) {
    nsplit = 1;
  }
  if (nsplit == 0 || (top1 && nsplit > 1)) return COGNI_QMM_ERR_LIMIT;
  if (ex && nsplit > 1) return COGNI_QMM_ERR_LIMIT;  // the fused exchange needs the rows complete in one launch
  const int per = (nblk + nsplit - 1) / nsplit;
  for (int b0 = 0; b0 < nblk; b0 += per) {
    const int nb_here = nblk - b0 < per ? nblk - b0 : per;
    Params p{};
    size_t smem = 0;
    const int S = nslabs > 0 ? nslabs : 1;
    if (!make_plan<TYPE>(nb_here / S * 256, nbk, p, smem, thin)) return COGNI_QMM_ERR_LIMIT;
    p.nslabs = S;
    p.ws = region.ws;
    p.ws_tickets = region.tickets;
    if (ex) p.ex = *ex;
    p.ex_wait = ex_wait;
    p.y_pitch = y_pitch;
    p.row_bytes = (long long)nblk * C::BB;  // the pitch of the whole rows
    p.x = d_x + b0 * 256;
    p.x_up = d_x_up ? d_x_up + b0 * 256 : nullptr;
    p.norm_w = d_norm_w ? d_norm_w + b0 * 256 : nullptr;
    p.norm_x = d_x;
    p.norm_dim = in_dim;
    p.x_pitch = in_dim;
    p.norm_eps = norm_eps;
    p.batch = batch;
    p.resident = resident;
    p.debug = nbk > 2 ? (g_imma_debug & 4) : g_imma_debug;
    p.njobs = nj;
    for (int j = 0; j < nj; j++) {
      p.jobs[j].w = static_cast<const uint8_t *>(d_w[j]) + (long long)b0 * C::BB;
      p.jobs[j].y = d_y ? d_y[j] : nullptr;
      p.jobs[j].out_dim = out_dims[j];
      p.tcum[j + 1] = p.tcum[j] + (out_dims[j] + kR - 1) / kR;
      if (b0 == 0) {
        p.jobs[j].addend = d_addend ? d_addend[j] : nullptr;
      } else {  // later column ranges add onto what the earlier ones stored
        p.jobs[j].addend = p.jobs[j].y;
      }
    }
    p.addend_stride = b0 == 0 ? addend_stride : -1;  // -1: the stride of y (per job)
    const int sms = sm_count();
    const int groups = p.tcum[nj] < sms / S ? p.tcum[nj] : sms / S;
    const int grid = groups * S;
    if (top1) {
      p.part_keys = top1->part_keys;
      p.counter = top1->counter;
      p.top_idx = top1->top_idx;
      p.top_val = top1->top_val;
      p.top_key = top1->top_key;
      p.index_base = top1->index_base;
    }
    int st;
    if constexpr (TYPE != kIQ4_NL) {
      if (nbk == 1) st = p.pair == 2 ? launch_instance<TYPE, 1, 2>(p, smem, grid, s) : launch_instance<TYPE, 1, 1>(p, smem, grid, s);
      else if (nbk == 2) st = p.pair == 2 ? launch_instance<TYPE, 2, 2>(p, smem, grid, s) : launch_instance<TYPE, 2, 1>(p, smem, grid, s);
      else if (nbk == 4) st = launch_instance<TYPE, 4, 1>(p, smem, grid, s);
      else st = launch_instance<TYPE, 8, 1>(p, smem, grid, s);
    } else {
      st = nbk == 4 ? launch_instance<TYPE, 4, 1>(p, smem, grid, s) : launch_instance<TYPE, 8, 1>(p, smem, grid, s);
    }
    if (st) return st;
  }
  return COGNI_QMM_OK;
}

// njobs weight matrices (same type and in_dim), one x: the reference's qmatvec_many
// (src/ml/gguf/qwen35_cpu.cr:1419-1490) and dual GEMV (q4k_dual_gemv_probe.ptx:5) as one launch
// per 32 matrices, 8 batch rows and column range.
template <int TYPE>
int gemv_typed(int njobs, const void *const *d_w, const float *d_x, const float *const *d_addend,
               int64_t addend_stride, float *const *d_y, const int *out_dims, int in_dim, int batch,
               int resident, const Params *top1, cudaStream_t s, const float *d_x_up = nullptr,
               const float *d_norm_w = nullptr, float norm_eps = 0.f, const Exchange *ex = nullptr,
               int ex_wait = 0, long long y_pitch = 0) {

  const int width = top1 ? top1_pass_width<TYPE>(in_dim, batch)
                         : (batch <= 2 ? batch : batch_pass_width<TYPE>(in_dim, batch));
  if (width == 0) return COGNI_QMM_ERR_LIMIT;
  // the fused exchange raises its flags once: the call has to be one launch
  if (ex && (njobs > kMaxJobs || batch > width)) return COGNI_QMM_ERR_LIMIT;
  for (int b0 = 0; b0 < batch; b0 += width) {
    const int nbat = batch - b0 < width ? batch - b0 : width;
    Params t1{};  // this pass's rows of the top-1 outputs and scratch slots
    if (top1) {
      const int tiles = (out_dims[0] + kR - 1) / kR, sms = sm_count();
      t1 = *top1;
      t1.part_keys = top1->part_keys + (long long)b0 * (tiles < sms ? tiles : sms);
      t1.top_idx = top1->top_idx + b0;
      t1.top_val = top1->top_val + b0;
      t1.top_key = top1->top_key ? top1->top_key + b0 : nullptr;
    }
    for (int j0 = 0; j0 < njobs; j0 += kMaxJobs) {
      const int nj = njobs - j0 < kMaxJobs ? njobs - j0 : kMaxJobs;
      const float *add[kMaxJobs];
      float *ys[kMaxJobs];
      for (int j = 0; j < nj; j++) {
        add[j] = d_addend && d_addend[j0 + j] ? d_addend[j0 + j] + (long long)b0 * addend_stride : nullptr;
        ys[j] = d_y ? d_y[j0 + j] + (long long)b0 * out_dims[j0 + j] : nullptr;
      }
      const int st = run_pass<TYPE>(nj, d_w + j0, d_x + (long long)b0 * in_dim, d_addend ? add : nullptr,
                                    addend_stride, d_y ? ys : nullptr, out_dims + j0, in_dim, nbat, resident,
                                    top1 ? &t1 : nullptr, s, d_x_up ? d_x_up + (long long)b0 * in_dim : nullptr, d_norm_w,
                                    norm_eps, ex, ex_wait, y_pitch);
      if (st) return st;
    }
  }
  return COGNI_QMM_OK;
}

}  // namespace

void gemv_imma_set_debug(int mode) { g_imma_debug = mode; }
void gemv_imma_set_pair(int pair) { g_imma_force_pair = pair; }
void gemv_imma_set_min_splits(int n) { g_imma_min_splits = n < 1 ? 1 : n; }
void gemv_imma_set_slabs(int n) { g_imma_force_slabs = n < 0 ? 0 : n; }

bool gemv_imma_supports(int type, const void *d_w, const float *d_x, int in_dim, int batch, bool top1) {
  if (type != kQ8_0 && type != kQ4_K && type != kQ5_K && type != kQ6_K && type != kIQ4_NL) return false;
  if (batch < 1 || batch > 64) return false;
  if ((reinterpret_cast<uintptr_t>(d_w) & 15) || (reinterpret_cast<uintptr_t>(d_x) & 15)) return false;
  if (in_dim % 256 != 0 || in_dim > kMaxItems * 256) return false;
  // the activations (of a column range of the rows, if need be), the warps' areas and at least
  // three stages must fit into shared memory; the fused top-1 needs whole rows in one launch
  auto ok = [&](auto tag) {
    constexpr int T = decltype(tag)::value;
    if (top1) return top1_pass_width<T>(in_dim, batch) != 0;
    if (batch > 2) return batch_pass_width<T>(in_dim, batch) != 0;
    return column_splits<T>(in_dim, batch) != 0;
  };
  switch (type) {
    case kQ4_K: return ok(std::integral_constant<int, kQ4_K>{});
    case kQ5_K: return ok(std::integral_constant<int, kQ5_K>{});
    case kQ8_0: return ok(std::integral_constant<int, kQ8_0>{});
    case kIQ4_NL: return ok(std::integral_constant<int, kIQ4_NL>{});
    default: return ok(std::integral_constant<int, kQ6_K>{});
  }
}

int launch_gemv_imma_many(int type, int njobs, const void *const *d_w, const float *d_x,
                          const float *const *d_addend, int64_t addend_stride, float *const *d_y,
                          const int *out_dims, int in_dim, int batch, int resident, cudaStream_t s) {
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s);
    case kQ5_K: return gemv_typed<kQ5_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s);
    case kQ8_0: return gemv_typed<kQ8_0>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s);
    case kIQ4_NL: return gemv_typed<kIQ4_NL>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s);
    case kQ6_K: return gemv_typed<kQ6_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

// The same with the outputs exchanged between the GPUs of the box inside the launch (ex) and,
// optionally, the wait for the preceding exchange before x is read.
int launch_gemv_imma_many_exchange(int type, int njobs, const void *const *d_w, const float *d_x,
                                   const float *const *d_addend, int64_t addend_stride,
                                   float *const *d_y, const int *out_dims, int in_dim, int batch,
                                   int resident, const cogni_qmm_exchange *cex, int wait_previous,
                                   int64_t y_pitch, cudaStream_t s) {
  Exchange ex{};
  ex.world = cex->world;
  ex.rank = cex->rank;
  for (int g = 0; g < cex->world && g < kMaxRanks; g++) ex.peer_delta[g] = g == cex->rank ? 0 : cex->peer_offset[g];
  ex.epoch = cex->epoch;
  ex.ticket = cex->ticket;
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, nullptr, 0.f, &ex, wait_previous, y_pitch);
    case kQ5_K: return gemv_typed<kQ5_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, nullptr, 0.f, &ex, wait_previous, y_pitch);
    case kQ8_0: return gemv_typed<kQ8_0>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, nullptr, 0.f, &ex, wait_previous, y_pitch);
    case kIQ4_NL: return gemv_typed<kIQ4_NL>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, nullptr, 0.f, &ex, wait_previous, y_pitch);
    case kQ6_K: return gemv_typed<kQ6_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, nullptr, 0.f, &ex, wait_previous, y_pitch);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

int launch_gemv_imma(int type, const void *d_w, const float *d_x, const float *d_addend,
                     int64_t addend_stride, float *d_y, int in_dim, int out_dim, int batch,
                     int resident, cudaStream_t s) {
  return launch_gemv_imma_many(type, 1, &d_w, d_x, d_addend ? &d_addend : nullptr, addend_stride,
                               &d_y, &out_dim, in_dim, batch, resident, s);
}

// y = addend + W (silu(gate) * up): the SwiGLU product is formed while the activations are quantised
int launch_gemv_swiglu_imma(int type, const void *d_w, const float *d_gate, const float *d_up,
                            const float *d_addend, int64_t addend_stride, float *d_y, int in_dim,
                            int out_dim, int batch, int resident, cudaStream_t s) {
  const float *const *add = d_addend ? &d_addend : nullptr;
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(1, &d_w, d_gate, add, addend_stride, &d_y, &out_dim, in_dim, batch, resident, nullptr, s, d_up);
    case kQ5_K: return gemv_typed<kQ5_K>(1, &d_w, d_gate, add, addend_stride, &d_y, &out_dim, in_dim, batch, resident, nullptr, s, d_up);
    case kQ6_K: return gemv_typed<kQ6_K>(1, &d_w, d_gate, add, addend_stride, &d_y, &out_dim, in_dim, batch, resident, nullptr, s, d_up);
    case kQ8_0: return gemv_typed<kQ8_0>(1, &d_w, d_gate, add, addend_stride, &d_y, &out_dim, in_dim, batch, resident, nullptr, s, d_up);
    case kIQ4_NL: return gemv_typed<kIQ4_NL>(1, &d_w, d_gate, add, addend_stride, &d_y, &out_dim, in_dim, batch, resident, nullptr, s, d_up);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

// y_j = addend_j + W_j (RMSNorm(x) * norm_w): the normalisation happens while x is quantised
int launch_gemv_many_rmsnorm_imma(int type, int njobs, const void *const *d_w, const float *d_x,
                                  const float *d_norm_w, float eps, const float *const *d_addend,
                                  int64_t addend_stride, float *const *d_y, const int *out_dims,
                                  int in_dim, int batch, int resident, cudaStream_t s) {
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, d_norm_w, eps);
    case kQ5_K: return gemv_typed<kQ5_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, d_norm_w, eps);
    case kQ6_K: return gemv_typed<kQ6_K>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, d_norm_w, eps);
    case kQ8_0: return gemv_typed<kQ8_0>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, d_norm_w, eps);
    case kIQ4_NL: return gemv_typed<kIQ4_NL>(njobs, d_w, d_x, d_addend, addend_stride, d_y, out_dims, in_dim, batch, resident, nullptr, s, nullptr, d_norm_w, eps);
    default: return COGNI_QMM_ERR_TYPE;
  }
}

int launch_gemv_top1_imma(int type, const void *d_w, const float *d_x, int in_dim, int out_dim,
                          int batch, int32_t index_base, void *d_scratch, int32_t *d_idx,
                          float *d_val, long long *d_key, int resident, cudaStream_t s,
                          const float *d_norm_w, float norm_eps) {
  Params t{};
  t.counter = static_cast<unsigned *>(d_scratch);
  t.part_keys = reinterpret_cast<long long *>(static_cast<char *>(d_scratch) +
                                              (((size_t)batch * 4 + 7) & ~(size_t)7));
  t.top_idx = d_idx;
  t.top_val = d_val;
  t.top_key = d_key;
  t.index_base = index_base;
  switch (type) {
    case kQ4_K: return gemv_typed<kQ4_K>(1, &d_w, d_x, nullptr, 0, nullptr, &out_dim, in_dim, batch, resident, &t, s, nullptr, d_norm_w, norm_eps);
    case kQ5_K: return gemv_typed<kQ5_K>(1, &d_w, d_x, nullptr, 0, nullptr, &out_dim, in_dim, batch, resident, &t, s, nullptr, d_norm_w, norm_eps);
    case kQ8_0: return gemv_typed<kQ8_0>(1, &d_w, d_x, nullptr, 0, nullptr, &out_dim, in_dim, batch, resident, &t, s, nullptr, d_norm_w, norm_eps);
    case kIQ4_NL: return gemv_typed<kIQ4_NL>(1, &d_w, d_x, nullptr, 0, nullptr, &out_dim, in_dim, batch, resident, &t, s, nullptr, d_norm_w, norm_eps);
    case kQ6_K: return gemv_typed<kQ6_K>(1, &d_w, d_x, nullptr, 0, nullptr, &out_dim, in_dim, batch, resident, &t, s, nullptr, d_norm_w, norm_eps);
    default: return COGNI_QMM_ERR_TYPE;
  }
}


unsigned gemv_imma_timeouts() {
  unsigned v = 0;
  cudaMemcpyFromSymbol(&v, g_pipe_wait_timeouts, sizeof(v));
  return v;
}

// After an expired wait: clears this file's counter and the K-slab tickets (a launch that gave up
// may have left some drawn).  Synchronises the device.
int gemv_imma_reset_timeouts() {
  cudaError_t e = cudaDeviceSynchronize();
  const unsigned zero = 0;
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_pipe_wait_timeouts, &zero, sizeof(zero));
  void *tickets = nullptr;
  if (e == cudaSuccess) e = cudaGetSymbolAddress(&tickets, g_slab_tickets);
  if (e == cudaSuccess) e = cudaMemset(tickets, 0, sizeof(unsigned) * kWsSlots * kWsTickets);
  return (int)e;
}

namespace {
// One warp waits on an mbarrier that nothing ever arrives at, with the given limit: the wait runs
// out, is counted, and the kernel returns.  Exercises the give-up path of every bounded wait.
__global__ void expire_wait_kernel(unsigned long long limit_ns, int *gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_fence_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {  // one waiter, one count
    const bool ok = mbar_wait(smem_u32(&bar), 0, limit_ns);
    if (gave_up) *gave_up = ok ? 0 : 1;
  }
}
}  // namespace

namespace {
__global__ void exchange_unpack_kernel(const uint2 *words, long long n, unsigned epoch, float *out) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  uint2 w;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 0;; spin++) {
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(w.x), "=r"(w.y) : "l"(words + i) : "memory");
    if (w.y == epoch) break;
    if ((spin & 255u) == 255u) {
      if (pipe_broken()) break;
      if (global_ns() - t0 > kPipeWaitLimitNs) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        break;
      }
    }
  }
  out[i] = __uint_as_float(w.x);
}
}  // namespace

int launch_exchange_unpack(const void *d_words, int64_t n, unsigned epoch, float *d_out, cudaStream_t s) {
  exchange_unpack_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const uint2 *>(d_words), n, epoch, d_out);
  return (int)cudaGetLastError();
}

int launch_expire_wait(unsigned limit_us, cudaStream_t s) {
  if (limit_us == 0 || limit_us > 100000) return COGNI_QMM_ERR_ARG;  // at most 0.1 s
  expire_wait_kernel<<<1, 32, 0, s>>>((unsigned long long)limit_us * 1000ull, nullptr);
  return (int)cudaGetLastError();
}

}  // namespace cogni
