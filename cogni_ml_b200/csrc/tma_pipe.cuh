// mbarrier / bulk-async-copy / programmatic-dependent-launch helpers shared by the tiled kernels.
//
// Every wait on an mbarrier is bounded by a wall-clock limit: on expiry the waiter records the
// event in a device counter, treats the wait as satisfied and carries on, so a kernel always runs
// to completion (its results are then invalid; cogni_qmm_wait_timeouts() reports it and
// cogni_qmm_reset_wait_timeouts() clears the counters once the host has dealt with it).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace cogni {

constexpr unsigned long long kPipeWaitLimitNs = 1000000000ull;

// one counter per translation unit that includes this header; summed by the host accessor
static __device__ unsigned int g_pipe_wait_timeouts;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_n(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
// try_wait that lets the hardware keep the warp suspended for up to `hint_ns` while the phase is
// incomplete, instead of returning to a polling loop that competes for issue slots
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Waits for the phase with the given parity; gives up after kPipeWaitLimitNs.  Once any wait of
// the process has expired, later waits give up at their first slow-path check, so a broken
// pipeline costs one time limit in total rather than one per wait.  Returns false when it gave
// up: a consumer may carry on with invalid data, a producer must stop issuing copies.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          unsigned long long limit_ns = kPipeWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 1;; spin++) {
    if (mbar_try_wait_suspend(bar, parity, 20000u)) return true;
    __nanosleep(spin < 4 ? 32 : 256);
    if ((spin & 15u) == 0) {
      if (*reinterpret_cast<volatile unsigned int *>(&g_pipe_wait_timeouts) != 0u) return false;
      if (global_ns() - t0 > limit_ns) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        return false;
      }
    }
  }
}
// The same wait with cluster-scope acquire: for a barrier that threads of the peer CTA of a
// cluster arrive on after writing their own shared memory.
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(hint_ns)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity,
                                                  unsigned long long limit_ns = kPipeWaitLimitNs) {
  if (mbar_try_wait_cluster(bar, parity, 0u)) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 1;; spin++) {
    if (mbar_try_wait_cluster(bar, parity, 20000u)) return true;
    __nanosleep(spin < 4 ? 32 : 256);
    if ((spin & 15u) == 0) {
      if (*reinterpret_cast<volatile unsigned int *>(&g_pipe_wait_timeouts) != 0u) return false;
      if (global_ns() - t0 > limit_ns) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        return false;
      }
    }
  }
}
// Acquire / release accesses to counters and flags in shared memory at CTA scope: the data they
// publish is ordinary shared memory written before the release and read after the acquire.
__device__ __forceinline__ int ld_acquire_shared(const int *p) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.b32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_shared(int *p, int v) {
  asm volatile("st.release.cta.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
__device__ __forceinline__ void add_release_shared(int *p, int v) {
  asm volatile("red.release.cta.shared::cta.add.s32 [%0], %1;" ::"r"(smem_u32(p)), "r"(v) : "memory");
}
// Waits until a monotone counter in shared memory reaches `target`, with the same limit and
// give-up rule as mbar_wait.  Counters cannot be misread the way a phase parity can when a
// waiter is several phases ahead of the barrier.
__device__ __forceinline__ bool spin_until_ge(const int *counter, int target) {
  if (ld_acquire_shared(counter) >= target) return true;
  const unsigned long long t0 = global_ns();
  for (unsigned spin = 1;; spin++) {
    if (ld_acquire_shared(counter) >= target) return true;
    __nanosleep(64);
    if ((spin & 63u) == 0) {
      if (*reinterpret_cast<volatile unsigned int *>(&g_pipe_wait_timeouts) != 0u) return false;
      if (global_ns() - t0 > kPipeWaitLimitNs) {
        atomicAdd(&g_pipe_wait_timeouts, 1u);
        return false;
      }
    }
  }
}
__device__ __forceinline__ bool pipe_broken() {
  return *reinterpret_cast<volatile unsigned int *>(&g_pipe_wait_timeouts) != 0u;
}
// A producer that stops after a failed wait must not let its CTA retire while bulk copies it
// issued are still landing in the CTA's shared memory: it sits out a time that any copy in
// flight completes in (they take microseconds), independent of the state of the mbarriers.
__device__ __forceinline__ void drain_copies_in_flight() {
  const unsigned long long t0 = global_ns();
  while (global_ns() - t0 < 200000ull) {
  }
}
// 1-D bulk copy global -> shared, completion counted in bytes on an mbarrier.
// src, dst 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
// Programmatic dependent launch: let the next kernel of the stream start launching / wait until
// the previous kernel of the stream has completed and its writes are visible.  Both are no-ops
// for a kernel that was not launched with the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grid() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

}  // namespace cogni
