// PTX wrappers shared by the tensor-core kernels: mbarriers with bounded waits, TMA tile loads, tcgen05
// (MMA issue, commit, tensor-memory loads, fences), named barriers and the shared-memory matrix descriptor.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace i8l {

// Host: tensor map of a bf16 [rows, K] matrix in boxes of 128 x 128 elements, unswizzled (defined with the
// other tensor-map code next to the GEMM launcher).
int make_tile_map_bf16(CUtensorMap* map, const void* ptr, int64_t rows, int64_t K);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One poll: returns when the phase has completed or after the hardware's own time limit.  HINT adds
// a suspend-time hint operand: it measured 1.3 % faster for the whole-K kernels (long waits by idle
// warps) and 1 % slower for the block-scaled ones (short waits on the critical path).
template <bool HINT>
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if (HINT) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(1000000u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
  }
  return ok;
}
// Bounded wait.  A poll whose phase is incomplete parks the thread in hardware (about 4 us on a
// B200, whatever suspend-time hint is given) and returns early when the phase completes, so a wait
// is one instruction in the common case and the loop below runs only for waits longer than that.
// The limit is a poll count (2^19 polls, about 2 s): no timer, no 64-bit arithmetic in the hot loops.
// Returns false when the limit is hit or another warp has set the abort flag.
constexpr uint32_t WAIT_MAX_POLLS = 1u << 19;
template <bool HINT = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t max_polls = WAIT_MAX_POLLS) {
  if (mbar_try_wait<HINT>(bar, parity)) return true;
  for (uint32_t spin = 1; spin < max_polls; ++spin) {
    if (mbar_try_wait<HINT>(bar, parity)) return true;
    if ((spin & 63u) == 0 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}
// The same bound for a caller that cannot leave its loop: returns when the phase has completed, or after
// the limit with the abort flag set; once the flag is set (by any warp) a wait gives up after one poll.
template <bool HINT = false>
__device__ __forceinline__ void mbar_wait_or_flag(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  uint32_t max_polls = WAIT_MAX_POLLS) {
  if (mbar_try_wait<HINT>(bar, parity)) return;
  for (uint32_t spin = 1; spin < max_polls; ++spin) {
    if (*abort_flag) return;
    if (mbar_try_wait<HINT>(bar, parity)) return;
  }
  *abort_flag = 1;
}
// Non-suspending poll and a bounded spin on it, for the one wait that sits on the critical path of the
// block-scaled kinds (the epilogue's wait for a finished accumulator): a suspended try_wait wakes up some
// hundred cycles after the phase completes, a spinning warp sees it at once (measured 4 % on the whole GEMM;
// the epilogue warps have nothing else to issue while they wait).  The limit scales the poll limit by the
// ratio of the two polls' durations; once the abort flag is set the spin ends at the next check.
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ void mbar_spin_or_flag(uint32_t bar, uint32_t parity, volatile int* abort_flag, uint32_t max_polls) {
  if (mbar_test_wait(bar, parity)) return;
  for (uint32_t poll = 0; poll < max_polls; ++poll) {
    for (int i = 0; i < 512; ++i)
      if (mbar_test_wait(bar, parity)) return;
    if (*abort_flag) return;
  }
  *abort_flag = 1;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
// --- CTA-pair (cta_group::2) variants ---------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA load whose completion is signalled on a barrier of either CTA of the pair (no multicast).
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {  // arrives on `bar` in both CTAs of the pair
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ void tc_commit_pair_local(uint32_t bar) {  // arrives on the executing CTA's barrier only
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void named_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void named_arrive(int id, int nthreads) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// Shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (the layout TMA writes with CU_TENSOR_MAP_SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
  uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;              // leading byte offset (unused with swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;    // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;              // descriptor version for sm_100
  d |= (uint64_t)2 << 61;              // SWIZZLE_128B
  return d;
}
}  // namespace i8l
