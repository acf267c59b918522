// Thin inline-PTX wrappers for the sm_100a features the two fused Ulysses
// exchange GEMMs use: mbarriers, TMA (cp.async.bulk.tensor, never with
// cluster multicast), tcgen05 tensor-core MMA with TMEM accumulators, and
// system-scope release/acquire accesses for the cross-GPU hand-off flags.
//
// Every wait in this file is bounded: it polls, and after `timeout_ns` of
// wall time (read from %globaltimer) it gives up and returns false so the
// caller can record an error code and leave the kernel normally.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mup {

// ---------------------------------------------------------------------------
// Small helpers
// ---------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// 64-bit words in shared memory that one CTA of a cluster writes and the other
// polls (relaxed, cluster scope: strong accesses, a word is never seen torn).
__device__ __forceinline__ void st_relaxed_cluster_smem_u64(uint32_t cluster_smem_addr, uint64_t value) {
  asm volatile("st.relaxed.cluster.shared::cluster.u64 [%0], %1;" ::"r"(cluster_smem_addr), "l"(value) : "memory");
}
__device__ __forceinline__ uint64_t ld_relaxed_cluster_smem_u64(uint32_t local_smem_addr) {
  uint64_t v;
  asm volatile("ld.relaxed.cluster.shared::cta.u64 %0, [%1];" : "=l"(v) : "r"(local_smem_addr) : "memory");
  return v;
}

// One lane of the (fully converged) warp; the same lane every time.
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// Address of `local_smem_addr` inside CTA `cta_rank` of this cluster
// (shared::cluster window).
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t local_smem_addr, uint32_t cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(cta_rank));
  return r;
}

__device__ __forceinline__ void cluster_arrive_release() {
  asm volatile("barrier.cluster.arrive.release;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait_acquire() {
  asm volatile("barrier.cluster.wait.acquire;" ::: "memory");
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrive on a barrier that may live in another CTA of the cluster.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Programmatic dependent launch. `grid_dep_launch` lets the next kernel of the
// stream be scheduled while this one still runs (it then sits in its own
// `grid_dep_wait`); `grid_dep_wait` returns once the previous kernel has
// completed and its memory operations are visible. Both are no-ops for a
// kernel launched without the programmatic-serialization attribute.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Non-blocking test of a phase (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. `abort_flag` is a CTA-shared word any role sets when it
// gives up; a set flag makes every other wait give up at its next check.
// `spin` polls with the non-suspending test_wait instead of try_wait (which may
// park the thread for a hardware-chosen time before it looks again).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile uint32_t* abort_flag,
                                                  uint64_t timeout_ns, bool spin = false) {
  if (spin) {
    if (mbar_test_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 1;; ++it) {
      if (mbar_test_wait(bar, parity)) return true;
      if ((it & 0x3ffu) == 0) {
        if (*abort_flag != 0u) return false;
        if (globaltimer_ns() - t0 > timeout_ns) return false;
      }
    }
  }
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 0xffu) == 0) {
      if (*abort_flag != 0u) return false;
      if (globaltimer_ns() - t0 > timeout_ns) return false;
    }
  }
}

// ---------------------------------------------------------------------------
// Proxy fences
// ---------------------------------------------------------------------------

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies). No cluster multicast anywhere.
// ---------------------------------------------------------------------------

__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// global -> this CTA's shared memory, completion on a barrier of this CTA.
__device__ __forceinline__ void tma_load_2d(uint32_t smem_dst, const CUtensorMap* map, int c0,
                                            int c1, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar)
      : "memory");
}

// global -> this CTA's shared memory; the completion barrier may belong to
// the other CTA of a cta_group::2 pair (`cluster_bar` is a shared::cluster
// address). Each CTA loads its own half: this is not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t smem_dst, const CUtensorMap* map, int c0,
                                                 int c1, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(cluster_bar)
      : "memory");
}

// L2 eviction-priority policies for the cache-hinted copies below.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}

// The two loads above with an L2 eviction-priority hint.
__device__ __forceinline__ void tma_load_2d_hint(uint32_t smem_dst, const CUtensorMap* map, int c0,
                                                 int c1, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair_hint(uint32_t smem_dst, const CUtensorMap* map,
                                                      int c0, int c1, uint32_t cluster_bar,
                                                      uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      ".L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(cluster_bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d_hint(const CUtensorMap* map, int c0, int c1,
                                                  uint32_t smem_src, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group.L2::cache_hint [%0, {%1, %2}], [%3], %4;" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(c0), "r"(c1), "r"(smem_src), "l"(policy)
      : "memory");
}

// shared memory -> global (possibly a peer GPU's mapped memory).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, int c0, int c1,
                                             uint32_t smem_src) {
  asm volatile(
      "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(c0), "r"(c1), "r"(smem_src)
      : "memory");
}

__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM management, MMA, commit, TMEM loads
// ---------------------------------------------------------------------------

template <int G>
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  if constexpr (G == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot),
                 "r"(ncols)
                 : "memory");
  }
}

template <int G>
__device__ __forceinline__ void tmem_relinquish() {
  if constexpr (G == 1) {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  } else {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
}

template <int G>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if constexpr (G == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  } else {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
  }
}

__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem]^T, BF16 inputs, FP32 accumulate.
template <int G>
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  if constexpr (G == 1) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Arrive (count 1) on `bar` of this CTA once every MMA issued so far by this
// thread has finished reading shared memory / writing TMEM.
__device__ __forceinline__ void umma_commit_1(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// cta_group::2 form; `cluster_bar` is a shared::cluster address, so the same
// event can be delivered to either CTA of the pair with one commit each.
__device__ __forceinline__ void umma_commit_2(uint32_t cluster_bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar)
      : "memory");
}

// One commit delivered to the barrier at the same shared-memory offset in
// every CTA named by `cta_mask` (an mbarrier arrival, not a data load).
__device__ __forceinline__ void umma_commit_2_mask(uint32_t bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"(cta_mask)
      : "memory");
}

// One 64-wide K step of the main loop as a single instruction sequence for the
// issuing thread: a non-blocking test of the NEXT stage's full barrier is
// issued first, then the four 16-wide MMAs of this stage and the commit that
// releases it; the test's result is read only after the commit, so the
// barrier round trip (~70 cycles for a thread that does nothing else) overlaps
// the MMA issue slots instead of adding to them. Returns non-zero when the
// next stage was already full.
template <int G>
__device__ __forceinline__ uint32_t umma_kstep4_probe_next(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                           uint32_t idesc, uint32_t accumulate_first,
                                                           uint32_t commit_bar, uint32_t next_full_bar,
                                                           uint32_t next_parity) {
  uint32_t next_ready;
  if constexpr (G == 1) {
    asm volatile(
        "{\n"
        ".reg .pred pn, pa;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 pn, [%7], %8;\n"
        "setp.ne.b32 pa, %5, 0;\n"
        "add.u64 a1, %2, 2;\n"
        "add.u64 b1, %3, 2;\n"
        "add.u64 a2, %2, 4;\n"
        "add.u64 b2, %3, 4;\n"
        "add.u64 a3, %2, 6;\n"
        "add.u64 b3, %3, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, pa;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %4, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %4, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %4, 1;\n"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
        "selp.u32 %0, 1, 0, pn;\n"
        "}\n"
        : "=r"(next_ready)
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(commit_bar),
          "r"(next_full_bar), "r"(next_parity)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred pn, pa;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3;\n"
        ".reg .b16 both;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 pn, [%7], %8;\n"
        "setp.ne.b32 pa, %5, 0;\n"
        "mov.b16 both, 3;\n"
        "add.u64 a1, %2, 2;\n"
        "add.u64 b1, %3, 2;\n"
        "add.u64 a2, %2, 4;\n"
        "add.u64 b2, %3, 4;\n"
        "add.u64 a3, %2, 6;\n"
        "add.u64 b3, %3, 6;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %2, %3, %4, pa;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a1, b1, %4, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a2, b2, %4, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a3, b3, %4, 1;\n"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%6], both;\n"
        "selp.u32 %0, 1, 0, pn;\n"
        "}\n"
        : "=r"(next_ready)
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(commit_bar),
          "r"(next_full_bar), "r"(next_parity)
        : "memory");
  }
  return next_ready;
}

// The same step for an item of two parts: the A tile of the stage feeds two
// accumulators (two W boxes, two instruction descriptors), eight MMAs between
// the probe and the commit.
template <int G>
__device__ __forceinline__ uint32_t umma_kstep8_probe_next(uint32_t d_tmem0, uint32_t d_tmem1, uint64_t a_desc,
                                                           uint64_t b_desc0, uint64_t b_desc1, uint32_t idesc0,
                                                           uint32_t idesc1, uint32_t accumulate_first,
                                                           uint32_t commit_bar, uint32_t next_full_bar,
                                                           uint32_t next_parity) {
  uint32_t next_ready;
  if constexpr (G == 1) {
    asm volatile(
        "{\n"
        ".reg .pred pn, pa;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3, c1, c2, c3;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 pn, [%10], %11;\n"
        "setp.ne.b32 pa, %8, 0;\n"
        "add.u64 a1, %3, 2;\n"
        "add.u64 a2, %3, 4;\n"
        "add.u64 a3, %3, 6;\n"
        "add.u64 b1, %4, 2;\n"
        "add.u64 b2, %4, 4;\n"
        "add.u64 b3, %4, 6;\n"
        "add.u64 c1, %5, 2;\n"
        "add.u64 c2, %5, 4;\n"
        "add.u64 c3, %5, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %3, %4, %6, pa;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a1, b1, %6, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a2, b2, %6, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], a3, b3, %6, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], %3, %5, %7, pa;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a1, c1, %7, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a2, c2, %7, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%2], a3, c3, %7, 1;\n"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%9];\n"
        "selp.u32 %0, 1, 0, pn;\n"
        "}\n"
        : "=r"(next_ready)
        : "r"(d_tmem0), "r"(d_tmem1), "l"(a_desc), "l"(b_desc0), "l"(b_desc1), "r"(idesc0), "r"(idesc1),
          "r"(accumulate_first), "r"(commit_bar), "r"(next_full_bar), "r"(next_parity)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred pn, pa;\n"
        ".reg .b64 a1, a2, a3, b1, b2, b3, c1, c2, c3;\n"
        ".reg .b16 both;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 pn, [%10], %11;\n"
        "setp.ne.b32 pa, %8, 0;\n"
        "mov.b16 both, 3;\n"
        "add.u64 a1, %3, 2;\n"
        "add.u64 a2, %3, 4;\n"
        "add.u64 a3, %3, 6;\n"
        "add.u64 b1, %4, 2;\n"
        "add.u64 b2, %4, 4;\n"
        "add.u64 b3, %4, 6;\n"
        "add.u64 c1, %5, 2;\n"
        "add.u64 c2, %5, 4;\n"
        "add.u64 c3, %5, 6;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], %3, %4, %6, pa;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a1, b1, %6, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a2, b2, %6, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%1], a3, b3, %6, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%2], %3, %5, %7, pa;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%2], a1, c1, %7, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%2], a2, c2, %7, 1;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%2], a3, c3, %7, 1;\n"
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%9], both;\n"
        "selp.u32 %0, 1, 0, pn;\n"
        "}\n"
        : "=r"(next_ready)
        : "r"(d_tmem0), "r"(d_tmem1), "l"(a_desc), "l"(b_desc0), "l"(b_desc1), "r"(idesc0), "r"(idesc1),
          "r"(accumulate_first), "r"(commit_bar), "r"(next_full_bar), "r"(next_parity)
        : "memory");
  }
  return next_ready;
}

// 32 lanes x 32 consecutive FP32 columns: thread t of the warp receives row
// (lane quarter base + t), registers = columns.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major BF16 tile stored as rows of
// 128 bytes (64 BF16) with the 128-byte swizzle TMA applies: 8-row groups are
// 1024 bytes apart (stride byte offset), the leading byte offset is unused
// for swizzled K-major operands (encoded 1), descriptor version 1 (sm_100),
// layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor for kind::f16 with BF16 A and B (both K-major) and
// FP32 accumulation: c_format F32 (bit 4), a/b format BF16 (bits 7, 10),
// N>>3 at bit 17, M>>4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// System-scope accesses for cross-GPU flags
// ---------------------------------------------------------------------------

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}
__device__ __forceinline__ void fence_acq_rel_gpu() {
  asm volatile("fence.acq_rel.gpu;" ::: "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_gpu_u64(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add_u64(uint64_t* p, uint64_t v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// 16-byte coherent load that does not allocate in L1 (a pulled row is read
// once by this SM; the copy that matters lands in L2 through the store).
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

}  // namespace mup
