// Slot hand-off folded into the kernels that produce or consume the slots.
//
// A sync point is a number in one sequence that every rank of the group walks
// through in the same order. "Signal e" = store e into entry `rank` of every
// peer's flag array (system-scope release) once ALL CTAs (or pull warps) of
// this kernel have finished the work the signal stands for; "wait e" = poll
// this rank's own flag array until every entry has reached e (system-scope
// acquire, bounded). A stand-alone barrier is signal + wait in one tiny
// kernel; folding the signal into the tail of the kernel before it and the
// wait into the head of the kernel after it removes two launches per
// operation and lets the wait overlap with work that does not need it.
#pragma once

#include "mup_ptx.cuh"

namespace mup {

struct SyncParams {
  uint32_t* flags[8];              // flags[p] = rank p's flag array (mapped in this process); null: no hand-off
  unsigned long long* done;        // device counter, only ever incremented
  unsigned long long done_target;  // value of *done once every participant of this launch has arrived
  uint32_t* status;                // error word (host-visible), may be null
  unsigned long long timeout_ns;
  uint32_t wait_epoch;             // 0: nothing to wait for
  uint32_t signal_epoch;           // 0: nothing to signal
  int up;
  int rank;
};

constexpr uint32_t kSyncStatusFlagTimeout = 7;  // same code as the stand-alone barrier

// Poll until peer `peer` has signalled `wait_epoch`. Callers give every peer its
// own thread (lanes 0 .. up-1) so that the polls overlap, then combine the
// results with a vote. Returns false when the wait ran out (the status word
// then holds the code).
__device__ __forceinline__ bool sync_wait_one(const SyncParams& sp, int peer) {
  if (sp.wait_epoch == 0u || sp.flags[0] == nullptr || peer >= sp.up) return true;
  const uint32_t* flag = sp.flags[sp.rank] + peer;
  const uint64_t t0 = globaltimer_ns();
  uint32_t it = 0;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - sp.wait_epoch) < 0) {
    if ((++it & 0x1fu) == 0) {
      if (globaltimer_ns() - t0 > sp.timeout_ns) {
        if (sp.status != nullptr) {
          *reinterpret_cast<volatile uint32_t*>(sp.status) =
              (kSyncStatusFlagTimeout << 24) | (static_cast<uint32_t>(peer) & 0xFFFFFFu);
        }
        return false;
      }
      __nanosleep(100);
    }
  }
  return true;
}

// Whole-warp form: lanes 0 .. up-1 poll one peer each.
__device__ __forceinline__ bool sync_wait_warp(const SyncParams& sp, int lane) {
  const bool mine = sync_wait_one(sp, lane);
  return __all_sync(0xffffffffu, mine);
}

// Called by one thread per participant after that participant's work (and the
// work of the threads it synchronised with) is complete. The last arrival
// publishes `signal_epoch` to every peer.
__device__ __forceinline__ void sync_arrive_and_signal(const SyncParams& sp) {
  if (sp.signal_epoch == 0u || sp.flags[0] == nullptr) return;
  fence_acq_rel_gpu();
  const unsigned long long before = atomicAdd(sp.done, 1ull);
  if (before + 1ull == sp.done_target) {
    fence_acq_rel_sys();
    for (int peer = 0; peer < sp.up; ++peer) st_release_sys(sp.flags[peer] + sp.rank, sp.signal_epoch);
  }
}

}  // namespace mup
