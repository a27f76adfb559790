// Device side of the event system: u64 monotonic counters, one 128-byte cell
// per event per rank.  Phase p of an event is complete on a rank when its cell
// there holds arity * (p + 1); nothing is ever reset.
//
//   notify(ev, dst)  one posted reduction (+1, release) into rank dst's cell:
//                    gpu scope for the own rank, system scope for a peer.
//                    Exactly one thread per arity contribution may call it.
//   wait(ev, target) thread 0 of the block polls the LOCAL cell (acquire) with
//                    a nanosleep back-off and a time budget, then the block's
//                    worker barrier publishes the result.  Returns false when
//                    the budget ran out (the caller reports and winds down);
//                    nothing in this library spins without a bound.
//
//
// Payload rule.  A flag-only wait does not fence the whole block at system
// scope (that costs ~1.7 us per wait).  Payload that a PEER GPU wrote before
// its notify must therefore be read with the system-scope loads of common.cuh
// (ld_sys_u4 / ld_sys_f32 / ld_acquire_sys_f4), which bypass the non-coherent
// L1; payload written by this GPU's own blocks may be read with plain loads.
//
// Device counterpart of mega_dsa_cp/events/core.py:40-134 of the reference.
#pragma once

#include "common.cuh"

namespace mdc {

constexpr int kCellBytes = 128;

struct EventSet {
  unsigned char* base;     // this rank's cells
  const int64_t* offsets;  // [world] byte offset of each rank's cells from `base`
  int32_t my_rank;
  int32_t world;

  __device__ unsigned long long* cell(int ev) const {
    return reinterpret_cast<unsigned long long*>(base + static_cast<int64_t>(ev) * kCellBytes);
  }
  __device__ unsigned long long* peer_cell(int ev, int dst) const {
    return reinterpret_cast<unsigned long long*>(base + offsets[dst] + static_cast<int64_t>(ev) * kCellBytes);
  }
  // single-issuer notify
  __device__ void notify_1t(int ev, int dst) const {
    if (dst == my_rank) red_release_gpu_add_u64(cell(ev), 1ull);
    else red_release_sys_add_u64(peer_cell(ev, dst), 1ull);
  }
  // notify after the whole block has fenced (system scope) and met at a barrier: the ordering is
  // already established, so the reduction itself carries none.  A release per notify would make a
  // task with one notify per rank pay a system-scope fence per rank.
  __device__ void notify_1t_fenced(int ev, int dst) const {
    if (dst == my_rank) red_relaxed_gpu_add_u64(cell(ev), 1ull);
    else red_relaxed_sys_add_u64(peer_cell(ev, dst), 1ull);
  }
  // single-thread bounded poll; returns the last value seen through *seen
  __device__ bool poll_1t(int ev, unsigned long long target, bool sys, long long budget_ns,
                          unsigned long long* seen, uint32_t max_backoff = 512) const {
    const unsigned long long* p = cell(ev);
    unsigned long long v = sys ? ld_acquire_sys_u64(p) : ld_acquire_gpu_u64(p);
    if (v < target) {
      const unsigned long long t0 = global_timer_ns();
      uint32_t backoff = 32;
      while (v < target) {
        nanosleep(backoff);
        if (backoff < max_backoff) backoff <<= 1;
        v = sys ? ld_acquire_sys_u64(p) : ld_acquire_gpu_u64(p);
        if (v < target && static_cast<long long>(global_timer_ns() - t0) > budget_ns) break;
      }
    }
    *seen = v;
    return v >= target;
  }
};

}  // namespace mdc
