// Device view of the symmetric payload arena: every rank holds the same
// layout, so a byte offset plus the per-rank base offset addresses any peer's
// copy.  Payload reaches a peer either by plain 16-byte stores (posted over
// NVLink) or by one bulk copy shared -> peer global (push_start / push_finish);
// a notify with release semantics at system scope follows the payload.
//
// Device counterpart of mega_dsa_cp/comm/device.py:11-44 and
// comm/primitives.py:29-93 of the reference.
#pragma once

#include "common.cuh"

namespace mdc {

struct PeerBuffer {
  unsigned char* base;     // this rank's arena
  const int64_t* offsets;  // [world] byte offset of each rank's arena from `base`
  int32_t my_rank;
  int32_t world;
  int64_t mc_base;         // NVLS multicast address of the arena, 0 when unavailable

  __device__ unsigned char* local_ptr(int64_t off) const { return base + off; }
  __device__ unsigned char* peer_ptr(int64_t off, int dst) const { return base + offsets[dst] + off; }
  __device__ bool has_mc() const { return mc_base != 0; }
};

// Starts an asynchronous bulk copy of `bytes` (multiple of 16) from shared
// memory to (peer) global memory.  One thread; the shared source must have been
// made visible to the async proxy (fence_proxy_async_smem after the writes and
// a barrier).
__device__ inline void push_start(void* gdst, const void* smem_src, uint32_t bytes) {
  bulk_s2g(gdst, smem_src, bytes);
  bulk_commit();
}
// Completes every push this thread started and orders it before a following
// notify.  Keep unrelated work between start and finish: the wait exposes the
// transfer's completion latency.
__device__ inline void push_finish() {
  bulk_wait_all();
  fence_proxy_async_global();
}

// Copies `bytes` (multiple of 16, 16-byte aligned) from local global memory to a
// peer with all worker threads; plain vector stores, posted.
__device__ inline void copy_to_peer(void* gdst, const void* gsrc, int bytes) {
  const uint4* s = static_cast<const uint4*>(gsrc);
  uint4* d = static_cast<uint4*>(gdst);
  for (int i = threadIdx.x; i < bytes / 16; i += kBlockThreads) d[i] = s[i];
}

}  // namespace mdc
