// Register-resident variant of the block radix select (see radix.cuh): when a
// block selects among at most 256 * E elements, every thread keeps its E keys
// (position it * 256 + tid) in registers for all passes, so the data is read
// once and the histogram passes never wait on memory.  Keys are u32 with 0
// reserved for "no element".  The 256 worker threads of a block take part.
#pragma once

#include "common.cuh"
#include "radix.cuh"

namespace mdc {

constexpr int kSelListCap = 512;  // keys still undecided when the search moves from the block to one warp

template <int E>
struct RegSelectScratch {
  uint32_t hist[256 + 32];
  int32_t bnd, c_gt, hist_bnd, pad;
  int32_t wcnt[kWarps];
  int32_t gt[E * kWarps + 1];
  int32_t eq[E * kWarps + 1];
  uint32_t list[kSelListCap];
  int32_t list_n, fin_gt;
  uint32_t fin_tau;
  int32_t pad2;
};

// K-th largest key among the non-zero keys: returns the threshold th with
// "selected <=> key > th.tau, or key == th.tau and rank among equals (position
// order) < th.need_eq"; th.n_sel = min(count, k).
//
// Bitwise search: tau grows from the top bit down, keeping a bit whenever at
// least k keys are >= the candidate; one block-wide count per bit (warp reduce +
// one shared atomic per warp), no per-element atomics; bits above the highest
// bit in which any two keys differ are copied from the maximum.  The counts also
// give the number of keys still undecided (those inside [tau, tau + 2^(bit+1))):
// once that window holds at most kSelListCap keys they are copied to a list and
// ONE warp finishes the remaining bits on its own, without block barriers.  For
// spread-out keys that happens after a handful of block-wide passes instead of
// up to 32; keys that are all alike (constant logits) run the full search.
template <int E, typename Scratch>
__device__ Threshold<uint32_t> block_select_regs(const uint32_t (&key)[E], int k, Scratch& sc) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Threshold<uint32_t> th;
  int mine = 0;
#pragma unroll
  for (int it = 0; it < E; ++it) mine += key[it] != 0u;
  mine = __reduce_add_sync(0xffffffffu, mine);
  sync_workers();
  if (lane == 0) sc.wcnt[warp] = mine;
  sync_workers();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) total += sc.wcnt[w];
  if (total <= k) {
    th.tau = 0;
    th.need_eq = 0x7fffffff;
    th.n_sel = total;
    return th;
  }
  uint32_t kmax = 0u, kmin = 0xffffffffu;
#pragma unroll
  for (int it = 0; it < E; ++it) {
    kmax = max(kmax, key[it]);
    if (key[it] != 0u) kmin = min(kmin, key[it]);
  }
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  if (lane == 0) {
    sc.hist[warp] = kmax;
    sc.hist[8 + warp] = kmin;
  }
  for (int i = tid; i < 128; i += kBlockThreads) sc.hist[32 + i] = 0;
  if (tid == 0) sc.list_n = 0;
  sync_workers();
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    kmax = max(kmax, sc.hist[w]);
    kmin = min(kmin, sc.hist[8 + w]);
  }
  const int top_bit = 31 - __clz(static_cast<int>((kmax ^ kmin) | 1u));  // highest differing bit
  uint32_t tau = (top_bit == 31) ? 0u : (kmax & ~((2u << top_bit) - 1u));
  // keys >= tau (all of them so far) and keys >= the upper end of the undecided window (none so far)
  int c_ge_tau = total, c_ge_hi = 0;
  int bit = top_bit;
#pragma unroll 1
  for (; bit >= 0; --bit) {
    if (c_ge_tau - c_ge_hi <= kSelListCap && bit >= 2) break;  // few keys left undecided: one warp finishes
    const uint32_t cand = tau | (1u << bit);
    int c = 0;
#pragma unroll
    for (int it = 0; it < E; ++it) c += key[it] >= cand;
    c = __reduce_add_sync(0xffffffffu, c);
    if (lane == 0) atomicAdd(&sc.hist[32 + bit], static_cast<uint32_t>(c));
    sync_workers();
    const int cb = static_cast<int>(sc.hist[32 + bit]);
    if (cb >= k) {
      tau = cand;
      c_ge_tau = cb;
    } else {
      c_ge_hi = cb;
    }
  }
  int count_gt;
  if (bit >= 0) {
    // undecided keys: same bits as tau above `bit`.  A warp reserves its slots with ONE atomic (a
    // shared-memory atomic per key on a single counter would serialise: ~30 cycles each).
    int n_mine = 0;
#pragma unroll
    for (int it = 0; it < E; ++it) n_mine += key[it] != 0u && ((key[it] ^ tau) >> bit) >> 1 == 0u;
    int n_warp;
    int slot = warp_excl_scan(n_mine, lane, &n_warp);
    int base = 0;
    if (lane == 31) base = atomicAdd(&sc.list_n, n_warp);
    slot += __shfl_sync(0xffffffffu, base, 31);
#pragma unroll
    for (int it = 0; it < E; ++it) {
      if (key[it] != 0u && ((key[it] ^ tau) >> bit) >> 1 == 0u) {
        if (slot < kSelListCap) sc.list[slot] = key[it];
        ++slot;
      }
    }
    sync_workers();
    if (warp == 0) {
      constexpr int PER = kSelListCap / 32;
      const int n = min(sc.list_n, kSelListCap);
      uint32_t lk[PER];
#pragma unroll
      for (int j = 0; j < PER; ++j) lk[j] = (j * 32 + lane < n) ? sc.list[j * 32 + lane] : 0u;
      uint32_t t2 = tau;
#pragma unroll 1
      for (int b = bit; b >= 0; --b) {
        const uint32_t cand = t2 | (1u << b);
        int c = 0;
#pragma unroll
        for (int j = 0; j < PER; ++j) c += lk[j] >= cand;
        c = __reduce_add_sync(0xffffffffu, c) + c_ge_hi;
        if (c >= k) t2 = cand;
      }
      int g = 0;
#pragma unroll
      for (int j = 0; j < PER; ++j) g += lk[j] > t2;
      g = __reduce_add_sync(0xffffffffu, g) + c_ge_hi;
      if (lane == 0) {
        sc.fin_tau = t2;
        sc.fin_gt = g;
      }
    }
    sync_workers();
    tau = sc.fin_tau;
    count_gt = sc.fin_gt;
  } else {
    int gt = 0;
#pragma unroll
    for (int it = 0; it < E; ++it) gt += key[it] > tau;
    gt = __reduce_add_sync(0xffffffffu, gt);
    if (lane == 0) atomicAdd(&sc.hist[64 + 32], static_cast<uint32_t>(gt));
    sync_workers();
    count_gt = static_cast<int>(sc.hist[64 + 32]);
  }
  th.tau = tau;
  th.need_eq = k - count_gt;
  th.n_sel = k;
  return th;
}

// Position-ordered output slots of the selected elements.  The caller supplies
// per element two predicates: sure(it) (selected outright) and tie(it)
// (selected iff fewer than need_eq ties precede it in position order).
// slot[it] receives the element's output index, or -1; the caller then moves
// the data in a loop of its own, free of warp votes, so its loads overlap.
// Returns the number of selected elements.
template <int E, typename Scratch, typename Sure, typename Tie>
__device__ int block_emit_regs(int need_eq, Scratch& sc, Sure sure, Tie tie, int (&slot)[E]) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  sync_workers();
#pragma unroll
  for (int it = 0; it < E; ++it) {
    const uint32_t gb = __ballot_sync(0xffffffffu, sure(it));
    const uint32_t eb = __ballot_sync(0xffffffffu, tie(it));
    if (lane == 0) {
      sc.gt[it * kWarps + warp] = __popc(gb);
      sc.eq[it * kWarps + warp] = __popc(eb);
    }
  }
  sync_workers();
  if (warp == 0) {  // exclusive scans of both tables in (it, warp) order
    constexpr int N = E * kWarps, PER = N / 32;
    int g[PER], q[PER], gs = 0, qs = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      g[j] = sc.gt[lane * PER + j];
      q[j] = sc.eq[lane * PER + j];
      gs += g[j];
      qs += q[j];
    }
    int gtot, qtot;
    int gb = warp_excl_scan(gs, lane, &gtot), qb = warp_excl_scan(qs, lane, &qtot);
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      sc.gt[lane * PER + j] = gb;
      sc.eq[lane * PER + j] = qb;
      gb += g[j];
      qb += q[j];
    }
    if (lane == 31) {
      sc.gt[N] = gb;
      sc.eq[N] = qb;
    }
  }
  sync_workers();
  const uint32_t lt = (1u << lane) - 1u;
#pragma unroll
  for (int it = 0; it < E; ++it) {
    const bool s = sure(it), t = tie(it);
    const uint32_t eb = __ballot_sync(0xffffffffu, t);
    const int eq_before = sc.eq[it * kWarps + warp];
    const bool take = s || (t && eq_before + __popc(eb & lt) < need_eq);
    const uint32_t tb = __ballot_sync(0xffffffffu, take);
    slot[it] = take ? sc.gt[it * kWarps + warp] + min(eq_before, need_eq) + __popc(tb & lt) : -1;
  }
  const int total = sc.gt[E * kWarps] + min(sc.eq[E * kWarps], need_eq);
  sync_workers();
  return total;
}

}  // namespace mdc
