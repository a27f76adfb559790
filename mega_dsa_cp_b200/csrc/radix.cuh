// Block-wide exact top-k by radix select, shared by the fused local top-k of
// the indexer tile and by the candidate merge tile.
//
// Keys are unsigned integers whose order is the selection order (larger is
// better): u32 = sortable(logit) when positions break ties, u64 =
// (sortable(logit) << 32) | ~id for explicit ids.  The select walks the key
// bytes from the top, one 256-bin histogram per byte over the elements that
// still match the prefix found so far; lanes of a warp that hit the same bin are
// combined with match.any before touching shared memory, so a histogram costs
// one shared atomic per distinct bin per warp instead of one per element.  The
// emit is deterministic: output slot = number of selected elements at lower
// positions, computed from warp ballots, never from atomics.
#pragma once

#include "common.cuh"

namespace mdc {

constexpr int kBitsListCap = 256;  // undecided keys at which the bitwise search moves from the block to one warp

struct SelectScratch {
  uint32_t hist[256 + 32];  // 256 bins + one dummy bin per lane for non-matching elements
  int32_t bnd, c_gt, hist_bnd, total;
  int32_t wgt[kWarps], weq[kWarps];
  uint32_t list[kBitsListCap];
  int32_t list_n, fin_gt, fin_eq;
  uint32_t fin_tau;
};

template <typename KeyT>
struct Threshold {
  KeyT tau;         // selected: key > tau, or key == tau and rank among equals < need_eq
  int32_t need_eq;
  int32_t n_sel;    // number of selected elements = min(total valid, k)
};

// src(pos, valid) -> key.  All threads of the block call this with the same
// arguments; n_pos is the padded position space, k >= 1.
template <typename KeyT, typename Src>
__device__ Threshold<KeyT> block_select_threshold(Src src, int n_pos, int k, SelectScratch& sc) {
  constexpr int NPASS = static_cast<int>(sizeof(KeyT));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int iters = ceil_div(n_pos, kBlockThreads);
  Threshold<KeyT> th;

  // total number of valid elements
  int mine = 0;
  for (int it = 0; it < iters; ++it) {
    int pos = it * kBlockThreads + tid;
    bool valid = false;
    if (pos < n_pos) (void)src(pos, valid);
    mine += valid ? 1 : 0;
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  sync_workers();  // scratch may still be in use by a previous call
  if (lane == 0) sc.wgt[warp] = mine;
  sync_workers();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) total += sc.wgt[w];
  if (total <= k) {
    th.tau = 0;
    th.need_eq = 0x7fffffff;
    th.n_sel = total;
    sync_workers();
    return th;
  }

  KeyT prefix = 0;
  int remaining = k;
  bool done = false;
#pragma unroll 1
  for (int p = 0; p < NPASS && !done; ++p) {
    const int shift = 8 * (NPASS - 1 - p);
    for (int i = tid; i < 256 + 32; i += kBlockThreads) sc.hist[i] = 0;
    sync_workers();
    for (int it = 0; it < iters; ++it) {
      int pos = it * kBlockThreads + tid;
      bool valid = false;
      KeyT key = 0;
      if (pos < n_pos) key = src(pos, valid);
      bool hit = valid;
      if (p > 0) hit = hit && ((key >> (shift + 8)) == (prefix >> (shift + 8)));
      uint32_t bin = hit ? static_cast<uint32_t>((key >> shift) & 0xff) : 256u + lane;
      uint32_t peers = __match_any_sync(0xffffffffu, bin);
      if (hit && lane == __ffs(peers) - 1) atomicAdd(&sc.hist[bin], __popc(peers));
    }
    sync_workers();
    if (warp == 0) {
      // lane l owns bins 255-8l .. 248-8l, scanned from the top
      uint32_t c[8];
      int local = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        c[j] = sc.hist[255 - 8 * lane - j];
        local += c[j];
      }
      int tot;
      int cum = warp_excl_scan(local, lane, &tot);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (cum < remaining && cum + static_cast<int>(c[j]) >= remaining) {
          sc.bnd = 255 - 8 * lane - j;
          sc.c_gt = cum;
          sc.hist_bnd = c[j];
        }
        cum += c[j];
      }
    }
    sync_workers();
    prefix |= static_cast<KeyT>(sc.bnd) << shift;
    remaining -= sc.c_gt;
    if (sc.hist_bnd == remaining) done = true;  // the boundary bin is taken whole
    sync_workers();
  }
  if (done) {
    if (prefix == 0) {
      th.tau = 0;
      th.need_eq = 0x7fffffff;
    } else {
      th.tau = prefix - 1;
      th.need_eq = 0;
    }
  } else {
    th.tau = prefix;
    th.need_eq = remaining;
  }
  th.n_sel = k;
  return th;
}

// Same contract as block_select_threshold for u32 keys (0 = no element) that
// are cheap to re-read (shared memory): a bitwise search for the k-th largest
// key, one block-wide count per bit, no per-element atomics.  key(pos) -> u32.
template <typename KeyFn>
__device__ Threshold<uint32_t> block_select_bits(KeyFn key, int n_pos, int k, SelectScratch& sc, int* n_eq_out = nullptr) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Threshold<uint32_t> th;
  uint32_t kmax = 0u, kmin = 0xffffffffu;
  int mine = 0;
  for (int pos = tid; pos < n_pos; pos += kBlockThreads) {
    const uint32_t kv = key(pos);
    mine += kv != 0u;
    kmax = max(kmax, kv);
    if (kv != 0u) kmin = min(kmin, kv);
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  sync_workers();
  if (lane == 0) {
    sc.wgt[warp] = mine;
    sc.hist[warp] = kmax;
    sc.hist[8 + warp] = kmin;
  }
  for (int i = tid; i < 128; i += kBlockThreads) sc.hist[32 + i] = 0;
  sync_workers();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    total += sc.wgt[w];
    kmax = max(kmax, sc.hist[w]);
    kmin = min(kmin, sc.hist[8 + w]);
  }
  if (total <= k) {
    th.tau = 0;
    th.need_eq = 0x7fffffff;
    th.n_sel = total;
    sync_workers();
    return th;
  }
  const int top_bit = 31 - __clz(static_cast<int>((kmax ^ kmin) | 1u));
  uint32_t tau = (top_bit == 31) ? 0u : (kmax & ~((2u << top_bit) - 1u));
#pragma unroll 1
  for (int bit = top_bit; bit >= 0; --bit) {
    const uint32_t cand = tau | (1u << bit);
    int c = 0;
    for (int pos = tid; pos < n_pos; pos += kBlockThreads) c += key(pos) >= cand;
    c = __reduce_add_sync(0xffffffffu, c);
    if (lane == 0) atomicAdd(&sc.hist[32 + bit], static_cast<uint32_t>(c));
    sync_workers();
    if (static_cast<int>(sc.hist[32 + bit]) >= k) tau = cand;
  }
  int gt = 0, eq = 0;
  for (int pos = tid; pos < n_pos; pos += kBlockThreads) {
    const uint32_t kv = key(pos);
    gt += kv > tau;
    eq += kv == tau;
  }
  gt = __reduce_add_sync(0xffffffffu, gt);
  eq = __reduce_add_sync(0xffffffffu, eq);
  if (lane == 0) {
    atomicAdd(&sc.hist[96], static_cast<uint32_t>(gt));
    atomicAdd(&sc.hist[97], static_cast<uint32_t>(eq));
  }
  sync_workers();
  th.tau = tau;
  th.need_eq = k - static_cast<int>(sc.hist[96]);
  th.n_sel = k;
  if (n_eq_out) *n_eq_out = static_cast<int>(sc.hist[97]);  // keys equal to the threshold
  sync_workers();
  return th;
}

// block_select_bits for a u32 key array in shared memory (16-byte aligned, n_pos a multiple of 4
// or padded with zeros up to one).  Every loop stays rolled, so the code is a few hundred bytes and
// runs out of the instruction cache: work that a block does once per task is bound by instruction
// fetch when it is written as straight-line code (measured on the candidate merge: 5.3 stall cycles
// per issued instruction waiting for instructions, 60 % instruction-cache hit rate).
// The counts of the search also tell how many keys are still undecided (inside
// [tau, tau + 2^(bit+1))); once at most kBitsListCap are left they are copied to a list and ONE
// warp settles the remaining bits without block barriers.  Spread-out keys get there after about
// ten block-wide passes instead of 32; keys that are all alike run the full search.
__device__ inline Threshold<uint32_t> block_select_bits_smem(const uint32_t* keys, int n_pos, int k, SelectScratch& sc,
                                                             int* n_eq_out = nullptr) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n4 = n_pos >> 2;
  const uint4* k4 = reinterpret_cast<const uint4*>(keys);
  Threshold<uint32_t> th;
  uint32_t kmax = 0u, kmin = 0xffffffffu;
  int mine = 0;
#pragma unroll 2
  for (int i = tid; i < n4; i += kBlockThreads) {
    const uint4 q = k4[i];
    const uint32_t v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mine += v[j] != 0u;
      kmax = max(kmax, v[j]);
      kmin = min(kmin, v[j] != 0u ? v[j] : 0xffffffffu);
    }
  }
  for (int i = (n4 << 2) + tid; i < n_pos; i += kBlockThreads) {
    const uint32_t v = keys[i];
    mine += v != 0u;
    kmax = max(kmax, v);
    kmin = min(kmin, v != 0u ? v : 0xffffffffu);
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  sync_workers();
  if (lane == 0) {
    sc.wgt[warp] = mine;
    sc.hist[warp] = kmax;
    sc.hist[8 + warp] = kmin;
  }
  for (int i = tid; i < 128; i += kBlockThreads) sc.hist[32 + i] = 0;
  if (tid == 0) sc.list_n = 0;
  sync_workers();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    total += sc.wgt[w];
    kmax = max(kmax, sc.hist[w]);
    kmin = min(kmin, sc.hist[8 + w]);
  }
  if (total <= k) {
    th.tau = 0;
    th.need_eq = 0x7fffffff;
    th.n_sel = total;
    sync_workers();
    return th;
  }
  const int top_bit = 31 - __clz(static_cast<int>((kmax ^ kmin) | 1u));
  uint32_t tau = (top_bit == 31) ? 0u : (kmax & ~((2u << top_bit) - 1u));
  // keys >= tau (all of them so far) and keys >= the upper end of the undecided window (none so far)
  int c_ge_tau = total, c_ge_hi = 0;
  int bit = top_bit;
#pragma unroll 1
  for (; bit >= 0; --bit) {
    if (c_ge_tau - c_ge_hi <= kBitsListCap && bit >= 2) break;
    const uint32_t cand = tau | (1u << bit);
    int c = 0;
#pragma unroll 2
    for (int i = tid; i < n4; i += kBlockThreads) {
      const uint4 q = k4[i];
      c += (q.x >= cand) + (q.y >= cand) + (q.z >= cand) + (q.w >= cand);
    }
    for (int i = (n4 << 2) + tid; i < n_pos; i += kBlockThreads) c += keys[i] >= cand;
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
  if (bit >= 0) {
    // the undecided keys (same bits as tau above `bit`) -> list; a warp reserves its slots with one atomic
    const int n_iter = ceil_div(n_pos, kBlockThreads);
#pragma unroll 1
    for (int it = 0; it < n_iter; ++it) {
      const int i = it * kBlockThreads + tid;
      const uint32_t v = i < n_pos ? keys[i] : 0u;
      const bool in = v != 0u && ((v ^ tau) >> bit) >> 1 == 0u;
      const uint32_t m = __ballot_sync(0xffffffffu, in);
      if (m != 0u) {
        int base = 0;
        if (lane == 0) base = atomicAdd(&sc.list_n, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0);
        const int slot = base + __popc(m & ((1u << lane) - 1u));
        if (in && slot < kBitsListCap) sc.list[slot] = v;
      }
    }
    sync_workers();
    if (warp == 0) {
      constexpr int PER = kBitsListCap / 32;
      const int n = min(sc.list_n, kBitsListCap);
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
      int g = 0, e = 0;
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        g += lk[j] > t2;
        e += lk[j] == t2;
      }
      g = __reduce_add_sync(0xffffffffu, g) + c_ge_hi;
      e = __reduce_add_sync(0xffffffffu, e);
      if (lane == 0) {
        sc.fin_tau = t2;
        sc.fin_gt = g;
        sc.fin_eq = e;
      }
    }
    sync_workers();
    th.tau = sc.fin_tau;
    th.need_eq = k - sc.fin_gt;
    th.n_sel = k;
    if (n_eq_out) *n_eq_out = sc.fin_eq;
    sync_workers();
    return th;
  }
  int gt = 0, eq = 0;
#pragma unroll 2
  for (int i = tid; i < n4; i += kBlockThreads) {
    const uint4 q = k4[i];
    gt += (q.x > tau) + (q.y > tau) + (q.z > tau) + (q.w > tau);
    eq += (q.x == tau) + (q.y == tau) + (q.z == tau) + (q.w == tau);
  }
  for (int i = (n4 << 2) + tid; i < n_pos; i += kBlockThreads) {
    gt += keys[i] > tau;
    eq += keys[i] == tau;
  }
  gt = __reduce_add_sync(0xffffffffu, gt);
  eq = __reduce_add_sync(0xffffffffu, eq);
  if (lane == 0) {
    atomicAdd(&sc.hist[96], static_cast<uint32_t>(gt));
    atomicAdd(&sc.hist[97], static_cast<uint32_t>(eq));
  }
  sync_workers();
  th.tau = tau;
  th.need_eq = k - static_cast<int>(sc.hist[96]);
  th.n_sel = k;
  if (n_eq_out) *n_eq_out = static_cast<int>(sc.hist[97]);  // keys equal to the threshold
  sync_workers();
  return th;
}

// The k-th largest of the valid (non-zero) u32 keys of a shared-memory array by histograms instead of
// one block-wide pass per bit: the keys' common upper bits are skipped (kmax ^ kmin), then each level
// histograms the next 11 bits of the keys that are still undecided (2048 bins: spread-out keys meet
// little contention), finds the boundary bin and descends into it; as soon as the boundary bin holds at
// most kBitsListCap keys they are copied to a list and one warp settles the remaining bits.  Three
// levels cover 32 bits.  Same result and conventions as block_select_bits_smem.  hist: 2048 words of
// shared memory.  keys: 16-byte aligned, n_pos a multiple of 4 or zero-padded to one.
__device__ inline Threshold<uint32_t> block_select_hist_smem(const uint32_t* keys, int n_pos, int k, SelectScratch& sc,
                                                            uint32_t* hist, int* n_eq_out = nullptr) {
  constexpr int kBins = 2048, kBits = 11, PER = kBins / kBlockThreads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n4 = n_pos >> 2;
  const uint4* k4 = reinterpret_cast<const uint4*>(keys);
  Threshold<uint32_t> th;
  uint32_t kmax = 0u, kmin = 0xffffffffu;
  int mine = 0;
  for (int i = tid; i < n4; i += kBlockThreads) {
    const uint4 q = k4[i];
    const uint32_t v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      mine += v[j] != 0u;
      kmax = max(kmax, v[j]);
      kmin = min(kmin, v[j] != 0u ? v[j] : 0xffffffffu);
    }
  }
  for (int i = (n4 << 2) + tid; i < n_pos; i += kBlockThreads) {
    const uint32_t v = keys[i];
    mine += v != 0u;
    kmax = max(kmax, v);
    kmin = min(kmin, v != 0u ? v : 0xffffffffu);
  }
  mine = __reduce_add_sync(0xffffffffu, mine);
  kmax = __reduce_max_sync(0xffffffffu, kmax);
  kmin = __reduce_min_sync(0xffffffffu, kmin);
  sync_workers();
  if (lane == 0) {
    sc.wgt[warp] = mine;
    sc.hist[warp] = kmax;
    sc.hist[8 + warp] = kmin;
  }
  sync_workers();
  int total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    total += sc.wgt[w];
    kmax = max(kmax, sc.hist[w]);
    kmin = min(kmin, sc.hist[8 + w]);
  }
  if (total <= k) {
    th.tau = 0;
    th.need_eq = 0x7fffffff;
    th.n_sel = total;
    sync_workers();
    return th;
  }
  int lo_bits = 32 - __clz(static_cast<int>((kmax ^ kmin) | 1u));   // the low bits in which valid keys differ
  uint32_t prefix = lo_bits >= 32 ? 0u : (kmax >> lo_bits) << lo_bits;
  int remaining = k;   // rank of the wanted key among the keys that share `prefix` above lo_bits
#pragma unroll 1
  while (true) {
    const int shift = max(0, lo_bits - kBits);
    const uint32_t bmask = (1u << (lo_bits - shift)) - 1u;
    for (int i = tid; i < kBins; i += kBlockThreads) hist[i] = 0u;
    if (tid == 0) {
      sc.bnd = 0;
      sc.c_gt = 0;
      sc.hist_bnd = 0;
      sc.list_n = 0;
    }
    sync_workers();
    for (int i = tid; i < n4; i += kBlockThreads) {
      const uint4 q = k4[i];
      const uint32_t v[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool in = v[j] != 0u && (lo_bits >= 32 || ((v[j] ^ prefix) >> lo_bits) == 0u);
        if (in) atomicAdd(&hist[(v[j] >> shift) & bmask], 1u);
      }
    }
    for (int i = (n4 << 2) + tid; i < n_pos; i += kBlockThreads) {
      const uint32_t v = keys[i];
      if (v != 0u && (lo_bits >= 32 || ((v ^ prefix) >> lo_bits) == 0u)) atomicAdd(&hist[(v >> shift) & bmask], 1u);
    }
    sync_workers();
    uint32_t c[PER];
    int local = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      c[j] = hist[kBins - 1 - PER * tid - j];
      local += static_cast<int>(c[j]);
    }
    int wtot;
    int cum = warp_excl_scan(local, lane, &wtot);
    if (lane == 0) sc.wgt[warp] = wtot;
    sync_workers();
    for (int w = 0; w < warp; ++w) cum += sc.wgt[w];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (cum < remaining && cum + static_cast<int>(c[j]) >= remaining) {   // (one thread at most)
        sc.bnd = kBins - 1 - PER * tid - j;
        sc.c_gt = cum;
        sc.hist_bnd = static_cast<int>(c[j]);
      }
      cum += static_cast<int>(c[j]);
    }
    sync_workers();
    const int inside = sc.hist_bnd;
    prefix |= static_cast<uint32_t>(sc.bnd) << shift;
    remaining -= sc.c_gt;
    lo_bits = shift;
    sync_workers();
    if (shift == 0) {   // the bin is one key value: `inside` keys equal it, `remaining` of them are wanted
      th.tau = prefix;
      th.need_eq = remaining;
      th.n_sel = k;
      if (n_eq_out) *n_eq_out = inside;
      return th;
    }
    if (inside <= kBitsListCap) break;
  }
  // the keys of the boundary bin -> list; one warp settles their low lo_bits bits
  {
    const int n_iter = ceil_div(n_pos, kBlockThreads);
#pragma unroll 1
    for (int it = 0; it < n_iter; ++it) {
      const int i = it * kBlockThreads + tid;
      const uint32_t v = i < n_pos ? keys[i] : 0u;
      const bool in = v != 0u && ((v ^ prefix) >> lo_bits) == 0u;
      const uint32_t m = __ballot_sync(0xffffffffu, in);
      if (m != 0u) {
        int base = 0;
        if (lane == 0) base = atomicAdd(&sc.list_n, __popc(m));
        base = __shfl_sync(0xffffffffu, base, 0);
        const int slot = base + __popc(m & ((1u << lane) - 1u));
        if (in && slot < kBitsListCap) sc.list[slot] = v;
      }
    }
  }
  sync_workers();
  if (warp == 0) {
    constexpr int LPER = kBitsListCap / 32;
    const int ln = min(sc.list_n, kBitsListCap);
    uint32_t lk[LPER];
#pragma unroll
    for (int j = 0; j < LPER; ++j) lk[j] = (j * 32 + lane < ln) ? sc.list[j * 32 + lane] : 0u;
    uint32_t t2 = prefix;
#pragma unroll 1
    for (int bit = lo_bits - 1; bit >= 0; --bit) {
      const uint32_t cand = t2 | (1u << bit);
      int cnt = 0;
#pragma unroll
      for (int j = 0; j < LPER; ++j) cnt += lk[j] >= cand;
      cnt = __reduce_add_sync(0xffffffffu, cnt);
      if (cnt >= remaining) t2 = cand;
    }
    int g = 0, e = 0;
#pragma unroll
    for (int j = 0; j < LPER; ++j) {
      g += lk[j] > t2;
      e += lk[j] == t2;
    }
    g = __reduce_add_sync(0xffffffffu, g);
    e = __reduce_add_sync(0xffffffffu, e);
    if (lane == 0) {
      sc.fin_tau = t2;
      sc.fin_gt = g;
      sc.fin_eq = e;
    }
  }
  sync_workers();
  th.tau = sc.fin_tau;
  th.need_eq = remaining - sc.fin_gt;
  th.n_sel = k;
  if (n_eq_out) *n_eq_out = sc.fin_eq;
  sync_workers();
  return th;
}

// Deterministic emit of the selected elements in position order.
// emit(pos, slot) is called once per selected element; returns the count.
template <typename KeyT, typename Src, typename Emit>
__device__ int block_emit_selected(Src src, int n_pos, Threshold<KeyT> th, SelectScratch& sc, Emit emit) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = ceil_div(ceil_div(n_pos, kWarps), 32) * 32;
  const int lo = warp * seg;
  const int hi = min(n_pos, lo + seg);
  int gt = 0, eq = 0;
  for (int base = lo; base < hi; base += 32) {
    int pos = base + lane;
    bool valid = false;
    KeyT key = 0;
    if (pos < hi) key = src(pos, valid);
    gt += __popc(__ballot_sync(0xffffffffu, valid && key > th.tau));
    eq += __popc(__ballot_sync(0xffffffffu, valid && key == th.tau));
  }
  sync_workers();
  if (lane == 0) {
    sc.wgt[warp] = gt;
    sc.weq[warp] = eq;
  }
  sync_workers();
  int gt_before = 0, eq_before = 0, gt_all = 0, eq_all = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) {
      gt_before += sc.wgt[w];
      eq_before += sc.weq[w];
    }
    gt_all += sc.wgt[w];
    eq_all += sc.weq[w];
  }
  int out_run = gt_before + min(eq_before, th.need_eq);
  int eq_run = eq_before;
  const uint32_t lt = (1u << lane) - 1u;
  for (int base = lo; base < hi; base += 32) {
    int pos = base + lane;
    bool valid = false;
    KeyT key = 0;
    if (pos < hi) key = src(pos, valid);
    bool g = valid && key > th.tau;
    bool e = valid && key == th.tau;
    uint32_t eb = __ballot_sync(0xffffffffu, e);
    bool take = g || (e && (eq_run + __popc(eb & lt)) < th.need_eq);
    uint32_t tb = __ballot_sync(0xffffffffu, take);
    if (take) emit(pos, out_run + __popc(tb & lt));
    out_run += __popc(tb);
    eq_run += __popc(eb);
  }
  sync_workers();
  return gt_all + min(eq_all, th.need_eq);
}

// block_emit_selected for u32 keys that sit in shared memory (0 = no element): four positions per
// 16-byte load, one warp prefix scan per 128 positions instead of two ballots per 32, and the scan
// over ties only where a warp actually meets one.  Same slots, same order, same return value.
// Falls back to the generic routine when the array is not 16-byte aligned or n_pos is not a
// multiple of 4.
template <typename Emit>
__device__ int block_emit_keys(const uint32_t* vb, int n_pos, Threshold<uint32_t> th, SelectScratch& sc, Emit emit) {
  if ((n_pos & 3) != 0 || (smem_u32(vb) & 15u) != 0u) {
    return block_emit_selected<uint32_t>([&](int pos, bool& valid) { valid = vb[pos] != 0u; return vb[pos]; }, n_pos, th,
                                         sc, emit);
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = ceil_div(ceil_div(n_pos, kWarps), 128) * 128;
  const int lo = min(n_pos, warp * seg), hi = min(n_pos, lo + seg);
  const bool all = th.need_eq == 0x7fffffff;  // every valid key is selected (valid keys are >= 1)
  const uint32_t tau = all ? 0u : th.tau;
  const int need_eq = all ? 0 : th.need_eq;
  int g = 0, e = 0;
  for (int pos = lo + 4 * lane; pos < hi; pos += 128) {
    const uint4 k = *reinterpret_cast<const uint4*>(vb + pos);
    g += (k.x > tau) + (k.y > tau) + (k.z > tau) + (k.w > tau);
    if (!all) e += (k.x == tau) + (k.y == tau) + (k.z == tau) + (k.w == tau);
  }
  g = __reduce_add_sync(0xffffffffu, g);
  e = __reduce_add_sync(0xffffffffu, e);
  sync_workers();
  if (lane == 0) {
    sc.wgt[warp] = g;
    sc.weq[warp] = e;
  }
  sync_workers();
  int gt_before = 0, eq_before = 0, gt_all = 0, eq_all = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) {
      gt_before += sc.wgt[w];
      eq_before += sc.weq[w];
    }
    gt_all += sc.wgt[w];
    eq_all += sc.weq[w];
  }
  int out_run = gt_before + min(eq_before, need_eq);
  int eq_run = eq_before;
  const bool ties_here = !all && sc.weq[warp] != 0;
  for (int base = lo; base < hi; base += 128) {
    const int pos = base + 4 * lane;
    uint4 k = make_uint4(0u, 0u, 0u, 0u);
    if (pos < hi) k = *reinterpret_cast<const uint4*>(vb + pos);
    const uint32_t kk[4] = {k.x, k.y, k.z, k.w};
    uint32_t take = 0u;
    int e_tot = 0;
    if (ties_here) {
      int e_cnt = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) e_cnt += kk[i] == tau;
      const int e_excl = warp_excl_scan(e_cnt, lane, &e_tot);
      int room = need_eq - (eq_run + e_excl);  // ties this thread may still take, in position order
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const bool t = kk[i] > tau || (kk[i] == tau && room-- > 0);
        take |= static_cast<uint32_t>(t) << i;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) take |= static_cast<uint32_t>(kk[i] > tau) << i;
    }
    int t_tot;
    int slot = out_run + warp_excl_scan(__popc(take), lane, &t_tot);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if ((take >> i) & 1u) emit(pos + i, slot++);
    }
    out_run += t_tot;
    eq_run += e_tot;
  }
  sync_workers();
  return gt_all + min(eq_all, need_eq);
}

}  // namespace mdc
