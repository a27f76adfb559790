// Candidate-merge tile: exact top-k over L variable-length candidate lists of
// one (b, t), emitted in padded input order so that every rank that merges the
// same all-gathered lists writes bit-identical output.
//
// Key = (sortable(logit) << 32) | ~id: larger key <=> larger logit, ties by
// smaller id.  The lists are re-read from global memory (L2-resident, 8 B per
// candidate) once per radix pass; passes stop as soon as the boundary bin is
// taken whole, which for distinct logits happens after the four value bytes.
#pragma once

#include "common.cuh"
#include "radix.cuh"
#include "radix_regs.cuh"

namespace mdc {

constexpr int kMergeMaxLists = 256;


constexpr int kMergeRegE = 32;  // register path: up to 256 * 32 = 8192 candidate positions per row

constexpr int kMergeBigE = 64;  // keys of up to 256 * 64 = 16384 positions stay in registers for the search

struct MergeSmem {
  union {
    SelectScratch sel;
    RegSelectScratch<kMergeRegE> rsel;
    RegSelectScratch<kMergeBigE> rsel_big;
  };
  int32_t cnt[kMergeMaxLists];
  int32_t off[kMergeMaxLists + 1];  // compact staging: first staged position of each list
  int32_t qoff[kMergeMaxLists + 1]; // compact staging: first 16-byte quad of each list (a list of n entries has ceil(n/4))
};

// The L lists of one row: list l holds values at v + l * stride, ids at
// i + l * stride, its count at c[l * c_stride] (strides in 4-byte elements).
struct MergeLists {
  const float* v;
  const int32_t* i;
  const int32_t* c;
  int64_t stride, c_stride;
};

__device__ inline float ld_f32(const float* p, bool sys) { return sys ? ld_sys_f32(p) : __ldg(p); }

// SYS: the lists were written by peer GPUs (loads must bypass the L1).
// Called by the 256 worker threads.  out_v / out_i / out_c point at this row's output.
template <bool SYS>
__device__ inline int merge_lists_tile(const MergeLists& ls, int L, int maxK, int top_k, float* out_v, int32_t* out_i,
                                       int32_t* out_c, int32_t* dbg, MergeSmem& sm) {
  const int tid = threadIdx.x;
  sync_workers();
  for (int l = tid; l < L; l += kBlockThreads) {
    const int32_t* cp = ls.c + l * ls.c_stride;
    int c = SYS ? __float_as_int(ld_sys_f32(reinterpret_cast<const float*>(cp))) : *cp;
    sm.cnt[l] = max(0, min(c, maxK));
  }
  sync_workers();
  auto src = [&](int pos, bool& valid) -> unsigned long long {
    const int l = pos / maxK, j = pos - l * maxK;
    valid = j < sm.cnt[l];
    if (!valid) return 0ull;
    const uint32_t hi = sortable_u32(ld_f32(ls.v + l * ls.stride + j, SYS));
    const uint32_t lo = ~static_cast<uint32_t>(__float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS)));
    return (static_cast<unsigned long long>(hi) << 32) | lo;
  };
  const int n_pos = L * maxK;
  Threshold<unsigned long long> th = block_select_threshold<unsigned long long>(src, n_pos, top_k, sm.sel);
  int n = block_emit_selected<unsigned long long>(src, n_pos, th, sm.sel, [&](int pos, int slot) {
    if (slot < top_k) {
      const int l = pos / maxK, j = pos - l * maxK;
      out_v[slot] = ld_f32(ls.v + l * ls.stride + j, SYS);
      out_i[slot] = __float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS));
    }
  });
  if (tid == 0) {
    *out_c = min(n, top_k);
    if (n != th.n_sel && dbg) atomicAdd(dbg, 1);
  }
  return min(n, top_k);
}

// Register-resident path of merge_lists_tile for L * maxK <= 256 * E: one read
// of the lists, a u32 select on the logits, and -- only when equal logits
// straddle the boundary -- a second u32 select on ~id among the tied entries.
template <int E, bool SYS>
__device__ inline int merge_lists_regs(const MergeLists& ls, int L, int maxK, int top_k, float* out_v, int32_t* out_i,
                                       int32_t* out_c, int32_t* dbg, MergeSmem& sm) {
  const int tid = threadIdx.x;
  const int n_pos = L * maxK;
  sync_workers();
  for (int l = tid; l < L; l += kBlockThreads) {
    const int32_t* cp = ls.c + l * ls.c_stride;
    int c = SYS ? __float_as_int(ld_sys_f32(reinterpret_cast<const float*>(cp))) : *cp;
    sm.cnt[l] = max(0, min(c, maxK));
  }
  sync_workers();
  uint32_t key[E];
#pragma unroll
  for (int it = 0; it < E; ++it) {
    const int pos = it * kBlockThreads + tid;
    key[it] = 0u;
    if (pos < n_pos) {
      const int l = pos / maxK, j = pos - l * maxK;
      if (j < sm.cnt[l]) key[it] = max(sortable_u32(ld_f32(ls.v + l * ls.stride + j, SYS)), 1u);
    }
  }
  const Threshold<uint32_t> th = block_select_regs<E>(key, top_k, sm.rsel);
  // classify, then reuse key[] for the id keys of the tied entries
  unsigned long long sure_m = 0ull, tie_m = 0ull;
  int need = 0;
  if (th.need_eq == 0x7fffffff) {
#pragma unroll
    for (int it = 0; it < E; ++it) sure_m |= static_cast<unsigned long long>(key[it] != 0u) << it;
  } else {
#pragma unroll
    for (int it = 0; it < E; ++it) {
      sure_m |= static_cast<unsigned long long>(key[it] > th.tau) << it;
      const bool tied = th.need_eq > 0 && key[it] == th.tau;
      tie_m |= static_cast<unsigned long long>(tied) << it;
    }
    if (th.need_eq > 0) {
#pragma unroll
      for (int it = 0; it < E; ++it) {
        const int pos = it * kBlockThreads + tid;
        uint32_t k2 = 0u;
        if ((tie_m >> it) & 1ull) {
          const int l = pos / maxK, j = pos - l * maxK;
          k2 = ~static_cast<uint32_t>(__float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS)));
          k2 = max(k2, 1u);
        }
        key[it] = k2;
      }
      const Threshold<uint32_t> t2 = block_select_regs<E>(key, th.need_eq, sm.rsel);
      unsigned long long tie2 = 0ull;
#pragma unroll
      for (int it = 0; it < E; ++it) {
        if (t2.need_eq == 0x7fffffff) {
          sure_m |= static_cast<unsigned long long>(key[it] != 0u) << it;
        } else {
          sure_m |= static_cast<unsigned long long>(key[it] > t2.tau) << it;
          tie2 |= static_cast<unsigned long long>(t2.need_eq > 0 && key[it] != 0u && key[it] == t2.tau) << it;
        }
      }
      tie_m = tie2;
      need = (t2.need_eq == 0x7fffffff) ? 0 : t2.need_eq;
    } else {
      tie_m = 0ull;
    }
  }
  int slot[E];
  const int n = block_emit_regs<E>(
      need, sm.rsel, [&](int it) { return ((sure_m >> it) & 1ull) != 0; }, [&](int it) { return ((tie_m >> it) & 1ull) != 0; },
      slot);
#pragma unroll
  for (int it = 0; it < E; ++it) {
    if (slot[it] >= 0 && slot[it] < top_k) {
      const int pos = it * kBlockThreads + tid;
      const int l = pos / maxK, j = pos - l * maxK;
      out_v[slot[it]] = ld_f32(ls.v + l * ls.stride + j, SYS);
      out_i[slot[it]] = __float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS));
    }
  }
  if (tid == 0) {
    *out_c = min(n, top_k);
    if (n != th.n_sel && dbg) atomicAdd(dbg, 1);
  }
  return min(n, top_k);
}

// Stages the padded lists of one row into shared memory: vb[pos] = sortable key
// of the logit (0 = empty position), ib[pos] = id.  The loads carry no branch
// (invalid positions read element 0 of their list and are masked afterwards),
// so a thread's loads of one batch are all in flight together.
template <bool SYS>
__device__ inline void merge_load_counts(const MergeLists& ls, int L, int maxK, MergeSmem& sm) {
  sync_workers();
  for (int l = threadIdx.x; l < L; l += kBlockThreads) {
    const int32_t* cp = ls.c + l * ls.c_stride;
    int c = SYS ? __float_as_int(ld_sys_f32(reinterpret_cast<const float*>(cp))) : *cp;
    sm.cnt[l] = max(0, min(c, maxK));
  }
  sync_workers();
}

// counts must have been loaded (merge_load_counts)
template <bool SYS>
__device__ inline void merge_stage_lists(const MergeLists& ls, int L, int maxK, MergeSmem& sm, uint32_t* vb, int32_t* ib) {
  const int tid = threadIdx.x;
  const int n_pos = L * maxK;
  const bool vec = (maxK & 3) == 0 && (ls.stride & 3) == 0 &&
                   ((reinterpret_cast<uintptr_t>(ls.v) | reinterpret_cast<uintptr_t>(ls.i)) & 15) == 0;
  if (vec) {
    // four consecutive positions of one list per 16-byte load, eight loads of each kind in flight per thread
    constexpr int U = 8;
    const int n_vec = n_pos >> 2, k4 = maxK >> 2;
    for (int q0 = tid; q0 < n_vec; q0 += U * kBlockThreads) {
      float4 v[U];
      int4 f[U];
      int cnt[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int qi = min(q0 + u * kBlockThreads, n_vec - 1);
        const int l = qi / k4, j = (qi - l * k4) << 2;
        cnt[u] = sm.cnt[l] - j;  // valid positions of this quad: those below cnt
        const int64_t off = l * ls.stride + j;
        if (SYS) {  // lists written by peer GPUs: system-scope loads that bypass the L1
          const uint4 a = ld_sys_u4(reinterpret_cast<const uint4*>(ls.v + off));
          const uint4 b = ld_sys_u4(reinterpret_cast<const uint4*>(ls.i + off));
          v[u] = make_float4(__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w));
          f[u] = make_int4(static_cast<int>(b.x), static_cast<int>(b.y), static_cast<int>(b.z), static_cast<int>(b.w));
        } else {
          v[u] = __ldg(reinterpret_cast<const float4*>(ls.v + off));
          f[u] = __ldg(reinterpret_cast<const int4*>(ls.i + off));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int qi = q0 + u * kBlockThreads;
        if (qi < n_vec) {
          uint4 kv;
          kv.x = cnt[u] > 0 ? max(sortable_u32(v[u].x), 1u) : 0u;
          kv.y = cnt[u] > 1 ? max(sortable_u32(v[u].y), 1u) : 0u;
          kv.z = cnt[u] > 2 ? max(sortable_u32(v[u].z), 1u) : 0u;
          kv.w = cnt[u] > 3 ? max(sortable_u32(v[u].w), 1u) : 0u;
          reinterpret_cast<uint4*>(vb)[qi] = kv;
          if (ib) reinterpret_cast<int4*>(ib)[qi] = f[u];
        }
      }
    }
    sync_workers();
    return;
  }
  constexpr int U = 8;
  int l = tid / maxK, j = tid - l * maxK;  // position tid, advanced by 256 per step
  const int dl = kBlockThreads / maxK, dj = kBlockThreads - dl * maxK;
  for (int pos0 = tid; pos0 < n_pos; pos0 += U * kBlockThreads) {
    float v[U], f[U];
    bool ok[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool in = pos0 + u * kBlockThreads < n_pos;
      ok[u] = in && j < sm.cnt[in ? l : 0];
      const int64_t off = ok[u] ? l * ls.stride + j : 0;
      v[u] = ld_f32(ls.v + off, SYS);
      f[u] = ld_f32(reinterpret_cast<const float*>(ls.i) + off, SYS);
      l += dl;
      j += dj;
      if (j >= maxK) {
        j -= maxK;
        ++l;
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int pos = pos0 + u * kBlockThreads;
      if (pos < n_pos) {
        // key 0 marks an empty position; a real logit never maps to 0 after the clamp
        vb[pos] = ok[u] ? max(sortable_u32(v[u]), 1u) : 0u;
        if (ib) ib[pos] = ok[u] ? __float_as_int(f[u]) : 0;
      }
    }
  }
  sync_workers();
}

// Compact staging for lists that are mostly empty (candidates that passed a threshold): only the valid
// entries are staged, list after list, so the search and the emit run over sum(cnt) positions instead
// of L * maxK.  The staged order is the padded order without its holes: same output.  Returns the
// staged length, padded with empty positions to a multiple of four.
template <bool SYS>
__device__ inline int merge_stage_compact(const MergeLists& ls, int L, MergeSmem& sm, uint32_t* vb, int32_t* ib,
                                           bool max_quads_ok = false) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid < 32) {  // exclusive prefix of the counts (L <= 256: eight per lane)
    int c[8], sum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      c[j] = lane * 8 + j < L ? sm.cnt[lane * 8 + j] : 0;
      sum += c[j];
    }
    int total;
    int run = warp_excl_scan(sum, lane, &total);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (lane * 8 + j <= L) sm.off[lane * 8 + j] = run;
      run += c[j];
    }
    if (lane == 31 && L == 256) sm.off[256] = total;
    int qsum = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) qsum += (c[j] + 3) >> 2;
    int qtotal;
    int qrun = warp_excl_scan(qsum, lane, &qtotal);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (lane * 8 + j <= L) sm.qoff[lane * 8 + j] = qrun;
      qrun += (c[j] + 3) >> 2;
    }
    if (lane == 31 && L == 256) sm.qoff[256] = qtotal;
  }
  sync_workers();
  const int n = sm.off[L], n4 = (n + 3) & ~3;
  const bool vec = (ls.stride & 3) == 0 && ((reinterpret_cast<uintptr_t>(ls.v) | reinterpret_cast<uintptr_t>(ls.i)) & 15) == 0 &&
                   max_quads_ok;
  if (vec) {
    // One 16-byte load of each kind per four consecutive entries of a list, eight of each in flight per
    // thread: a row of ~18000 entries from 16 lists is two round trips instead of seventeen.  The last
    // quad of a list may reach past its count (never past the list's padded length): masked below.
    const int nq = sm.qoff[L];
    constexpr int U = 8;
    for (int q0 = tid; q0 < nq; q0 += U * kBlockThreads) {
      int li[U], j[U];
      uint4 a[U], bq[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int q = q0 + u * kBlockThreads;
        li[u] = -1;
        j[u] = 0;
        if (q < nq) {
          int lo = 0, hi = L;  // the list l with qoff[l] <= q < qoff[l + 1]
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (sm.qoff[mid] <= q) lo = mid;
            else hi = mid;
          }
          li[u] = lo;
          j[u] = (q - sm.qoff[lo]) << 2;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t at = li[u] >= 0 ? li[u] * ls.stride + j[u] : 0;
        if (SYS) {
          a[u] = ld_sys_u4(reinterpret_cast<const uint4*>(ls.v + at));
          bq[u] = ld_sys_u4(reinterpret_cast<const uint4*>(ls.i + at));
        } else {
          a[u] = __ldg(reinterpret_cast<const uint4*>(ls.v + at));
          bq[u] = __ldg(reinterpret_cast<const uint4*>(ls.i + at));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (li[u] < 0) continue;
        const int dst = sm.off[li[u]] + j[u], left = sm.cnt[li[u]] - j[u];
        const uint32_t av[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
        const uint32_t bv[4] = {bq[u].x, bq[u].y, bq[u].z, bq[u].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (e < left) {
            vb[dst + e] = max(sortable_u32(__uint_as_float(av[e])), 1u);
            ib[dst + e] = static_cast<int32_t>(bv[e]);
          }
        }
      }
    }
    if (tid < n4 - n) {
      vb[n + tid] = 0u;
      ib[n + tid] = 0;
    }
    sync_workers();
    return n4;
  }
  constexpr int U = 4;  // positions per thread whose loads are in flight together
  for (int pos0 = tid; pos0 < n4; pos0 += U * kBlockThreads) {
    int64_t src[U];
    float v[U], f[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int pos = pos0 + u * kBlockThreads;
      src[u] = -1;
      if (pos < n) {
        int lo = 0, hi = L;  // the list l with off[l] <= pos < off[l + 1]
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (sm.off[mid] <= pos) lo = mid;
          else hi = mid;
        }
        src[u] = lo * ls.stride + (pos - sm.off[lo]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t at = src[u] >= 0 ? src[u] : 0;   // (an empty position reads element 0 and is masked below)
      v[u] = ld_f32(ls.v + at, SYS);
      f[u] = ld_f32(reinterpret_cast<const float*>(ls.i) + at, SYS);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int pos = pos0 + u * kBlockThreads;
      if (pos < n4) {
        vb[pos] = src[u] >= 0 ? max(sortable_u32(v[u]), 1u) : 0u;
        ib[pos] = src[u] >= 0 ? __float_as_int(f[u]) : 0;
      }
    }
  }
  sync_workers();
  return n4;
}

__device__ inline int workers_sum(int x, int32_t* wcnt) {
  x = __reduce_add_sync(0xffffffffu, x);
  sync_workers();
  if ((threadIdx.x & 31) == 0) wcnt[threadIdx.x >> 5] = x;
  sync_workers();
  int t = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) t += wcnt[w];
  return t;
}

__device__ inline float unsortable_f32(uint32_t kv) {
  return __uint_as_float((kv & 0x80000000u) ? (kv ^ 0x80000000u) : ~kv);
}

// Staged rows of up to 256 * E positions: the search runs on register keys (no
// shared-memory traffic per bit; this loop is hot), the position-ordered emit is a
// rolled loop over shared memory.  Work that a block does once per task is bound by
// instruction fetch when it is fully unrolled, so only the hot search is.
template <int E>
__device__ inline int merge_staged_hybrid(int n_pos, int top_k, float* out_v, int32_t* out_i, int32_t* out_c, int32_t* dbg,
                                          MergeSmem& sm, const uint32_t* vb, const int32_t* ib) {
  const int tid = threadIdx.x;
  auto put = [&](int pos, int slot) {
    if (slot < top_k) {
      out_v[slot] = unsortable_f32(vb[pos]);
      out_i[slot] = ib[pos];
    }
  };
  Threshold<uint32_t> th;
  int n_eq = 0;
  {
    uint32_t key[E];
#pragma unroll
    for (int it = 0; it < E; ++it) {
      const int pos = it * kBlockThreads + tid;
      key[it] = pos < n_pos ? vb[pos] : 0u;
    }
    th = block_select_regs<E>(key, top_k, sm.rsel_big);
    if (th.need_eq != 0x7fffffff) {
      int c = 0;
#pragma unroll
      for (int it = 0; it < E; ++it) c += key[it] == th.tau;
      n_eq = workers_sum(c, sm.rsel_big.wcnt);
    }
  }
  const int expect = th.n_sel;
  int n;
  sync_workers();
  if (th.need_eq == 0x7fffffff || n_eq == th.need_eq) {
    n = block_emit_keys(vb, n_pos, th, sm.sel, put);
  } else {
    const uint32_t tau = th.tau;
    auto key2 = [&](int pos) -> uint32_t {
      const uint32_t kv = vb[pos];
      return kv > tau ? 0xffffffffu : (kv == tau ? max(~static_cast<uint32_t>(ib[pos]), 1u) : 0u);
    };
    Threshold<uint32_t> t2;
    {
      uint32_t k2[E];
#pragma unroll
      for (int it = 0; it < E; ++it) {
        const int pos = it * kBlockThreads + tid;
        k2[it] = pos < n_pos ? key2(pos) : 0u;
      }
      t2 = block_select_regs<E>(k2, top_k, sm.rsel_big);
    }
    sync_workers();
    n = block_emit_selected<uint32_t>([&](int pos, bool& valid) { const uint32_t k2 = key2(pos); valid = k2 != 0u; return k2; },
                                      n_pos, t2, sm.sel, put);
  }
  if (tid == 0) {
    *out_c = min(n, top_k);
    if (n != expect && dbg) atomicAdd(dbg, 1);
  }
  return min(n, top_k);
}

// Staged rows of any size: bitwise search over the shared-memory keys.  Ties on
// the logit are resolved in the same search by a second key: entries above the
// logit threshold rank highest, tied entries rank by ~id, everything else is out.
template <typename IdFn>
__device__ inline int merge_staged_bits(int n_pos, int top_k, float* out_v, int32_t* out_i, int32_t* out_c, int32_t* dbg,
                                        MergeSmem& sm, const uint32_t* vb, IdFn id_of, uint32_t* hist = nullptr) {
  const int tid = threadIdx.x;
  int n_eq = 0;
  // hist (2048 words of shared memory) given: the histogram search; else one block-wide pass per bit
  Threshold<uint32_t> th = hist ? block_select_hist_smem(vb, n_pos, top_k, sm.sel, hist, &n_eq)
                                : block_select_bits_smem(vb, n_pos, top_k, sm.sel, &n_eq);
  const int expect = th.n_sel;
  int n;
  auto put = [&](int pos, int slot) {
    if (slot < top_k) {
      out_v[slot] = unsortable_f32(vb[pos]);
      out_i[slot] = id_of(pos);
    }
  };
  if (th.need_eq == 0x7fffffff || n_eq == th.need_eq) {
    // everything valid, or every entry tied at the threshold is taken (distinct logits: the usual case)
    n = block_emit_keys(vb, n_pos, th, sm.sel, put);
  } else {
    const uint32_t tau = th.tau;
    auto key2 = [&](int pos) -> uint32_t {
      const uint32_t kv = vb[pos];
      return kv > tau ? 0xffffffffu : (kv == tau ? max(~static_cast<uint32_t>(id_of(pos)), 1u) : 0u);
    };
    Threshold<uint32_t> t2 = block_select_bits(key2, n_pos, top_k, sm.sel);
    n = block_emit_selected<uint32_t>([&](int pos, bool& valid) { const uint32_t k2 = key2(pos); valid = k2 != 0u; return k2; },
                                      n_pos, t2, sm.sel, put);
  }
  if (tid == 0) {
    *out_c = min(n, top_k);
    if (n != expect && dbg) atomicAdd(dbg, 1);
  }
  return min(n, top_k);
}

// Prefilter of a long staged row: one histogram pass over the top 11 key bits finds the bin that
// holds the k-th largest key; everything below that bin is dropped and the survivors (about k plus one
// bin's worth) are compacted, in position order, into vb2 / ib2.  The exact search and the emit then run
// over the survivors instead of over the whole row.  hist: 2048 words of shared memory; cap: capacity of
// vb2 / ib2.  Returns the compacted length (a multiple of four, padded with empty positions), or -1 when
// the survivors would not fit (heavily tied keys): the caller then works on the full row.
__device__ inline int merge_prefilter(const uint32_t* vb, const int32_t* ib, int n_pos, int top_k, MergeSmem& sm,
                                      uint32_t* hist, uint32_t* vb2, int32_t* ib2, int cap) {
  constexpr int kBins = 2048, kShift = 21;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < kBins; i += kBlockThreads) hist[i] = 0u;
  sync_workers();
  for (int pos = tid; pos < n_pos; pos += kBlockThreads) {
    const uint32_t k = vb[pos];
    if (k) atomicAdd(&hist[k >> kShift], 1u);
  }
  sync_workers();
  // thread t owns the bins kBins-1-8t .. kBins-8-8t, scanned from the top
  uint32_t c[8];
  int local = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c[j] = hist[kBins - 1 - 8 * tid - j];
    local += static_cast<int>(c[j]);
  }
  int wtot;
  int cum = warp_excl_scan(local, lane, &wtot);
  if (lane == 0) sm.sel.wgt[warp] = wtot;
  if (tid == 0) sm.sel.bnd = 0;   // fewer than k keys in all: everything survives
  sync_workers();
  for (int w = 0; w < warp; ++w) cum += sm.sel.wgt[w];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (cum < top_k && cum + static_cast<int>(c[j]) >= top_k) {
      sm.sel.bnd = kBins - 1 - 8 * tid - j;
      sm.sel.c_gt = cum + static_cast<int>(c[j]);   // survivors: keys in the bins >= the boundary bin
    }
    cum += static_cast<int>(c[j]);
  }
  if (tid == kBlockThreads - 1 && cum < top_k) sm.sel.c_gt = cum;   // (all keys: the last thread's running sum is the total)
  sync_workers();
  const uint32_t bin = static_cast<uint32_t>(sm.sel.bnd);
  const int n_keep = sm.sel.c_gt;
  sync_workers();
  if (((n_keep + 3) & ~3) > cap) return -1;
  Threshold<uint32_t> th;
  th.tau = bin ? (bin << kShift) - 1u : 0u;
  th.need_eq = 0;
  th.n_sel = n_keep;
  const int n = block_emit_keys(vb, n_pos, th, sm.sel, [&](int pos, int slot) {
    vb2[slot] = vb[pos];
    ib2[slot] = ib[pos];
  });
  const int n4 = (n + 3) & ~3;
  for (int i = n + tid; i < n4; i += kBlockThreads) {
    vb2[i] = 0u;
    ib2[i] = 0;
  }
  sync_workers();
  return n4;
}

// Picks the fastest path the row size allows: staged in shared memory (when
// `stage` offers 8 bytes per position) with register or shared-memory keys,
// else register keys read from global memory, else re-reading global memory per pass.
template <bool SYS>
__device__ inline int merge_lists_auto(const MergeLists& ls, int L, int maxK, int top_k, float* out_v, int32_t* out_i,
                                       int32_t* out_c, int32_t* dbg, MergeSmem& sm, unsigned char* stage = nullptr,
                                       int stage_bytes = 0) {
  int n_pos = L * maxK;
  int n_valid = -1;
  if (stage && maxK >= 1) {
    merge_load_counts<SYS>(ls, L, maxK, sm);
    n_valid = 0;
    for (int l = 0; l < L; ++l) n_valid += sm.cnt[l];
  }
  const int n_cap = ((n_valid + 3) & ~3) + 4;
  // mostly holes, or too long to stage with its holes: stage the entries only
  const bool compact = n_valid >= 0 && (n_valid * 2 <= n_pos || n_pos * 8 > stage_bytes) && n_cap * 8 <= stage_bytes;
  if (stage && maxK >= 1 && (compact || n_pos * 8 <= stage_bytes)) {
    uint32_t* vb = reinterpret_cast<uint32_t*>(stage);
    int32_t* ib = reinterpret_cast<int32_t*>(stage) + (compact ? n_cap : n_pos);
    if (compact) n_pos = merge_stage_compact<SYS>(ls, L, sm, vb, ib, (maxK & 3) == 0);
    else merge_stage_lists<SYS>(ls, L, maxK, sm, vb, ib);
    {
      // Nothing to select when the lists hold no more than top_k entries between them (one rank's
      // list passing through the cross-rank merge, short contexts): every valid position is
      // emitted, in position order like the general path.
      if (n_valid <= top_k) {
        Threshold<uint32_t> all;
        all.tau = 0u;  // valid keys are >= 1
        all.need_eq = 0;
        all.n_sel = n_valid;
        all.need_eq = 0x7fffffff;
        const int n = block_emit_keys(
            vb, n_pos, all, sm.sel,
            [&](int pos, int slot) {
              if (slot < top_k) {
                out_v[slot] = unsortable_f32(vb[pos]);
                out_i[slot] = ib[pos];
              }
            });
        if (threadIdx.x == 0) {
          *out_c = n;
          if (n != n_valid && dbg) atomicAdd(dbg, 1);
        }
        return n;
      }
    }
    const int used = (compact ? n_cap : n_pos) * 8;
    // room behind the staged row for a 2048-word histogram: the histogram search instead of one pass per bit
    uint32_t* hist = stage_bytes - used >= 2048 * 4 ? reinterpret_cast<uint32_t*>(stage + used) : nullptr;
    // a long row (several full lists): one histogram pass drops what cannot reach the top k, and every later
    // pass (search, emit) runs over about k survivors instead of the whole row
    const int cap = ((stage_bytes - used - 2048 * 4) / 8) & ~3;
    // (worth its fixed cost from about four lists' worth: measured 26.8 against 23.7 us at 2.6 x top_k candidates)
    if (n_valid >= 4 * top_k && n_pos % 4 == 0 && cap >= top_k + 4) {
      uint32_t* vb2 = hist + 2048;
      int32_t* ib2 = reinterpret_cast<int32_t*>(vb2) + cap;
      const int n2 = merge_prefilter(vb, ib, n_pos, top_k, sm, hist, vb2, ib2, cap);
      if (n2 >= 0)
        return merge_staged_bits(n2, top_k, out_v, out_i, out_c, dbg, sm, vb2, [&](int pos) { return ib2[pos]; }, hist);
    }
    if (hist)
      return merge_staged_bits(n_pos, top_k, out_v, out_i, out_c, dbg, sm, vb, [&](int pos) { return ib[pos]; }, hist);
    return merge_staged_bits(n_pos, top_k, out_v, out_i, out_c, dbg, sm, vb, [&](int pos) { return ib[pos]; });
  }
  if (stage && n_pos * 4 <= stage_bytes && maxK >= 1) {
    // too long for keys + ids: stage the keys only, fetch the few ids that are needed from global memory
    uint32_t* vb = reinterpret_cast<uint32_t*>(stage);
    merge_stage_lists<SYS>(ls, L, maxK, sm, vb, nullptr);
    return merge_staged_bits(n_pos, top_k, out_v, out_i, out_c, dbg, sm, vb, [&](int pos) {
      const int l = pos / maxK, j = pos - l * maxK;
      return __float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS));
    });
  }
  if (n_pos <= kBlockThreads * kMergeRegE)
    return merge_lists_regs<kMergeRegE, SYS>(ls, L, maxK, top_k, out_v, out_i, out_c, dbg, sm);
  return merge_lists_tile<SYS>(ls, L, maxK, top_k, out_v, out_i, out_c, dbg, sm);
}

// stage = optional dynamic shared memory of stage_bytes for the shared-memory path
__device__ inline void merge_topk_tile(const mdc_merge_topk_params& p, int row, MergeSmem& sm, unsigned char* stage = nullptr,
                                       int stage_bytes = 0) {
  MergeLists ls;
  const int64_t base = static_cast<int64_t>(row) * p.L * p.maxK;
  ls.v = p.cand_v + base;
  ls.i = p.cand_i + base;
  ls.c = p.cand_c + static_cast<int64_t>(row) * p.L;
  ls.stride = p.maxK;
  ls.c_stride = 1;
  merge_lists_auto<false>(ls, p.L, p.maxK, p.top_k, p.out_v + static_cast<int64_t>(row) * p.top_k,
                          p.out_i + static_cast<int64_t>(row) * p.top_k, p.out_c + row, p.dbg, sm, stage, stage_bytes);
}


}  // namespace mdc
