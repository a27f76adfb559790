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

struct MergeSmem {
  union {
    SelectScratch sel;
    RegSelectScratch<kMergeRegE> rsel;
  };
  int32_t cnt[kMergeMaxLists];
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

// Shared-memory path for rows of up to `cap` positions: logits and ids are
// staged once (vb / ib, `cap` words each), selected by bitwise search, and
// emitted from shared memory.  Ties on the logit are resolved in the same
// search by a second key: entries above the logit threshold rank highest, tied
// entries rank by ~id, everything else is out.
template <bool SYS>
__device__ inline int merge_lists_smem(const MergeLists& ls, int L, int maxK, int top_k, float* out_v, int32_t* out_i,
                                       int32_t* out_c, int32_t* dbg, MergeSmem& sm, uint32_t* vb, int32_t* ib) {
  const int tid = threadIdx.x;
  const int n_pos = L * maxK;
  sync_workers();
  for (int l = tid; l < L; l += kBlockThreads) {
    const int32_t* cp = ls.c + l * ls.c_stride;
    int c = SYS ? __float_as_int(ld_sys_f32(reinterpret_cast<const float*>(cp))) : *cp;
    sm.cnt[l] = max(0, min(c, maxK));
  }
  sync_workers();
  for (int pos = tid; pos < n_pos; pos += kBlockThreads) {
    const int l = pos / maxK, j = pos - l * maxK;
    const bool valid = j < sm.cnt[l];
    // key 0 marks an empty position; a real logit never maps to 0 after the clamp
    vb[pos] = valid ? max(sortable_u32(ld_f32(ls.v + l * ls.stride + j, SYS)), 1u) : 0u;
    ib[pos] = valid ? __float_as_int(ld_f32(reinterpret_cast<const float*>(ls.i + l * ls.stride + j), SYS)) : 0;
  }
  sync_workers();
  Threshold<uint32_t> th = block_select_bits([&](int pos) { return vb[pos]; }, n_pos, top_k, sm.sel);
  const int expect = th.n_sel;
  int n;
  auto put = [&](int pos, int slot) {
    if (slot < top_k) {
      const uint32_t kv = vb[pos];
      out_v[slot] = __uint_as_float((kv & 0x80000000u) ? (kv ^ 0x80000000u) : ~kv);
      out_i[slot] = ib[pos];
    }
  };
  if (th.need_eq == 0x7fffffff) {
    n = block_emit_selected<uint32_t>([&](int pos, bool& valid) { valid = vb[pos] != 0u; return vb[pos]; }, n_pos, th,
                                      sm.sel, put);
  } else {
    const uint32_t tau = th.tau;
    auto key2 = [&](int pos) -> uint32_t {
      const uint32_t kv = vb[pos];
      return kv > tau ? 0xffffffffu : (kv == tau ? max(~static_cast<uint32_t>(ib[pos]), 1u) : 0u);
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

// picks the fastest path the row size allows: registers, shared memory (when
// `stage` offers 8 bytes per position), else re-reading global memory per pass
template <bool SYS>
__device__ inline int merge_lists_auto(const MergeLists& ls, int L, int maxK, int top_k, float* out_v, int32_t* out_i,
                                       int32_t* out_c, int32_t* dbg, MergeSmem& sm, unsigned char* stage = nullptr,
                                       int stage_bytes = 0) {
  const int n_pos = L * maxK;
  if (n_pos <= kBlockThreads * kMergeRegE)
    return merge_lists_regs<kMergeRegE, SYS>(ls, L, maxK, top_k, out_v, out_i, out_c, dbg, sm);
  if (stage && n_pos * 8 <= stage_bytes)
    return merge_lists_smem<SYS>(ls, L, maxK, top_k, out_v, out_i, out_c, dbg, sm, reinterpret_cast<uint32_t*>(stage),
                                 reinterpret_cast<int32_t*>(stage) + n_pos);
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
