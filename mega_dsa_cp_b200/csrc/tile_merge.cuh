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

namespace mdc {

constexpr int kMergeMaxLists = 256;

struct MergeSmem {
  SelectScratch sel;
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

__device__ inline void merge_topk_tile(const mdc_merge_topk_params& p, int row, MergeSmem& sm) {
  MergeLists ls;
  const int64_t base = static_cast<int64_t>(row) * p.L * p.maxK;
  ls.v = p.cand_v + base;
  ls.i = p.cand_i + base;
  ls.c = p.cand_c + static_cast<int64_t>(row) * p.L;
  ls.stride = p.maxK;
  ls.c_stride = 1;
  merge_lists_tile<false>(ls, p.L, p.maxK, p.top_k, p.out_v + static_cast<int64_t>(row) * p.top_k,
                          p.out_i + static_cast<int64_t>(row) * p.top_k, p.out_c + row, p.dbg, sm);
}


}  // namespace mdc
