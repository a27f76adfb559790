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

__device__ inline void merge_topk_tile(const mdc_merge_topk_params& p, int row, MergeSmem& sm) {
  const int tid = threadIdx.x;
  const int L = p.L, maxK = p.maxK;
  const int64_t base = static_cast<int64_t>(row) * L * maxK;
  const float* cv = p.cand_v + base;
  const int32_t* ci = p.cand_i + base;
  sync_workers();
  for (int l = tid; l < L; l += kBlockThreads) {
    int c = p.cand_c[static_cast<int64_t>(row) * L + l];
    sm.cnt[l] = max(0, min(c, maxK));
  }
  sync_workers();
  auto src = [&](int pos, bool& valid) -> unsigned long long {
    const int l = pos / maxK, j = pos - l * maxK;
    valid = j < sm.cnt[l];
    if (!valid) return 0ull;
    const uint32_t hi = sortable_u32(__ldg(cv + pos));
    const uint32_t lo = ~static_cast<uint32_t>(__ldg(ci + pos));
    return (static_cast<unsigned long long>(hi) << 32) | lo;
  };
  const int n_pos = L * maxK;
  Threshold<unsigned long long> th = block_select_threshold<unsigned long long>(src, n_pos, p.top_k, sm.sel);
  float* ov = p.out_v + static_cast<int64_t>(row) * p.top_k;
  int32_t* oi = p.out_i + static_cast<int64_t>(row) * p.top_k;
  const int top_k = p.top_k;
  int n = block_emit_selected<unsigned long long>(src, n_pos, th, sm.sel, [&](int pos, int slot) {
    if (slot < top_k) {
      ov[slot] = cv[pos];
      oi[slot] = ci[pos];
    }
  });
  if (tid == 0) {
    p.out_c[row] = min(n, top_k);
    if (n != th.n_sel && p.dbg) atomicAdd(p.dbg, 1);
  }
}

}  // namespace mdc
