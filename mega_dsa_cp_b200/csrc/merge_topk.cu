// Launch wrapper of the candidate-merge tile (see tile_merge.cuh).
#include "tile_merge.cuh"

namespace mdc {
constexpr int kMergeStageMax = 200 * 1024;  // rows of up to 25600 positions are staged in shared memory
constexpr int kMergeHistBytes = 2048 * 4;    // behind a staged row: the histogram of the threshold search
__global__ void __launch_bounds__(kBlockThreads) merge_topk_kernel(const __grid_constant__ mdc_merge_topk_params p) {
  __shared__ MergeSmem sm;
  extern __shared__ __align__(16) unsigned char stage[];
  const int n_pos = p.L * p.maxK;
  const int need = n_pos * 8 <= kMergeStageMax ? n_pos * 8 + kMergeHistBytes : (n_pos * 4 <= kMergeStageMax ? n_pos * 4 : 0);
  merge_topk_tile(p, blockIdx.x, sm, need ? stage : nullptr, need);
}
}  // namespace mdc

extern "C" int mdc_merge_topk_launch(const mdc_merge_topk_params* p, void* stream) {
  using namespace mdc;
  if (!p || !p->cand_v || !p->cand_i || !p->cand_c || !p->out_v || !p->out_i || !p->out_c) return MDC_ERR_NULL;
  if (p->B < 1 || p->q_len < 1 || p->L < 1 || p->L > kMergeMaxLists || p->maxK < 1 || p->top_k < 1)
    return MDC_ERR_BAD_SHAPE;
  if (static_cast<int64_t>(p->L) * p->maxK > (1ll << 30)) return MDC_ERR_TOO_LARGE;
  const int64_t n_pos = static_cast<int64_t>(p->L) * p->maxK;
  const int smem = n_pos * 8 <= kMergeStageMax ? static_cast<int>(n_pos * 8) + kMergeHistBytes
                                               : (n_pos * 4 <= kMergeStageMax ? static_cast<int>(n_pos * 4) : 0);
  MDC_CUDA_OK(cudaFuncSetAttribute(merge_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMergeStageMax + kMergeHistBytes));
  merge_topk_kernel<<<p->B * p->q_len, kBlockThreads, smem, static_cast<cudaStream_t>(stream)>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int mdc_attrs_merge_topk(cudaFuncAttributes* a) {
  return static_cast<int>(cudaFuncGetAttributes(a, mdc::merge_topk_kernel));
}
