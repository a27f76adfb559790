// Launch wrapper of the candidate-merge tile (see tile_merge.cuh).
#include "tile_merge.cuh"

namespace mdc {
__global__ void __launch_bounds__(kBlockThreads) merge_topk_kernel(const __grid_constant__ mdc_merge_topk_params p) {
  __shared__ MergeSmem sm;
  merge_topk_tile(p, blockIdx.x, sm);
}
}  // namespace mdc

extern "C" int mdc_merge_topk_launch(const mdc_merge_topk_params* p, void* stream) {
  using namespace mdc;
  if (!p || !p->cand_v || !p->cand_i || !p->cand_c || !p->out_v || !p->out_i || !p->out_c) return MDC_ERR_NULL;
  if (p->B < 1 || p->q_len < 1 || p->L < 1 || p->L > kMergeMaxLists || p->maxK < 1 || p->top_k < 1)
    return MDC_ERR_BAD_SHAPE;
  if (static_cast<int64_t>(p->L) * p->maxK > (1ll << 30)) return MDC_ERR_TOO_LARGE;
  merge_topk_kernel<<<p->B * p->q_len, kBlockThreads, 0, static_cast<cudaStream_t>(stream)>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int mdc_attrs_merge_topk(cudaFuncAttributes* a) {
  return static_cast<int>(cudaFuncGetAttributes(a, mdc::merge_topk_kernel));
}
