// Launch wrapper of the LSE-merge tile (see tile_lse_merge.cuh).
#include "tile_lse_merge.cuh"

namespace mdc {
constexpr int kLseHeadsPerBlock = 16;

__global__ void __launch_bounds__(kBlockThreads) lse_merge_kernel(const __grid_constant__ mdc_lse_merge_params p) {
  __shared__ float scale[kLseMaxSlices * kLseHeadsPerBlock];
  const int h0 = blockIdx.y * kLseHeadsPerBlock;
  lse_merge_tile<false>(p, blockIdx.x, h0, min(kLseHeadsPerBlock, p.H - h0), scale);
}
}  // namespace mdc

extern "C" int mdc_lse_merge_launch(const mdc_lse_merge_params* p, void* stream) {
  using namespace mdc;
  if (!p || !p->acc_o || !p->acc_lse || !p->o) return MDC_ERR_NULL;
  if (p->rows < 1 || p->H < 1 || p->D < 8 || p->D % 8) return MDC_ERR_BAD_SHAPE;
  if (p->n_slices < 1 || p->n_slices > p->n_slices_max || p->n_slices > kLseMaxSlices) return MDC_ERR_BAD_SHAPE;
  if (p->acc_dtype != MDC_DT_F32 && p->acc_dtype != MDC_DT_BF16) return MDC_ERR_BAD_FORMAT;
  if (p->out_dtype != MDC_DT_F32 && p->out_dtype != MDC_DT_BF16) return MDC_ERR_BAD_FORMAT;
  if ((reinterpret_cast<uintptr_t>(p->acc_o) | reinterpret_cast<uintptr_t>(p->o)) & 15) return MDC_ERR_BAD_ALIGN;
  dim3 grid(p->rows, ceil_div(p->H, kLseHeadsPerBlock));
  lse_merge_kernel<<<grid, kBlockThreads, 0, static_cast<cudaStream_t>(stream)>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int mdc_attrs_lse_merge(cudaFuncAttributes* a) {
  return static_cast<int>(cudaFuncGetAttributes(a, mdc::lse_merge_kernel));
}
