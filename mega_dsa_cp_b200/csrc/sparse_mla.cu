// Launch wrapper of the sparse-MLA tile (see tile_mla.cuh) and of the split
// combine that follows it when the slot range is split.
#include "tile_mla.cuh"
#include "tile_mla_umma.cuh"
#include "tile_lse_merge.cuh"

namespace mdc {

template <int DQK, int KVDT>
__global__ void __launch_bounds__(kBlockThreads, 1) mla_kernel(const __grid_constant__ mdc_sparse_mla_params p) {
  extern __shared__ __align__(128) unsigned char smem[];
  mla_tile<DQK, KVDT>(p, blockIdx.z, blockIdx.y, blockIdx.x, gridDim.x, smem);
}

__global__ void __launch_bounds__(kBlockThreads) mla_combine_kernel(const __grid_constant__ mdc_lse_merge_params p) {
  __shared__ float scale[kLseMaxSlices * 16];
  const int h0 = blockIdx.y * 16;
  lse_merge_tile<false>(p, blockIdx.x, h0, min(16, p.H - h0), scale);
}

// tcgen05 path: bf16 operands, blocks of 128 heads x 128 output columns
template <int DQK>
__global__ void __launch_bounds__(kMuThreads, 1) mla_umma_kernel(const __grid_constant__ mdc_sparse_mla_params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int hb = blockIdx.y >> 2, dq = blockIdx.y & 3;
  mla_umma_tile<DQK>(p, blockIdx.z, hb, dq, blockIdx.x, gridDim.x, smem);
}

template <int DQK>
static int launch_mla_umma(const mdc_sparse_mla_params& p, cudaStream_t st) {
  auto kern = mla_umma_kernel<DQK>;
  const int smem = MlaUmmaSmem<DQK>::kTotal + 1024;
  MDC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.n_splits, (p.H / kMuHeads) * (kMlaDv / kMuDv), p.B * p.q_len);
  kern<<<grid, kMuThreads, smem, st>>>(p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

// The tensor-memory path takes bf16 operands with heads in blocks of 128 and exact (unrounded) probabilities.
static bool mla_use_umma(const mdc_sparse_mla_params& p) {
  return p.kv_dtype == MDC_DT_BF16 && p.H % kMuHeads == 0 && p.fp8_p == 0;
}

template <int DQK, int KVDT>
static int launch_mla(const mdc_sparse_mla_params& p, cudaStream_t st) {
  auto kern = mla_kernel<DQK, KVDT>;
  const int smem = MlaSmem<DQK>::kTotal;
  MDC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.n_splits, p.H / kMlaHeads, p.B * p.q_len);
  kern<<<grid, kBlockThreads, smem, st>>>(p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int mla_check(const mdc_sparse_mla_params* p) {
  if (!p || !p->q || !p->kv_cmp || !p->pt_cmp || !p->k_valid || !p->o) return MDC_ERR_NULL;
  if (p->B < 1 || p->q_len < 1 || p->H < kMlaHeads || p->H % kMlaHeads) return MDC_ERR_BAD_SHAPE;
  if (p->d_v != kMlaDv || (p->d_qk != 576 && p->d_qk != 512)) return MDC_ERR_BAD_SHAPE;
  if (p->page_cmp < 1 || p->pt_cols < 1 || p->pages_cmp < 1) return MDC_ERR_BAD_SHAPE;
  if (p->kv_dtype != MDC_DT_BF16 && p->kv_dtype != MDC_DT_E4M3) return MDC_ERR_BAD_FORMAT;
  if (p->out_dtype != MDC_DT_F32 && p->out_dtype != MDC_DT_BF16) return MDC_ERR_BAD_FORMAT;
  if (p->n_splits < 1 || p->n_splits > kLseMaxSlices) return MDC_ERR_BAD_SHAPE;
  if (p->n_splits > 1) {
    if (!p->ws_o || !p->ws_lse) return MDC_ERR_NULL;
    if (p->o_stride != static_cast<int64_t>(p->H) * p->d_v) return MDC_ERR_BAD_SHAPE;
    if (p->lse && p->lse_stride != p->H) return MDC_ERR_BAD_SHAPE;
  }
  if (p->kv_win && p->pages_win < 1) return MDC_ERR_BAD_SHAPE;
  uintptr_t all = reinterpret_cast<uintptr_t>(p->q) | reinterpret_cast<uintptr_t>(p->kv_cmp) |
                  reinterpret_cast<uintptr_t>(p->kv_win) | reinterpret_cast<uintptr_t>(p->o) |
                  reinterpret_cast<uintptr_t>(p->ws_o);
  if (all & 15) return MDC_ERR_BAD_ALIGN;
  if ((p->o_stride * (p->out_dtype == MDC_DT_F32 ? 4 : 2)) & 7) return MDC_ERR_BAD_ALIGN;
  return MDC_OK;
}

}  // namespace mdc

extern "C" int mdc_sparse_mla_smem_bytes(const mdc_sparse_mla_params* p) {
  int rc = mdc::mla_check(p);
  if (rc != MDC_OK) return rc;
  if (mdc::mla_use_umma(*p))  // the tile the launch will take (+ slack for its 1024-byte aligned base)
    return (p->d_qk == 576 ? mdc::MlaUmmaSmem<576>::kTotal : mdc::MlaUmmaSmem<512>::kTotal) + 1024;
  return p->d_qk == 576 ? mdc::MlaSmem<576>::kTotal : mdc::MlaSmem<512>::kTotal;
}

extern "C" int mdc_sparse_mla_launch(const mdc_sparse_mla_params* p, void* stream) {
  using namespace mdc;
  int rc = mla_check(p);
  if (rc != MDC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (mla_use_umma(*p)) rc = p->d_qk == 576 ? launch_mla_umma<576>(*p, st) : launch_mla_umma<512>(*p, st);
  else if (p->d_qk == 576 && p->kv_dtype == MDC_DT_BF16) rc = launch_mla<576, MDC_DT_BF16>(*p, st);
  else if (p->d_qk == 512 && p->kv_dtype == MDC_DT_BF16) rc = launch_mla<512, MDC_DT_BF16>(*p, st);
  else if (p->d_qk == 576) rc = launch_mla<576, MDC_DT_E4M3>(*p, st);
  else rc = launch_mla<512, MDC_DT_E4M3>(*p, st);
  if (rc != MDC_OK || p->n_splits == 1) return rc;
  mdc_lse_merge_params m;
  m.acc_o = p->ws_o;
  m.acc_lse = p->ws_lse;
  m.o = p->o;
  m.lse = p->lse;
  m.rows = p->B * p->q_len;
  m.H = p->H;
  m.D = p->d_v;
  m.n_slices = m.n_slices_max = p->n_splits;
  m.acc_dtype = MDC_DT_F32;
  m.out_dtype = p->out_dtype;
  dim3 grid(m.rows, ceil_div(m.H, 16));
  mla_combine_kernel<<<grid, kBlockThreads, 0, st>>>(m);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int mdc_attrs_sparse_mla(cudaFuncAttributes* a) {
  return static_cast<int>(cudaFuncGetAttributes(a, mdc::mla_kernel<576, MDC_DT_BF16>));
}
