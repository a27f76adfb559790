// Launch wrappers of the KV-compressor tiles (see tile_compress.cuh): one block of 256 threads per sequence.
#include "tile_compress.cuh"

namespace mdc {

__global__ void __launch_bounds__(kBlockThreads) csa_step_kernel(const __grid_constant__ mdc_compress_params p) {
  __shared__ __align__(16) float stage[kCsaStatsF];
  csa_step_tile<true>(p, blockIdx.x, stage);
}
__global__ void __launch_bounds__(kBlockThreads) online_step_kernel(const __grid_constant__ mdc_compress_params p) {
  __shared__ __align__(16) float stage[kOnlStatsF];
  online_step_tile<true>(p, blockIdx.x, stage);
}
__global__ void __launch_bounds__(kBlockThreads) csa_finalize_kernel(const __grid_constant__ mdc_compress_params p) {
  __shared__ FinalizeSmem sm;
  csa_finalize_tile<true>(p, blockIdx.x, sm);
}
__global__ void __launch_bounds__(kBlockThreads) online_finalize_kernel(const __grid_constant__ mdc_compress_params p) {
  __shared__ FinalizeSmem sm;
  online_finalize_tile<true>(p, blockIdx.x, sm);
}
__global__ void __launch_bounds__(32) hadamard_quant_kernel(const float* x, uint8_t* out) {
  const float* row = x + static_cast<int64_t>(blockIdx.x) * kHdIdx;
  uint8_t* o = out + static_cast<int64_t>(blockIdx.x) * 68;
  hadamard_quant_warp(row, o, o + 64, MDC_FMT_MXFP4);
}

int compress_check(const mdc_compress_params* p, bool finalize) {
  if (!p || !p->seq_len || !p->arena.base || !p->arena.offsets || !p->events.base || !p->events.offsets) return MDC_ERR_NULL;
  // one new record per rank per step: at most cp positions per step
  if (p->B < 1 || p->cp < 1 || p->rank < 0 || p->rank >= p->cp || p->q_len < 1 || p->q_len > p->cp) return MDC_ERR_BAD_SHAPE;
  if (p->ratio != 4 && p->ratio != 64 && p->ratio != 128) return MDC_ERR_BAD_SHAPE;
  if (!finalize) {
    if (!p->new_attn || !p->ape_attn) return MDC_ERR_NULL;
    if (p->ratio == 4 && (!p->ring_attn || !p->ring_idx || !p->new_idx || !p->ape_idx)) return MDC_ERR_NULL;
    if (p->ratio != 4 && !p->state) return MDC_ERR_NULL;
  } else {
    if (!p->norm_w_attn || !p->freqs || !p->attn_pool) return MDC_ERR_NULL;
    if (p->ratio == 4 && !p->norm_w_idx) return MDC_ERR_NULL;
    if (p->attn_pool_dtype != MDC_DT_E4M3 && p->attn_pool_dtype != MDC_DT_BF16) return MDC_ERR_BAD_FORMAT;
    if (p->max_entries < 1 || p->wait_budget_ns <= 0) return MDC_ERR_BAD_SHAPE;
    if (p->ratio == 4 && p->idx_pool) {
      if (p->idx_fmt != MDC_FMT_MXFP4 && p->idx_fmt != MDC_FMT_NVFP4) return MDC_ERR_BAD_FORMAT;
      if (p->idx_page_tokens != 64 && p->idx_page_tokens != 128) return MDC_ERR_BAD_SHAPE;
      if (p->idx_fmt == MDC_FMT_MXFP4 && p->idx_page_tokens != 128) return MDC_ERR_BAD_SHAPE;
      if (p->max_entries % p->idx_page_tokens) return MDC_ERR_BAD_SHAPE;
    }
  }
  if (p->ratio == 4 && p->ring_slots != 0 && p->ring_slots * p->cp < 8) return MDC_ERR_BAD_SHAPE;  // the window holds 8 tokens
  if (p->stats_off & 15) return MDC_ERR_BAD_ALIGN;
  return MDC_OK;
}

}  // namespace mdc

extern "C" int mdc_compress_step_launch(const mdc_compress_params* p, void* stream) {
  using namespace mdc;
  int rc = compress_check(p, false);
  if (rc != MDC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->ratio == 4) csa_step_kernel<<<p->B, kBlockThreads, 0, st>>>(*p);
  else online_step_kernel<<<p->B, kBlockThreads, 0, st>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

extern "C" int mdc_compress_finalize_launch(const mdc_compress_params* p, void* stream) {
  using namespace mdc;
  int rc = compress_check(p, true);
  if (rc != MDC_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (p->ratio == 4) csa_finalize_kernel<<<p->B, kBlockThreads, 0, st>>>(*p);
  else online_finalize_kernel<<<p->B, kBlockThreads, 0, st>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

extern "C" int mdc_hadamard_quant_launch(const float* x, uint8_t* out, int32_t n, void* stream) {
  if (!x || !out) return MDC_ERR_NULL;
  if (n < 1) return MDC_ERR_BAD_SHAPE;
  mdc::hadamard_quant_kernel<<<n, 32, 0, static_cast<cudaStream_t>(stream)>>>(x, out);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}
