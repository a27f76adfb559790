// Launch wrapper of the indexer-logits tile (see tile_logits.cuh).
#include "tile_logits.cuh"

namespace mdc {

template <int FMT, int PAGE, int T>
__global__ void __launch_bounds__(kLogitsThreads, 1) logits_kernel(const __grid_constant__ mdc_logits_params p) {
  extern __shared__ unsigned char smem_raw[];
  // the UMMA operand block wants a 1024-byte aligned base
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  logits_tile<FMT, PAGE, T, kLogitsDecodeGroups, kLogitsGateGroups>(p, blockIdx.y, blockIdx.x, smem);
}

// Row mode: the blocks of one request form a cluster and select across their chunks.
template <int FMT, int PAGE, int T>
__global__ void __launch_bounds__(kLogitsThreads, 1) logits_row_kernel(const __grid_constant__ mdc_logits_params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  logits_tile<FMT, PAGE, T, kLogitsDecodeGroups, kLogitsGateGroups, true>(p, blockIdx.y, blockIdx.x, smem);
}

template <int FMT, int PAGE, int T>
static int launch_logits_row(const mdc_logits_params& p, cudaStream_t st, int smem) {
  auto kern = logits_row_kernel<FMT, PAGE, T>;
  MDC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_chunks, p.B);
  cfg.blockDim = dim3(kLogitsThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.n_chunks;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MDC_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p));
  return MDC_OK;
}

template <int FMT, int PAGE, int T>
static int launch_logits(const mdc_logits_params& p, cudaStream_t st, int smem) {
  if (p.row_v) return launch_logits_row<FMT, PAGE, T>(p, st, smem);
  auto kern = logits_kernel<FMT, PAGE, T>;
  MDC_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid(p.n_chunks, p.B);
  kern<<<grid, kLogitsThreads, smem, st>>>(p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

int logits_check(const mdc_logits_params* p) {
  if (!p) return MDC_ERR_NULL;
  if (!p->kv_pages || !p->q || !p->weights || !p->block_table) return MDC_ERR_NULL;
  if (p->fmt != MDC_FMT_MXFP4 && p->fmt != MDC_FMT_NVFP4) return MDC_ERR_BAD_FORMAT;
  if (p->q_fmt != MDC_Q_FP4 && p->q_fmt != MDC_Q_BF16) return MDC_ERR_BAD_FORMAT;
  if (p->q_fmt == MDC_Q_FP4 && !p->q_sf) return MDC_ERR_NULL;
  if (p->page_tokens != 64 && p->page_tokens != 128) return MDC_ERR_BAD_SHAPE;
  if (p->fmt == MDC_FMT_MXFP4 && p->page_tokens != 128) return MDC_ERR_BAD_SHAPE;
  if (p->heads != kIdxHeads || (p->q_len != 1 && p->q_len != 2)) return MDC_ERR_BAD_SHAPE;
  if (p->B < 1 || p->n_chunks < 1 || p->blocks_per_chunk < 1 || p->max_pages < 1) return MDC_ERR_BAD_SHAPE;
  if (p->n_chunks > 65535 * 32 || p->B > 65535) return MDC_ERR_BAD_SHAPE;
  const bool fused = p->cand_v != nullptr && !p->row_v;
  if (p->row_v) {
    if (!p->row_i || !p->row_c) return MDC_ERR_NULL;
    if (p->top_k < 1 || p->id_mul < 1) return MDC_ERR_BAD_SHAPE;
    if (p->n_chunks != 1 && p->n_chunks != 2 && p->n_chunks != 4 && p->n_chunks != 8) return MDC_ERR_BAD_SHAPE;
    if (p->blocks_per_chunk * p->page_tokens > kBlockThreads * kFusedRegE) return MDC_ERR_TOO_LARGE;
  } else if (fused) {
    if (!p->cand_i || !p->cand_c) return MDC_ERR_NULL;
    if (p->top_k < 1) return MDC_ERR_BAD_SHAPE;
    if (p->id_mul < 1) return MDC_ERR_BAD_SHAPE;
  } else if (!p->logits) {
    return MDC_ERR_NULL;
  }
  if (reinterpret_cast<uintptr_t>(p->kv_pages) & 15) return MDC_ERR_BAD_ALIGN;
  if (reinterpret_cast<uintptr_t>(p->q) & 7) return MDC_ERR_BAD_ALIGN;
  return MDC_OK;
}

static int logits_smem(const mdc_logits_params* p) {
  const bool fused = p->cand_v != nullptr || p->row_v != nullptr;
  const int ct = p->blocks_per_chunk * p->page_tokens;
  int total;
  if (p->fmt == MDC_FMT_MXFP4) total = logits_smem_layout<MDC_FMT_MXFP4, 128>(p->q_len, ct, fused).total;
  else if (p->page_tokens == 64) total = logits_smem_layout<MDC_FMT_NVFP4, 64>(p->q_len, ct, fused).total;
  else total = logits_smem_layout<MDC_FMT_NVFP4, 128>(p->q_len, ct, fused).total;
  // slack for the 1024-byte alignment of the base; at least 116 KB so that one
  // block owns an SM (each block allocates all of the SM's tensor memory)
  total += 1024;
  return total < 116 * 1024 ? 116 * 1024 : total;
}

}  // namespace mdc

extern "C" int mdc_logits_fp4_smem_bytes(const mdc_logits_params* p) {
  int rc = mdc::logits_check(p);
  if (rc != MDC_OK) return rc;
  return mdc::logits_smem(p);
}

extern "C" int mdc_logits_fp4_launch(const mdc_logits_params* p, void* stream) {
  using namespace mdc;
  int rc = logits_check(p);
  if (rc != MDC_OK) return rc;
  const int smem = logits_smem(p);
  if (smem > 227 * 1024) return MDC_ERR_TOO_LARGE;  // chunk too long to keep its scores on chip
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int key = (p->fmt == MDC_FMT_MXFP4 ? 0 : (p->page_tokens == 64 ? 1 : 2)) * 2 + (p->q_len - 1);
  switch (key) {
    case 0: return launch_logits<MDC_FMT_MXFP4, 128, 1>(*p, st, smem);
    case 1: return launch_logits<MDC_FMT_MXFP4, 128, 2>(*p, st, smem);
    case 2: return launch_logits<MDC_FMT_NVFP4, 64, 1>(*p, st, smem);
    case 3: return launch_logits<MDC_FMT_NVFP4, 64, 2>(*p, st, smem);
    case 4: return launch_logits<MDC_FMT_NVFP4, 128, 1>(*p, st, smem);
    default: return launch_logits<MDC_FMT_NVFP4, 128, 2>(*p, st, smem);
  }
}

int mdc_attrs_logits(cudaFuncAttributes* a) {
  return static_cast<int>(cudaFuncGetAttributes(a, mdc::logits_kernel<MDC_FMT_NVFP4, 64, 1>));
}
