// Library-wide C-ABI helpers: version, status strings, last CUDA error.
#include "common.cuh"

static thread_local int g_last_cuda_error = 0;

extern "C" void mdc_set_last_cuda_error(int e) { g_last_cuda_error = e; }
extern "C" int mdc_last_cuda_error(void) { return g_last_cuda_error; }
extern "C" int mdc_abi_version(void) { return MDC_ABI_VERSION; }

extern "C" const char* mdc_status_string(int code) {
  switch (code) {
    case MDC_OK: return "ok";
    case MDC_ERR_BAD_SHAPE: return "unsupported shape or count";
    case MDC_ERR_BAD_ALIGN: return "pointer or stride not aligned";
    case MDC_ERR_BAD_FORMAT: return "unknown format or dtype";
    case MDC_ERR_NULL: return "required pointer is null";
    case MDC_ERR_CUDA: return "CUDA runtime error (see mdc_last_cuda_error)";
    case MDC_ERR_TOO_LARGE: return "size exceeds a stated capacity";
    default: return "unknown status";
  }
}

int mdc_attrs_logits(cudaFuncAttributes* a);
int mdc_attrs_merge_topk(cudaFuncAttributes* a);
int mdc_attrs_lse_merge(cudaFuncAttributes* a);
int mdc_attrs_sparse_mla(cudaFuncAttributes* a);
int mdc_attrs_megakernel(cudaFuncAttributes* a);

extern "C" int mdc_kernel_attrs(int kernel_id, int* regs, int* static_smem, int* max_dynamic_smem) {
  cudaFuncAttributes a;
  int e;
  switch (kernel_id) {
    case MDC_K_LOGITS: e = mdc_attrs_logits(&a); break;
    case MDC_K_MERGE_TOPK: e = mdc_attrs_merge_topk(&a); break;
    case MDC_K_LSE_MERGE: e = mdc_attrs_lse_merge(&a); break;
    case MDC_K_SPARSE_MLA: e = mdc_attrs_sparse_mla(&a); break;
    case MDC_K_MEGAKERNEL: e = mdc_attrs_megakernel(&a); break;
    default: return MDC_ERR_BAD_FORMAT;
  }
  if (e != 0) {
    mdc_set_last_cuda_error(e);
    return MDC_ERR_CUDA;
  }
  if (regs) *regs = a.numRegs;
  if (static_smem) *static_smem = static_cast<int>(a.sharedSizeBytes);
  if (max_dynamic_smem) *max_dynamic_smem = a.maxDynamicSharedSizeBytes;
  return MDC_OK;
}
