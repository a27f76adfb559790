// Split sparse-MLA attention with its split workspace inside the library.
//
// mdc_sparse_mla_launch wants the caller to own the workspace that the slot
// splits write their partial outputs into.  Some callers have no way to get
// one at the point where they launch: a serving loop that handed every free
// byte of device memory to its KV-cache pool at start-up and never goes back
// to the allocator, or a decode step that runs on a latency-critical thread
// where entering the allocator (a lock, possibly a device synchronisation) is
// not acceptable.  For them this file keeps a fixed scratch block in the
// module's own device data segment, so the entry point below never calls an
// allocating routine -- no cudaMalloc / cudaFree, no pool, no framework tensor.
// The block is part of the library image: under CUDA's default lazy module
// loading its backing store (8 MiB + 16 KiB) is claimed when the FIRST call on
// a device looks the symbol up, and stays claimed until the process exits.
// Make that first call at start-up, before the application hands the rest of
// device memory to its pool: afterwards it could fail with an out-of-memory
// CUDA error (returned as MDC_ERR_CUDA), and later calls never touch the
// allocator again.
//
// Limits and rules:
//   * capacity: B * q_len * n_splits * H <= MDC_STATIC_WS_MAX_SLOTS (4096
//     partial rows of 512 fp32 = 8 MiB, plus 16 KiB of LSEs); larger requests
//     are rejected with MDC_ERR_TOO_LARGE and nothing is launched.
//   * the first call on a device is a warm-up: it loads the data segment and
//     looks up the scratch address once (with that device current), then
//     caches it.  Make it before any stream capture is begun -- the lookup is
//     not a stream operation -- and before memory gets tight (see above).
//   * nothing in the scratch has to start at zero: every (row, split, head)
//     slot that the combine kernel reads is written first by the attention
//     kernel of the same call, including the slots of empty splits (sum 0,
//     LSE -inf).  So the block is never cleared.
//   * a call whose status block comes back non-zero (a device-side give-up)
//     leaves `o` / `lse` undefined: the combine may have merged partials of an
//     earlier call that the aborted splits did not overwrite.
//   * there is ONE block per device: two calls whose kernels can overlap (two
//     streams, two host threads on the same device) race on it.  Serialise
//     them on one stream, or use mdc_sparse_mla_launch with separate
//     caller-owned workspaces.
#include <mutex>

#include "common.cuh"

namespace mdc {

constexpr int kStaticWsSlots = MDC_STATIC_WS_MAX_SLOTS;
constexpr int kStaticWsDv = 512;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) float g_static_ws_o[static_cast<size_t>(kStaticWsSlots) * kStaticWsDv];
static __device__ __align__(256) float g_static_ws_lse[kStaticWsSlots];

struct StaticWs {
  float* o = nullptr;
  float* lse = nullptr;
};
static StaticWs g_ws_of_device[kMaxDevices];
static std::mutex g_ws_mutex;

// Address of the scratch on the current device (set-up on first use).
static int static_ws_lookup(StaticWs* out) {
  int dev = -1;
  MDC_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return MDC_ERR_BAD_SHAPE;
  std::lock_guard<std::mutex> lock(g_ws_mutex);
  StaticWs& ws = g_ws_of_device[dev];
  if (!ws.o) {
    float* o = nullptr;
    float* lse = nullptr;
    MDC_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&o), g_static_ws_o));
    MDC_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&lse), g_static_ws_lse));
    if (!o || !lse) return MDC_ERR_CUDA;
    ws.lse = lse;
    ws.o = o;
  }
  *out = ws;
  return MDC_OK;
}

}  // namespace mdc

extern "C" int mdc_sparse_mla_launch_static_ws(const mdc_sparse_mla_params* p, void* stream) {
  using namespace mdc;
  if (!p) return MDC_ERR_NULL;
  if (p->B < 1 || p->q_len < 1 || p->H < 1 || p->n_splits < 1) return MDC_ERR_BAD_SHAPE;
  if (p->d_v != kStaticWsDv) return MDC_ERR_BAD_SHAPE;
  const long long slots = static_cast<long long>(p->B) * p->q_len * p->n_splits * p->H;
  if (slots > kStaticWsSlots) return MDC_ERR_TOO_LARGE;
  StaticWs ws;
  const int rc = static_ws_lookup(&ws);
  if (rc != MDC_OK) return rc;
  mdc_sparse_mla_params q = *p;  // same launch as the caller-workspace entry point, scratch swapped in
  q.ws_o = ws.o;
  q.ws_lse = ws.lse;
  return mdc_sparse_mla_launch(&q, stream);
}
