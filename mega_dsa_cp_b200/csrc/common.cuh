// Shared device/host helpers for the sm_100a kernels of this library:
// status codes, PTX wrappers (mbarrier, bulk copies, scoped loads/reductions,
// fences) and bounded spin-waits.  Every wait in this library gives up after a
// clock budget and reports through a status word instead of spinning forever.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/mdc.h"

namespace mdc {

constexpr int kBlockThreads = 256;   // every tile's worker part is written for 8 warps (warps 0..7)
constexpr int kWarps = kBlockThreads / 32;

// Barrier among the 256 worker threads only (warps 0..7); blocks may carry
// extra service warps that never join it.
__device__ inline void sync_workers() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

// ------------------------------------------------------------------ status
// A kernel that gives up on a wait (or finds an inconsistent input) records the
// first failure in a caller-visible 8-word block:
//   [0] code (MDC_DEV_*), [1] blockIdx.x, [2] detail a, [3] detail b,
//   [4..5] value seen (u64), [6..7] value wanted (u64)
__device__ inline void report_failure(int32_t* status, int code, int a, int b,
                                      unsigned long long seen, unsigned long long want) {
  if (status == nullptr) return;
  if (atomicCAS(reinterpret_cast<int*>(status), 0, code) == 0) {
    status[1] = static_cast<int32_t>(blockIdx.x);
    status[2] = a;
    status[3] = b;
    status[4] = static_cast<int32_t>(seen & 0xffffffffu);
    status[5] = static_cast<int32_t>(seen >> 32);
    status[6] = static_cast<int32_t>(want & 0xffffffffu);
    status[7] = static_cast<int32_t>(want >> 32);
    __threadfence_system();
  }
}

// ------------------------------------------------------------------ smem / mbarrier
__device__ inline uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ inline void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ inline void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ inline void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ inline void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ inline bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of an mbarrier phase.
__device__ inline bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait on an mbarrier phase.  try_wait itself suspends the thread for a
// hardware-defined slice, so the loop is not a hot spin; the clock is read only
// every 64 polls.  Returns false once `budget` clock cycles (about a second by
// default) have passed without the phase completing, or once the block-wide
// abort flag (optional) is raised by another role.
__device__ inline bool mbar_wait(uint64_t* bar, uint32_t parity, long long budget = (1ll << 31),
                                 const volatile uint32_t* abort_flag = nullptr) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  do {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (abort_flag && *abort_flag) return false;
  } while (clock64() - t0 < budget);
  return false;
}

// Predicated forms for "one lane signals": a predicated instruction instead of a
// divergent branch keeps the warp converged, which is much cheaper on a path
// that runs once per pipeline stage.
__device__ inline void mbar_arrive_if(uint64_t* bar, bool pred) {
  asm volatile("{\n .reg .pred p;\n setp.ne.u32 p, %1, 0;\n @p mbarrier.arrive.shared::cta.b64 _, [%0];\n}" ::"r"(
                   smem_u32(bar)),
               "r"(static_cast<uint32_t>(pred))
               : "memory");
}

// Shared-memory progress counters (cheaper to poll than an mbarrier for a
// thread that sits on the tensor-core issue path): release increment, acquire load.
__device__ inline void red_release_cta_shared_inc(uint32_t* p) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], 1;" ::"r"(smem_u32(p)) : "memory");
}
__device__ inline void red_release_cta_shared_inc_if(uint32_t* p, bool pred) {
  asm volatile("{\n .reg .pred p;\n setp.ne.u32 p, %1, 0;\n @p red.release.cta.shared::cta.add.u32 [%0], 1;\n}" ::"r"(
                   smem_u32(p)),
               "r"(static_cast<uint32_t>(pred))
               : "memory");
}
__device__ inline uint32_t ld_acquire_cta_shared_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(p)) : "memory");
  return v;
}
// Bounded wait until a shared counter reaches `target` (same give-up rules as mbar_wait).
__device__ inline bool counter_wait(const uint32_t* p, uint32_t target, long long budget = (1ll << 31),
                                    const volatile uint32_t* abort_flag = nullptr) {
  if (ld_acquire_cta_shared_u32(p) >= target) return true;
  const long long t0 = clock64();
  do {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      __nanosleep(20);  // a hot spin would take issue slots from the warps this one waits for
      if (ld_acquire_cta_shared_u32(p) >= target) return true;
    }
    if (abort_flag && *abort_flag) return false;
  } while (clock64() - t0 < budget);
  return false;
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier.  Both
// addresses 16-byte aligned, size a multiple of 16.
__device__ inline void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
// L2 cache policy for data that is read exactly once (a streamed cache): its lines are the first
// to be evicted, so the stream does not push out what the other tasks of a persistent kernel re-use
// every step -- their code above all: instructions live in the same L2, and a task whose code has
// been evicted pays a DRAM round trip per instruction-cache miss.
__device__ inline uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
// bulk_g2s with an L2 cache policy
__device__ inline void bulk_g2s_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(smem_dst)),
      "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}
// 1-D bulk copy shared -> global (local or peer memory), bulk-group completion.
__device__ inline void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst),
               "r"(smem_u32(smem_src)), "r"(bytes)
               : "memory");
}
__device__ inline void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ inline void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ inline void bulk_wait_all_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ inline void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }
__device__ inline void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16-byte cp.async (LDGSTS), used for row gathers.
__device__ inline void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc) : "memory");
}
__device__ inline void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ inline void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------ scoped memory ops
__device__ inline unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline unsigned long long ld_relaxed_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline void red_release_sys_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ inline void red_release_gpu_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ inline void red_relaxed_sys_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ inline void red_relaxed_gpu_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.relaxed.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ inline void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ inline void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ inline float4 ld_acquire_sys_f4(const float4* p) {
  // payload reads that must observe a peer's released stores without a fence:
  // relaxed.sys vector load after an acquire on the flag is sufficient; this
  // helper bypasses L1 (which is not coherent across GPUs).
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ inline uint4 ld_sys_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ inline float ld_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ inline void nanosleep(uint32_t ns) { asm volatile("nanosleep.u32 %0;" ::"r"(ns)); }
__device__ inline unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------------ warp helpers
__device__ inline float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ inline float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ inline int warp_excl_scan(int v, int lane, int* total) {
  int x = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int y = __shfl_up_sync(0xffffffffu, x, o);
    if (lane >= o) x += y;
  }
  *total = __shfl_sync(0xffffffffu, x, 31);
  return x - v;
}

// fp32 -> order-preserving u32 (larger float <=> larger key), bit-level.
__device__ __host__ inline uint32_t sortable_u32(float f) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(f);
#else
  union { float f; uint32_t u; } c; c.f = f; uint32_t u = c.u;
#endif
  return (u & 0x80000000u) ? ~u : (u ^ 0x80000000u);
}

}  // namespace mdc

#define MDC_CUDA_OK(expr)                                   \
  do {                                                      \
    cudaError_t _e = (expr);                                \
    if (_e != cudaSuccess) {                                \
      mdc_set_last_cuda_error(static_cast<int>(_e));        \
      return MDC_ERR_CUDA;                                  \
    }                                                       \
  } while (0)

extern "C" void mdc_set_last_cuda_error(int e);
