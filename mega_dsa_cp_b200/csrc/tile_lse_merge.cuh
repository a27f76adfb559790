// LSE-merge tile: combines normalised attention partials of several ranks (or
// KV splits) of one (b, t) row.  Pure bandwidth work: every partial element
// is read once with 16-byte loads, scaled by 2^(l_i - glse) and summed in fp32.
#pragma once

#include "common.cuh"

namespace mdc {

constexpr int kLseMaxSlices = 16;

template <bool SYS>
__device__ inline uint4 load16(const void* p) {
  if (SYS) return ld_sys_u4(static_cast<const uint4*>(p));
  return __ldg(static_cast<const uint4*>(p));
}

// One block handles heads [h0, h0 + n_heads) of one row.  `scale_smem` holds
// n_slices * n_heads floats.  SYS = partials may have been written by a peer
// GPU (loads bypass the non-coherent L1).
// Where the partials of one row live: slice i's (H, D) block at o + i * o_stride
// bytes, its (H,) LSE vector at lse + i * lse_stride floats.
struct LseSrc {
  const unsigned char* o;
  const float* lse;
  int64_t o_stride, lse_stride;
};

template <bool SYS>
__device__ inline void lse_merge_rows(const LseSrc& src, int ns, int H, int D, int acc_dtype, int out_dtype, void* o_out,
                                      float* lse_out, int h0, int n_heads, float* scale_smem);

template <bool SYS>
__device__ inline void lse_merge_tile(const mdc_lse_merge_params& p, int row, int h0, int n_heads, float* scale_smem) {
  const int esz = (p.acc_dtype == MDC_DT_F32) ? 4 : 2;
  LseSrc src;
  src.o = static_cast<const unsigned char*>(p.acc_o) + static_cast<int64_t>(row) * p.n_slices_max * p.H * p.D * esz;
  src.lse = p.acc_lse + static_cast<int64_t>(row) * p.n_slices_max * p.H;
  src.o_stride = static_cast<int64_t>(p.H) * p.D * esz;
  src.lse_stride = p.H;
  const int osz = (p.out_dtype == MDC_DT_F32) ? 4 : 2;
  lse_merge_rows<SYS>(src, p.n_slices, p.H, p.D, p.acc_dtype, p.out_dtype,
                      static_cast<unsigned char*>(p.o) + static_cast<int64_t>(row) * p.H * p.D * osz,
                      p.lse ? p.lse + static_cast<int64_t>(row) * p.H : nullptr, h0, n_heads, scale_smem);
}

// o_out / lse_out point at this row's (H, D) output block and (H,) LSE vector.
template <bool SYS>
__device__ inline void lse_merge_rows(const LseSrc& src, int ns, int H, int D, int acc_dtype, int out_dtype, void* o_out,
                                      float* lse_out, int h0, int n_heads, float* scale_smem) {
  const int tid = threadIdx.x;
  const float neg_inf = __int_as_float(0xff800000);
  sync_workers();
  for (int h = tid; h < n_heads; h += kBlockThreads) {
    const float* l = src.lse + h0 + h;
    float li[kLseMaxSlices];
    float g = neg_inf;
    for (int i = 0; i < ns; ++i) {
      li[i] = SYS ? ld_sys_f32(l + i * src.lse_stride) : l[i * src.lse_stride];
      g = fmaxf(g, li[i]);
    }
    const float anchor = (g == neg_inf) ? 0.f : g;
    float mass = 0.f;
    for (int i = 0; i < ns; ++i) mass += exp2f(li[i] - anchor);
    const bool live = mass > 0.f;
    const float glse = live ? g + log2f(mass) : neg_inf;
    for (int i = 0; i < ns; ++i) scale_smem[i * n_heads + h] = live ? exp2f(li[i] - glse) : 0.f;
    if (lse_out) lse_out[h0 + h] = glse;
  }
  sync_workers();
  const int vec = (acc_dtype == MDC_DT_F32) ? 4 : 8;  // elements per 16-byte load
  const int per_head = D / vec;
  const int esz = (acc_dtype == MDC_DT_F32) ? 4 : 2;
  for (int idx = tid; idx < n_heads * per_head; idx += kBlockThreads) {
    const int h = idx / per_head, d = (idx - h * per_head) * vec;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int i = 0; i < ns; ++i) {
      const float s = scale_smem[i * n_heads + h];
      const unsigned char* from = src.o + i * src.o_stride + (static_cast<int64_t>(h0 + h) * D + d) * esz;
      uint4 raw = load16<SYS>(from);
      if (acc_dtype == MDC_DT_F32) {
        acc[0] = fmaf(__uint_as_float(raw.x), s, acc[0]);
        acc[1] = fmaf(__uint_as_float(raw.y), s, acc[1]);
        acc[2] = fmaf(__uint_as_float(raw.z), s, acc[2]);
        acc[3] = fmaf(__uint_as_float(raw.w), s, acc[3]);
      } else {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] = fmaf(__uint_as_float(w[j] << 16), s, acc[2 * j]);
          acc[2 * j + 1] = fmaf(__uint_as_float(w[j] & 0xffff0000u), s, acc[2 * j + 1]);
        }
      }
    }
    const int64_t o_off = static_cast<int64_t>(h0 + h) * D + d;
    if (out_dtype == MDC_DT_F32) {
      float4* dst = reinterpret_cast<float4*>(static_cast<float*>(o_out) + o_off);
      dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      if (vec == 8) dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    } else {
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(o_out) + o_off;
      __nv_bfloat162 t0 = __floats2bfloat162_rn(acc[0], acc[1]);
      __nv_bfloat162 t1 = __floats2bfloat162_rn(acc[2], acc[3]);
      if (vec == 4) {
        uint2 out = make_uint2(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1));
        *reinterpret_cast<uint2*>(dst) = out;
      } else {
        __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[4], acc[5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(acc[6], acc[7]);
        uint4 out = make_uint4(*reinterpret_cast<uint32_t*>(&t0), *reinterpret_cast<uint32_t*>(&t1),
                               *reinterpret_cast<uint32_t*>(&t2), *reinterpret_cast<uint32_t*>(&t3));
        *reinterpret_cast<uint4*>(dst) = out;
      }
    }
  }
}

}  // namespace mdc
