// Sparse MLA decode-attention tile: 64 query heads of one (b, t) row against a
// range of KV slots (window pool + gathered pool), flash-decoding style.
//
// Eight warps: warp w owns heads 16*(w%4).. and, for Q.K^T, slots 32*(w/4)..
// of each 64-slot tile; for P.V it owns output columns 256*(w/4)...  Q, the
// current and the next KV tile (bf16, 16-byte chunks XOR-swizzled by row so
// ldmatrix is conflict free) and the probability tile live in shared memory;
// the 64 x 512 fp32 output accumulator lives in registers (128 per thread).
// KV rows are gathered with 16-byte cp.async (zero-filled when the slot is
// masked) one tile ahead of the math.  Tensor-core work is mma.sync m16n8k16
// bf16 with fp32 accumulation; e4m3 operands are widened to bf16 (exact) on
// their way into shared memory.
#pragma once

#include "common.cuh"
#include "fp4.cuh"

namespace mdc {

constexpr int kMlaHeads = 64;   // heads per block
constexpr int kMlaTile = 64;    // slots per tile
constexpr int kMlaDv = 512;
constexpr int kWinSlots = 128;
constexpr float kLog2e = 1.4426950408889634f;

template <int DQK>
struct MlaSmem {
  static constexpr int kRowB = DQK * 2;
  static constexpr int kQ = 0;
  static constexpr int kK0 = kMlaHeads * kRowB;
  static constexpr int kK1 = kK0 + kMlaTile * kRowB;
  static constexpr int kP = kK1 + kMlaTile * kRowB;
  static constexpr int kStat = kP + kMlaHeads * kMlaTile * 2;       // 2 x 64 floats max, 2 x 64 sum
  static constexpr int kValid = kStat + 2 * 64 * 4;                 // 2 x 64 ints (the sums reuse the max slots)
  static constexpr int kTotal = kValid + 2 * 64 * 4;
};

__device__ inline void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ inline void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ inline void cp_async16_zfill(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t n = valid ? 16u : 0u;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(n)
               : "memory");
}
__device__ inline uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&t);
}
// 4 e4m3 bytes -> 4 bf16 (two packed words), exact
__device__ inline void e4m3x4_to_bf16(uint32_t w, uint32_t& lo, uint32_t& hi) {
  uint32_t h0, h1;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h0) : "h"(static_cast<uint16_t>(w & 0xffff)));
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h1) : "h"(static_cast<uint16_t>(w >> 16)));
  __half2 a = *reinterpret_cast<__half2*>(&h0), b = *reinterpret_cast<__half2*>(&h1);
  float2 fa = __half22float2(a), fb = __half22float2(b);
  lo = pack_bf16x2(fa.x, fa.y);
  hi = pack_bf16x2(fb.x, fb.y);
}
__device__ inline float round_through_e4m3(float x) {
  uint16_t packed;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(packed) : "f"(0.f), "f"(x));
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h) : "h"(packed));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h & 0xffff)));
}

template <int DQK>
__device__ inline uint32_t swz(int row, int chunk) {
  return static_cast<uint32_t>(row * (DQK * 2) + ((chunk ^ (row & 7)) << 4));
}

// Where slot `sl` of row `r` comes from.  Returns nullptr when masked.
template <int DQK, int ESZ>
__device__ inline const unsigned char* mla_slot_ptr(const mdc_sparse_mla_params& p, int r, int sl, int k_valid,
                                                    int win_valid) {
  if (sl < kWinSlots) {
    if (sl >= win_valid || p.kv_win == nullptr) return nullptr;
    const int page = p.pt_win ? p.pt_win[r] : 0;
    if (page < 0 || page >= p.pages_win) {
      report_failure(p.status, MDC_DEV_BAD_INDEX, page, sl, 0, 0);
      return nullptr;
    }
    return static_cast<const unsigned char*>(p.kv_win) + (static_cast<int64_t>(page) * kWinSlots + sl) * DQK * ESZ;
  }
  if (sl >= k_valid) return nullptr;
  const int e = sl - kWinSlots;
  int64_t entry;
  if (p.page_cmp == 1) {
    entry = p.pt_cmp[static_cast<int64_t>(r) * p.pt_cols + e];
  } else {
    const int page = p.pt_cmp[static_cast<int64_t>(r) * p.pt_cols + e / p.page_cmp];
    entry = static_cast<int64_t>(page) * p.page_cmp + e % p.page_cmp;
  }
  if (entry < 0 || entry >= static_cast<int64_t>(p.pages_cmp) * p.page_cmp) {
    report_failure(p.status, MDC_DEV_BAD_INDEX, static_cast<int>(entry), sl, 0, 0);
    return nullptr;
  }
  return static_cast<const unsigned char*>(p.kv_cmp) + entry * DQK * ESZ;
}

// Stage one 64-slot KV tile into shared memory (asynchronously for bf16).
template <int DQK, int KVDT>
__device__ inline void mla_load_tile(const mdc_sparse_mla_params& p, int r, int slot0, int k_valid, int win_valid,
                                     unsigned char* sK, int32_t* sValid) {
  const int tid = threadIdx.x;
  if (KVDT == MDC_DT_BF16) {
    constexpr int kChunks = DQK / 8;  // 16-byte chunks per row
    for (int ci = tid; ci < kMlaTile * kChunks; ci += kBlockThreads) {
      const int s = ci / kChunks, ch = ci - s * kChunks;
      const unsigned char* src = mla_slot_ptr<DQK, 2>(p, r, slot0 + s, k_valid, win_valid);
      if (ch == 0) sValid[s] = src != nullptr;
      cp_async16_zfill(sK + swz<DQK>(s, ch), src ? src + ch * 16 : static_cast<const unsigned char*>(p.kv_cmp),
                       src != nullptr);
    }
  } else {
    constexpr int kChunks = DQK / 16;  // 16-byte chunks of e4m3 per row, each widens to two bf16 chunks
    for (int ci = tid; ci < kMlaTile * kChunks; ci += kBlockThreads) {
      const int s = ci / kChunks, ch = ci - s * kChunks;
      const unsigned char* src = mla_slot_ptr<DQK, 1>(p, r, slot0 + s, k_valid, win_valid);
      if (ch == 0) sValid[s] = src != nullptr;
      uint4 raw = make_uint4(0, 0, 0, 0);
      if (src) raw = __ldg(reinterpret_cast<const uint4*>(src + ch * 16));
      uint4 lo, hi;
      e4m3x4_to_bf16(raw.x, lo.x, lo.y);
      e4m3x4_to_bf16(raw.y, lo.z, lo.w);
      e4m3x4_to_bf16(raw.z, hi.x, hi.y);
      e4m3x4_to_bf16(raw.w, hi.z, hi.w);
      *reinterpret_cast<uint4*>(sK + swz<DQK>(s, 2 * ch)) = lo;
      *reinterpret_cast<uint4*>(sK + swz<DQK>(s, 2 * ch + 1)) = hi;
    }
  }
  cp_async_commit();
}

// r = b*q_len + t, hb = head block, split / n_splits = slice of the slot range.
// o_row / lse_row, when given, replace p.o / p.lse for this row: they point at
// the (H, d_v) block and the (H,) vector that receive the row's direct output
// (possibly in a peer GPU's memory).  Called by the 256 worker threads.
// NDV = output columns this call produces (512, or 256 starting at column dv0:
// half the accumulator registers, for blocks whose register budget is 128).
template <int DQK, int KVDT, int NDV = kMlaDv>
__device__ void mla_tile(const mdc_sparse_mla_params& p, int r, int hb, int split, int n_splits,
                         unsigned char* smem, void* o_row = nullptr, float* lse_row = nullptr, int dv0 = 0, bool to_row = false) {
  constexpr int NT = NDV / 16;            // 8-column accumulator tiles per warp
  const int col0 = dv0 + (NDV / 2) * (static_cast<int>(threadIdx.x) >> 7);  // first output column of this warp
  using SM = MlaSmem<DQK>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const int mt = warp & 3, half = warp >> 2;
  unsigned char* sQ = smem + SM::kQ;
  unsigned char* sKb[2] = {smem + SM::kK0, smem + SM::kK1};
  unsigned char* sP = smem + SM::kP;
  float* sMax = reinterpret_cast<float*>(smem + SM::kStat);   // [2][64]
  float* sSum = sMax;                                          // [2][64], after the last tile
  int32_t* sValid = reinterpret_cast<int32_t*>(smem + SM::kValid);  // [2][64]
  const float neg_inf = __int_as_float(0xff800000);
  const float scale_log2 = p.softmax_scale * kLog2e;

  const int k_valid = min(max(p.k_valid[r], 0), kWinSlots + p.pt_cols * p.page_cmp);
  const int win_valid = p.win_valid ? min(max(p.win_valid[r], 0), kWinSlots) : 0;
  const int n_tiles_all = ceil_div(k_valid, kMlaTile);
  const int first = (win_valid > 0 && p.kv_win) ? 0 : min(n_tiles_all, kWinSlots / kMlaTile);
  const int per = ceil_div(max(n_tiles_all - first, 0), n_splits);
  const int t_begin = first + split * per;
  const int t_end = min(n_tiles_all, t_begin + per);

  sync_workers();  // shared memory may be in use by the previous task of this block
  // ---- stage Q (64 heads x DQK) as bf16, swizzled
  {
    const int h0 = hb * kMlaHeads;
    if (KVDT == MDC_DT_BF16) {
      constexpr int kChunks = DQK / 8;
      const unsigned char* q = static_cast<const unsigned char*>(p.q) +
                               (static_cast<int64_t>(r) * p.H + h0) * DQK * 2;
      for (int ci = tid; ci < kMlaHeads * kChunks; ci += kBlockThreads) {
        const int h = ci / kChunks, ch = ci - h * kChunks;
        cp_async16_zfill(sQ + swz<DQK>(h, ch), q + (static_cast<int64_t>(h) * DQK * 2 + ch * 16), true);
      }
    } else {
      constexpr int kChunks = DQK / 16;
      const unsigned char* q = static_cast<const unsigned char*>(p.q) + (static_cast<int64_t>(r) * p.H + h0) * DQK;
      for (int ci = tid; ci < kMlaHeads * kChunks; ci += kBlockThreads) {
        const int h = ci / kChunks, ch = ci - h * kChunks;
        uint4 raw = __ldg(reinterpret_cast<const uint4*>(q + static_cast<int64_t>(h) * DQK + ch * 16));
        uint4 lo, hi;
        e4m3x4_to_bf16(raw.x, lo.x, lo.y);
        e4m3x4_to_bf16(raw.y, lo.z, lo.w);
        e4m3x4_to_bf16(raw.z, hi.x, hi.y);
        e4m3x4_to_bf16(raw.w, hi.z, hi.w);
        *reinterpret_cast<uint4*>(sQ + swz<DQK>(h, 2 * ch)) = lo;
        *reinterpret_cast<uint4*>(sQ + swz<DQK>(h, 2 * ch + 1)) = hi;
      }
    }
  }
  if (t_begin < t_end) mla_load_tile<DQK, KVDT>(p, r, t_begin * kMlaTile, k_valid, win_valid, sKb[0], sValid);
  else cp_async_commit();

  float acc_o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) acc_o[i][0] = acc_o[i][1] = acc_o[i][2] = acc_o[i][3] = 0.f;
  // running statistics of rows (16mt+g) and (16mt+g+8); the sink seeds split 0
  float run_max[2] = {neg_inf, neg_inf};
  float run_sum[2] = {0.f, 0.f};  // this warp's half of the slots only
  if (p.attn_sink && split == 0) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float sk = p.attn_sink[hb * kMlaHeads + 16 * mt + g + 8 * i];
      if (sk != neg_inf) {
        run_max[i] = sk;
        run_sum[i] = (half == 0) ? 1.f : 0.f;
      }
    }
  }

  const uint32_t sQ_u = smem_u32(sQ), sP_u = smem_u32(sP);
#pragma unroll 1
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buf = (tile - t_begin) & 1;
    cp_async_wait<0>();
    sync_workers();
    if (tile + 1 < t_end)
      mla_load_tile<DQK, KVDT>(p, r, (tile + 1) * kMlaTile, k_valid, win_valid, sKb[buf ^ 1], sValid + 64 * (buf ^ 1));
    else
      cp_async_commit();
    const uint32_t sK_u = smem_u32(sKb[buf]);
    const int32_t* valid = sValid + 64 * buf;

    // ---- S = Q K^T for 16 heads x 32 slots
    float acc_s[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i) acc_s[i][0] = acc_s[i][1] = acc_s[i][2] = acc_s[i][3] = 0.f;
    {
      const int a_row = 16 * mt + (lane & 15), a_cadd = lane >> 4;
      const int mi = lane >> 3, r8 = lane & 7;
      const int b_row0 = 32 * half + (mi >> 1) * 8 + r8, b_cadd = mi & 1;
#pragma unroll 4
      for (int k = 0; k < DQK / 16; ++k) {
        uint32_t a[4], b0[4], b1[4];
        ldsm_x4(a, sQ_u + swz<DQK>(a_row, 2 * k + a_cadd));
        ldsm_x4(b0, sK_u + swz<DQK>(b_row0, 2 * k + b_cadd));
        ldsm_x4(b1, sK_u + swz<DQK>(b_row0 + 16, 2 * k + b_cadd));
        mma_bf16_16816(acc_s[0], a, b0[0], b0[1]);
        mma_bf16_16816(acc_s[1], a, b0[2], b0[3]);
        mma_bf16_16816(acc_s[2], a, b1[0], b1[1]);
        mma_bf16_16816(acc_s[3], a, b1[2], b1[3]);
      }
    }
    // mask + partial row max over this warp's 32 slots
    float pm[2] = {neg_inf, neg_inf};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const bool ok = valid[32 * half + 8 * nt + 2 * c + j] != 0;
        if (!ok) acc_s[nt][j] = acc_s[nt][2 + j] = neg_inf;
        pm[0] = fmaxf(pm[0], acc_s[nt][j]);
        pm[1] = fmaxf(pm[1], acc_s[nt][2 + j]);
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      pm[i] = fmaxf(pm[i], __shfl_xor_sync(0xffffffffu, pm[i], 1));
      pm[i] = fmaxf(pm[i], __shfl_xor_sync(0xffffffffu, pm[i], 2));
    }
    if (c == 0) {
      sMax[half * 64 + 16 * mt + g] = pm[0];
      sMax[half * 64 + 16 * mt + g + 8] = pm[1];
    }
    sync_workers();
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int row = 16 * mt + g + 8 * i;
      const float tm = fmaxf(sMax[row], sMax[64 + row]);
      const float nm = fmaxf(run_max[i], tm);
      corr[i] = (nm == run_max[i]) ? 1.f : exp2f((run_max[i] - nm) * scale_log2);
      run_max[i] = nm;
    }
    float ps[2] = {0.f, 0.f};
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      float pv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = j >> 1;
        float x = (run_max[i] == neg_inf) ? 0.f : exp2f((acc_s[nt][j] - run_max[i]) * scale_log2);
        if (p.fp8_p) x = round_through_e4m3(x);
        pv[j] = x;
        ps[i] += x;
      }
      const int chunk = 4 * half + nt;
      const int row0 = 16 * mt + g;
      *reinterpret_cast<uint32_t*>(sP + row0 * 128 + ((chunk ^ (row0 & 7)) << 4) + 4 * c) = pack_bf16x2(pv[0], pv[1]);
      const int row1 = row0 + 8;
      *reinterpret_cast<uint32_t*>(sP + row1 * 128 + ((chunk ^ (row1 & 7)) << 4) + 4 * c) = pack_bf16x2(pv[2], pv[3]);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 1);
      ps[i] += __shfl_xor_sync(0xffffffffu, ps[i], 2);
      run_sum[i] = run_sum[i] * corr[i] + ps[i];
    }
    if (corr[0] != 1.f || corr[1] != 1.f) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        acc_o[nt][0] *= corr[0];
        acc_o[nt][1] *= corr[0];
        acc_o[nt][2] *= corr[1];
        acc_o[nt][3] *= corr[1];
      }
    }
    sync_workers();
    // ---- O += P V for 16 heads x 256 columns
    {
      const int a_row = 16 * mt + (lane & 15), a_cadd = lane >> 4;
      const int mi = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        uint32_t a[4];
        {
          const int chunk = 2 * kk + a_cadd;
          ldsm_x4(a, sP_u + a_row * 128 + ((chunk ^ (a_row & 7)) << 4));
        }
        const int v_row = 16 * kk + (mi & 1) * 8 + r8;
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t bv[4];
          ldsm_x4_t(bv, sK_u + swz<DQK>(v_row, col0 / 8 + 2 * np + (mi >> 1)));
          mma_bf16_16816(acc_o[2 * np], a, bv[0], bv[1]);
          mma_bf16_16816(acc_o[2 * np + 1], a, bv[2], bv[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
  sync_workers();
  // ---- combine the two slot halves' sums and write out
  if (c == 0) {
    sSum[half * 64 + 16 * mt + g] = run_sum[0];
    sSum[half * 64 + 16 * mt + g + 8] = run_sum[1];
  }
  sync_workers();
  const bool direct = n_splits == 1 || to_row;  // a split partial may also go to o_row / lse_row
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int row = 16 * mt + g + 8 * i;
    const int h = hb * kMlaHeads + row;
    const float sum = sSum[row] + sSum[64 + row];
    const bool live = sum > 0.f;
    const float inv = live ? p.output_scale / sum : 0.f;
    const float lse = live ? log2f(sum) + scale_log2 * run_max[i] : neg_inf;
    if (half == 0 && c == 0 && dv0 == 0) {
      if (direct) {
        if (lse_row) lse_row[h] = lse;
        else if (p.lse) p.lse[static_cast<int64_t>(r) * p.lse_stride + h] = lse;
      } else {
        p.ws_lse[(static_cast<int64_t>(r) * n_splits + split) * p.H + h] = lse;
      }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int col = col0 + 8 * nt + 2 * c;
      const float v0 = acc_o[nt][2 * i] * inv, v1 = acc_o[nt][2 * i + 1] * inv;
      if (!direct) {
        float* dst = p.ws_o + ((static_cast<int64_t>(r) * n_splits + split) * p.H + h) * kMlaDv + col;
        *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
      } else if (p.out_dtype == MDC_DT_F32) {
        float* dst = (o_row ? static_cast<float*>(o_row) : static_cast<float*>(p.o) + static_cast<int64_t>(r) * p.o_stride) +
                     static_cast<int64_t>(h) * kMlaDv + col;
        *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
      } else {
        __nv_bfloat16* dst = (o_row ? static_cast<__nv_bfloat16*>(o_row)
                                    : static_cast<__nv_bfloat16*>(p.o) + static_cast<int64_t>(r) * p.o_stride) +
                             static_cast<int64_t>(h) * kMlaDv + col;
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(v0, v1);
      }
    }
  }
}

}  // namespace mdc
