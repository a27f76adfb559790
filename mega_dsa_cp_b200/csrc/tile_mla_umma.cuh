// Sparse MLA decode-attention tile on the 5th-generation tensor cores: 128
// query heads of one (b, t) row against a range of KV slots, 128 of the 512
// output columns per block (four blocks cover a row's output; each repeats the
// cheap-to-issue Q.K^T so that the output accumulator fits tensor memory).
//
// Tensor memory (512 columns x 128 lanes, lane = head):
//   Q   DQK/2 columns   bf16 pairs, the A operand of S = Q K^T, loaded once
//   O   128 columns     fp32 output accumulator
//   S   64 columns      fp32 logits of the current 64-slot tile
//   P   32 columns      bf16 probabilities, the A operand of O += P V
// Shared memory: a ring of KV tiles, each 64 slots x DQK bf16 stored as DQK/64
// panels of 64 rows x 128 bytes with the 128-byte swizzle.  One image serves
// both products: a panel is a K-major B operand for Q K^T (row = slot, 64 dims
// per row) and, read "MN-major", the B operand of P V (for a fixed slot the 64
// output columns are contiguous), so V needs no transposed copy.
//
// Roles (448 threads): warps 0-3 softmax (thread = head: no cross-thread
// reductions; reads S with tcgen05.ld, writes P with tcgen05.st, rescales O
// only when the running maximum grew by more than 2^8), warps 4-11 gather KV
// rows with 16-byte cp.async (a warp instruction reads 512 contiguous bytes of
// one row), warp 12 issues the MMAs.  Per tile: 36 x (M128 N64 K16) for Q K^T,
// 4 x (M128 N128 K16) for P V.  All waits are bounded.
#pragma once

#include "common.cuh"
#include "tile_mla.cuh"
#include "umma.cuh"

namespace mdc {

constexpr int kMuHeads = 128;   // heads per block (= UMMA M)
constexpr int kMuTile = 64;     // slots per tile
constexpr int kMuDv = 128;      // output columns per block
constexpr int kMuThreads = 448;
constexpr int kMuGatherWarp0 = 4, kMuGatherWarps = 8, kMuIssueWarp = 12;

template <int DQK>
struct MlaUmmaSmem {
  static constexpr int kPanels = DQK / 64;
  static constexpr int kStageBytes = kPanels * kMuTile * 128;
  // as many stages as fit beside ~3 KB of bookkeeping in 226 KB
  static constexpr int kStages = (226 * 1024 - 3072) / kStageBytes >= 3 ? 3 : 2;
  static constexpr int kK = 0;
  static constexpr int kBars = kStages * kStageBytes;   // full[S], free[S], s_ready, p_ready, q_ready, o_final, qs_ready
  static constexpr int kMisc = kBars + (2 * kStages + 6) * 8;  // [0] tmem base, [1] abort flag
  static constexpr int kValid = kMisc + 64;                     // [S][8] bytes: validity bits of 8 slots per gather warp
  static constexpr int kTotal = kValid + kStages * 8 + 56;
};

namespace umma {
// Shared-memory B operand read MN-major with the 128-byte swizzle: for one K index (row of 128
// bytes) 64 consecutive N elements; 8 K rows form a 1024-byte atom.  lbo = bytes between
// consecutive 64-element N blocks, sbo = bytes between consecutive groups of 8 K rows.
__device__ inline uint64_t smem_desc_mn_sw128(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
// kind::f16 instruction descriptor, bf16 operands, fp32 accumulator; b_mn = B operand MN-major
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}
__device__ inline void tmem_ld32_f(uint32_t taddr, float (&v)[32]) {
  uint32_t u[32];
  tmem_ld32(taddr, u);
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(u[i]);
}
}  // namespace umma

__device__ inline float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Row pointers of this warp's 8 rows of one 64-slot tile: lane rr < 8 looks up row gw*8 + rr, so
// the 8 page-table reads of a tile are one instruction and not a chain (nullptr = masked slot).
template <int DQK>
__device__ inline const unsigned char* mla_umma_row_ptr(const mdc_sparse_mla_params& p, int r, int slot0, int k_valid,
                                                        int win_valid, int gw, int lane) {
  return lane < 8 ? mla_slot_ptr<DQK, 2>(p, r, slot0 + gw * 8 + lane, k_valid, win_valid) : nullptr;
}

// Gather one 64-slot tile: this warp's 8 rows, whose pointers sit in lanes 0-7 (`mine`).  Returns
// the validity bits of its rows.
template <int DQK>
__device__ inline uint32_t mla_umma_gather_rows(const mdc_sparse_mla_params& p, const unsigned char* mine,
                                                unsigned char* stage, int gw, int lane) {
  constexpr int kChunks = DQK / 8;  // 16-byte chunks per row
  const uint32_t bits = __ballot_sync(0xffffffffu, mine != nullptr) & 0xffu;
  const unsigned long long mine_u = reinterpret_cast<unsigned long long>(mine);
#pragma unroll
  for (int rr = 0; rr < 8; ++rr) {
    const int s = gw * 8 + rr;
    const unsigned char* src = reinterpret_cast<const unsigned char*>(__shfl_sync(0xffffffffu, mine_u, rr));
    const unsigned char* base = src ? src : static_cast<const unsigned char*>(p.kv_cmp);
#pragma unroll
    for (int ch = lane; ch < kChunks; ch += 32) {
      unsigned char* dst = stage + (ch >> 3) * (kMuTile * 128) + s * 128 + (((ch & 7) ^ (s & 7)) << 4);
      cp_async16_zfill(dst, base + ch * 16, src != nullptr);
    }
  }
  cp_async_commit();
  return bits;
}

// r = b*q_len + t, hb = block of 128 heads, dq = block of 128 output columns,
// split / n_splits = slice of the slot range.  o_row / lse_row, when given,
// replace p.o / p.lse for this row (they point at the row's (H, d_v) block and
// (H,) vector, possibly in a peer GPU's memory); with to_row a split's partial goes there too
// instead of the split workspace.  All kMuThreads threads call it.
template <int DQK>
__device__ void mla_umma_tile(const mdc_sparse_mla_params& p, int r, int hb, int dq, int split, int n_splits,
                              unsigned char* smem, void* o_row = nullptr, float* lse_row = nullptr, bool to_row = false) {
  using SM = MlaUmmaSmem<DQK>;
  constexpr int S = SM::kStages;
  constexpr uint32_t kQCols = DQK / 2, kOCol = kQCols, kSCol = kOCol + kMuDv, kPCol = kSCol + kMuTile;
  static_assert(kPCol + kMuTile / 2 <= 512, "tensor memory over-subscribed");
  static_assert(S >= 2 && SM::kPanels * kMuHeads * 128 <= (S - 1) * SM::kStageBytes,
                "the staged query must fit the KV ring behind its first stage");
  constexpr long long kBudget = 1ll << 31;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  unsigned char* kst = smem + SM::kK;
  unsigned char* qst = kst + SM::kStageBytes;   // the query rows are staged in stages 1.. while tile 0 lands in stage 0
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM::kBars);
  uint64_t* free_ = full + S;
  uint64_t* s_ready = free_ + S;
  uint64_t* p_ready = s_ready + 1;
  uint64_t* q_ready = p_ready + 1;
  uint64_t* o_final = q_ready + 1;
  uint64_t* qs_ready = o_final + 1;  // the query rows are staged in shared memory
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + SM::kMisc);
  volatile uint32_t* abort_flag = misc + 1;
  unsigned char* validb = smem + SM::kValid;
  const float neg_inf = __int_as_float(0xff800000);
  const float c2 = p.softmax_scale * kLog2e;

  const int k_valid = min(max(p.k_valid[r], 0), kWinSlots + p.pt_cols * p.page_cmp);
  const int win_valid = p.win_valid ? min(max(p.win_valid[r], 0), kWinSlots) : 0;
  const int n_tiles_all = ceil_div(k_valid, kMuTile);
  const int first = (win_valid > 0 && p.kv_win) ? 0 : min(n_tiles_all, kWinSlots / kMuTile);
  const int per = ceil_div(max(n_tiles_all - first, 0), n_splits);
  const int t_begin = first + split * per;
  const int n_my = max(0, min(n_tiles_all, t_begin + per) - t_begin);

  __syncthreads();  // shared memory may be in use by the previous task of this block
  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], kMuGatherWarps);
      mbar_init(&free_[s], 1);
    }
    mbar_init(s_ready, 1);
    mbar_init(p_ready, 4);
    mbar_init(q_ready, 4);
    mbar_init(o_final, 1);
    mbar_init(qs_ready, kMuGatherWarps);
    misc[1] = 0;
    mbar_fence_init();
  }
  if (warp == kMuIssueWarp) umma::tmem_alloc(misc, 512);
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = misc[0];
  auto give_up = [&](int what, int idx) {
    report_failure(p.status, MDC_DEV_COPY_TIMEOUT, 16 + what, idx, 0, 0);
    *abort_flag = 1;
  };

  if (warp < 4) {
    // ---------------- softmax warps: thread = head
    const int h = hb * kMuHeads + warp * 32 + lane;
    const uint32_t t_lane = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    {  // Q row -> tensor memory (bf16 pairs, 16 columns per store), from the copy the gather warps staged
      // in the (still empty) stages 1.. of the KV ring as DQK/64 panels of 128 rows x 128 bytes, 128-byte swizzle
      bool okq = mbar_wait(qs_ready, 0, kBudget, abort_flag);
      if (!okq && lane == 0) give_up(7, 0);
      const int row = warp * 32 + lane;
#pragma unroll 2
      for (int j = 0; j < static_cast<int>(kQCols) / 16; ++j) {
        uint32_t v[16];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int ch = 4 * j + u;
          const uint4 x = *reinterpret_cast<const uint4*>(qst + (ch >> 3) * (kMuHeads * 128) + row * 128 +
                                                          (((ch & 7) ^ (row & 7)) << 4));
          v[4 * u] = x.x; v[4 * u + 1] = x.y; v[4 * u + 2] = x.z; v[4 * u + 3] = x.w;
        }
        umma::tmem_st16(t_lane + 16 * j, v);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      mbar_arrive_if(q_ready, lane == 0);
    }
    float m_used = neg_inf, l = 0.f;
    if (p.attn_sink && split == 0) {
      const float sk = p.attn_sink[h];
      if (sk != neg_inf) {
        m_used = sk;
        l = 1.f;
      }
    }
    bool ok = true;
    for (int i = 0; i < n_my; ++i) {
      if (!mbar_wait(s_ready, i & 1, kBudget, abort_flag)) {
        if (lane == 0) give_up(0, i);
        ok = false;
        break;
      }
      umma::fence_after_sync();
      float sv[kMuTile];
      {
        float a[32], b[32];
        umma::tmem_ld32_f(t_lane + kSCol, a);
        umma::tmem_ld32_f(t_lane + kSCol + 32, b);
        umma::wait_ld();
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          sv[j] = a[j];
          sv[32 + j] = b[j];
        }
      }
      const uint2 vb = *reinterpret_cast<const uint2*>(validb + (i % S) * 8);
      // (one warp per scheduler: dependent chains are what costs here, so the maximum and the sum
      // run on four independent accumulators and a full tile skips the masking)
      if ((vb.x & vb.y) != 0xffffffffu) {
#pragma unroll
        for (int j = 0; j < kMuTile; ++j) {
          const bool valid = ((j < 32 ? vb.x >> j : vb.y >> (j - 32)) & 1u) != 0;
          sv[j] = valid ? sv[j] : neg_inf;
        }
      }
      float tm[4] = {neg_inf, neg_inf, neg_inf, neg_inf};
#pragma unroll
      for (int j = 0; j < kMuTile; j += 4) {
        tm[0] = fmaxf(tm[0], sv[j]);
        tm[1] = fmaxf(tm[1], sv[j + 1]);
        tm[2] = fmaxf(tm[2], sv[j + 2]);
        tm[3] = fmaxf(tm[3], sv[j + 3]);
      }
      const float tmax = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3]));
      // the reference maximum moves only when the tile maximum exceeds it by more than 2^8
      if (tmax > m_used && (m_used == neg_inf || (tmax - m_used) * c2 > 8.f)) {
        const float corr = (m_used == neg_inf) ? 0.f : exp2f((m_used - tmax) * c2);
        l *= corr;
        if (i > 0) {
#pragma unroll 1
          for (int cb = 0; cb < kMuDv / 32; ++cb) {
            uint32_t o[32];
            umma::tmem_ld32(t_lane + kOCol + 32 * cb, o);
            umma::wait_ld();
            uint32_t lo[16], hi[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              lo[j] = __float_as_uint(__uint_as_float(o[j]) * corr);
              hi[j] = __float_as_uint(__uint_as_float(o[16 + j]) * corr);
            }
            umma::tmem_st16(t_lane + kOCol + 32 * cb, lo);
            umma::tmem_st16(t_lane + kOCol + 32 * cb + 16, hi);
          }
        }
        m_used = tmax;
      }
      uint32_t pk[kMuTile / 2];
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      {
        // p = 2^((s - m) * c2) as one fused multiply-add and one ex2.approx; a masked slot (-inf)
        // gives 0, and with m = -inf (nothing valid so far) the whole tile is 0
        const bool dead = m_used == neg_inf;
        const float off = dead ? 0.f : -m_used * c2;
#pragma unroll
        for (int j = 0; j < kMuTile / 2; ++j) {
          const float p0 = dead ? 0.f : ex2_approx(fmaf(sv[2 * j], c2, off));
          const float p1 = dead ? 0.f : ex2_approx(fmaf(sv[2 * j + 1], c2, off));
          ps4[j & 3] += p0 + p1;
          pk[j] = pack_bf16x2(p0, p1);
        }
      }
      const float ps = (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      l += ps;
      {
        uint32_t lo[16], hi[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          lo[j] = pk[j];
          hi[j] = pk[16 + j];
        }
        umma::tmem_st16(t_lane + kPCol, lo);
        umma::tmem_st16(t_lane + kPCol + 16, hi);
      }
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      mbar_arrive_if(p_ready, lane == 0);
    }
    if (ok && n_my > 0 && !mbar_wait(o_final, 0, kBudget, abort_flag)) {
      if (lane == 0) give_up(1, n_my);
      ok = false;
    }
    umma::fence_after_sync();
    if (ok) {
      const bool live = l > 0.f;
      const float inv = live ? p.output_scale / l : 0.f;
      const float lse = live ? log2f(l) + c2 * m_used : neg_inf;
      const bool direct = n_splits == 1 || to_row;  // a split partial may also go to o_row / lse_row
      if (dq == 0) {
        if (direct) {
          if (lse_row) lse_row[h] = lse;
          else if (p.lse) p.lse[static_cast<int64_t>(r) * p.lse_stride + h] = lse;
        } else {
          p.ws_lse[(static_cast<int64_t>(r) * n_splits + split) * p.H + h] = lse;
        }
      }
      const int col0 = dq * kMuDv;
      // A bf16 row that goes to o_row (the owner's inbox, possibly on a peer GPU) is staged in shared
      // memory (the KV ring is idle now) and leaves as ONE 256-byte bulk copy per head: sixteen
      // 16-byte stores per thread over NVLink take an order of magnitude longer.
      const bool bulk_out = direct && o_row != nullptr && p.out_dtype != MDC_DT_F32;
      unsigned char* stage_row = kst + (warp * 32 + lane) * (kMuDv * 2);
#pragma unroll 1
      for (int cb = 0; cb < kMuDv / 32; ++cb) {
        float o[32];
        if (n_my > 0) {
          umma::tmem_ld32_f(t_lane + kOCol + 32 * cb, o);
          umma::wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0.f;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) o[j] *= inv;
        const int col = col0 + 32 * cb;
        if (bulk_out) {
          uint4* dst = reinterpret_cast<uint4*>(stage_row + 64 * cb);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(pack_bf16x2(o[8 * j], o[8 * j + 1]), pack_bf16x2(o[8 * j + 2], o[8 * j + 3]),
                                pack_bf16x2(o[8 * j + 4], o[8 * j + 5]), pack_bf16x2(o[8 * j + 6], o[8 * j + 7]));
        } else if (!direct) {
          float4* dst = reinterpret_cast<float4*>(p.ws_o + ((static_cast<int64_t>(r) * n_splits + split) * p.H + h) * kMlaDv + col);
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        } else if (p.out_dtype == MDC_DT_F32) {
          float* base = (o_row ? static_cast<float*>(o_row) : static_cast<float*>(p.o) + static_cast<int64_t>(r) * p.o_stride) +
                        static_cast<int64_t>(h) * kMlaDv + col;
          float4* dst = reinterpret_cast<float4*>(base);
#pragma unroll
          for (int j = 0; j < 8; ++j) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        } else {
          __nv_bfloat16* base = (o_row ? static_cast<__nv_bfloat16*>(o_row)
                                       : static_cast<__nv_bfloat16*>(p.o) + static_cast<int64_t>(r) * p.o_stride) +
                                static_cast<int64_t>(h) * kMlaDv + col;
          uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_uint4(pack_bf16x2(o[8 * j], o[8 * j + 1]), pack_bf16x2(o[8 * j + 2], o[8 * j + 3]),
                                pack_bf16x2(o[8 * j + 4], o[8 * j + 5]), pack_bf16x2(o[8 * j + 6], o[8 * j + 7]));
        }
      }
      if (bulk_out) {
        fence_proxy_async_smem();  // the copy engine reads the staged row through the async proxy
        bulk_s2g(static_cast<__nv_bfloat16*>(o_row) + static_cast<int64_t>(h) * kMlaDv + col0, stage_row, kMuDv * 2);
        bulk_commit();
        bulk_wait_all();           // the row has been written before this thread reaches the block's notify
        fence_proxy_async_global();
      }
    }
  } else if (warp >= kMuGatherWarp0 && warp < kMuGatherWarp0 + kMuGatherWarps) {
    // ---------------- gather warps: 8 rows of every tile each, up to two tiles in flight per warp
    const int gw = warp - kMuGatherWarp0;
    bool ok = true;
    {  // stage the 128 query rows (coalesced: a warp instruction copies 512 contiguous bytes of a row)
      constexpr int kChunks = DQK / 8;
      const unsigned char* q0 = static_cast<const unsigned char*>(p.q) +
                                (static_cast<int64_t>(r) * p.H + hb * kMuHeads) * DQK * 2;
      for (int rr = 0; rr < kMuHeads / kMuGatherWarps; ++rr) {
        const int row = gw * (kMuHeads / kMuGatherWarps) + rr;
#pragma unroll
        for (int ch = lane; ch < kChunks; ch += 32) {
          cp_async16_zfill(qst + (ch >> 3) * (kMuHeads * 128) + row * 128 + (((ch & 7) ^ (row & 7)) << 4),
                           q0 + static_cast<int64_t>(row) * DQK * 2 + ch * 16, true);
        }
      }
      cp_async_commit();
    }
    // row pointers are looked up one tile ahead, so the page-table read is not on the path
    const unsigned char* mine = n_my > 0 ? mla_umma_row_ptr<DQK>(p, r, t_begin * kMuTile, k_valid, win_valid, gw, lane)
                                         : nullptr;
    int i0 = 0;
    if (n_my > 0) {  // tile 0 goes into stage 0 behind the query copies: its latency hides under the query's
      const uint32_t bits = mla_umma_gather_rows<DQK>(p, mine, kst, gw, lane);
      if (n_my > 1) mine = mla_umma_row_ptr<DQK>(p, r, (t_begin + 1) * kMuTile, k_valid, win_valid, gw, lane);
      if (lane == 0) validb[gw] = static_cast<unsigned char>(bits);
      i0 = 1;
      cp_async_wait<1>();   // the query rows (the older group) have landed
    } else {
      cp_async_wait<0>();
    }
    {
      __syncwarp();
      mbar_arrive_if(qs_ready, lane == 0);
      // stages 1.. are free for KV tiles once the softmax warps have moved the rows into tensor memory
      if (!mbar_wait(q_ready, 0, kBudget, abort_flag)) {
        if (lane == 0) give_up(8, 0);
        ok = false;
      }
    }
    // Tiles [done, i) have been issued but not yet published.  A tile is published as soon as
    // its copies have landed -- never held back until the NEXT tile could be issued: when the
    // stage of the next tile is still in use, this warp first drains and publishes what it has
    // in flight (the tensor core is waiting for exactly that), then waits for the stage.
    int done = 0;
    auto publish = [&](int upto) {
      fence_proxy_async_smem();  // the tensor core reads the tiles through the async proxy
      __syncwarp();
      for (int t = done; t < upto; ++t) mbar_arrive_if(&full[t % S], lane == 0);
      done = upto;
    };
    if (i0 == 1 && ok) {  // tile 0 was issued before the query hand-over: it has had time to land, publish it now
      cp_async_wait<0>();
      publish(1);
    }
    for (int i = i0; i < n_my && ok; ++i) {
      const int st = i % S;
      if (i >= S) {
        const uint32_t par = ((i / S) - 1) & 1;
        if (!__all_sync(0xffffffffu, mbar_test(&free_[st], par))) {
          if (done < i) {
            cp_async_wait<0>();
            publish(i);
          }
          if (!mbar_wait(&free_[st], par, kBudget, abort_flag)) {
            if (lane == 0) give_up(2, i);
            ok = false;
            break;
          }
        }
      }
      const uint32_t bits = mla_umma_gather_rows<DQK>(p, mine, kst + st * SM::kStageBytes, gw, lane);
      if (i + 1 < n_my) mine = mla_umma_row_ptr<DQK>(p, r, (t_begin + i + 1) * kMuTile, k_valid, win_valid, gw, lane);
      if (lane == 0) validb[st * 8 + gw] = static_cast<unsigned char>(bits);
      if (i - done >= 1) {  // at most two tiles in flight per warp
        cp_async_wait<1>();
        publish(i);
      }
    }
    cp_async_wait<0>();
    if (ok && n_my > 0) publish(n_my);
  } else if (warp == kMuIssueWarp) {
    // ---------------- issue warp
    constexpr uint32_t idesc_qk = umma::idesc_bf16(kMuHeads, kMuTile, false);
    constexpr uint32_t idesc_pv = umma::idesc_bf16(kMuHeads, kMuDv, true);
    const uint32_t kst_u = smem_u32(kst);
    bool ok = mbar_wait(q_ready, 0, kBudget, abort_flag);
    if (!ok && lane == 0) give_up(3, 0);
    auto issue_pv = [&](int i) {  // O (+)= P V of tile i: 4 K-steps of 16 slots
      const uint32_t base = kst_u + (i % S) * SM::kStageBytes + (dq * kMuDv / 64) * (kMuTile * 128);
#pragma unroll
      for (int kk = 0; kk < kMuTile / 16; ++kk) {
        const uint64_t bdesc = umma::smem_desc_mn_sw128(base + kk * 2048, kMuTile * 128, 1024);
        umma::mma_f16_ts(tmem + kOCol, tmem + kPCol + 8 * kk, bdesc, idesc_pv, i > 0 || kk > 0);
      }
      umma::commit(&free_[i % S]);
    };
    for (int i = 0; i < n_my && ok; ++i) {
      ok = mbar_wait(&full[i % S], (i / S) & 1, kBudget, abort_flag);
      if (ok && i > 0) ok = mbar_wait(p_ready, (i - 1) & 1, kBudget, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) give_up(4, i);
        ok = false;
        break;
      }
      umma::fence_after_sync();
      if (umma::elect_one()) {
        if (i > 0) issue_pv(i - 1);
        const uint32_t base = kst_u + (i % S) * SM::kStageBytes;
#pragma unroll 4
        for (int k = 0; k < DQK / 16; ++k) {
          const uint64_t bdesc = umma::smem_desc_sw128(base + (k >> 2) * (kMuTile * 128) + (k & 3) * 32);
          umma::mma_f16_ts(tmem + kSCol, tmem + 8 * k, bdesc, idesc_qk, k > 0);
        }
        umma::commit(s_ready);
      }
      __syncwarp();
    }
    if (ok && n_my > 0) {
      ok = mbar_wait(p_ready, (n_my - 1) & 1, kBudget, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) give_up(5, n_my);
      } else {
        umma::fence_after_sync();
        if (umma::elect_one()) {
          issue_pv(n_my - 1);
          umma::commit(o_final);
        }
        __syncwarp();
        // The "free" arrivals of the last tiles have no consumer.  They are asynchronous: wait for
        // them here, or one could land after the barriers are invalidated below, on shared memory
        // that the block's next task already uses for something else.
        for (int i = max(0, n_my - S); i < n_my; ++i) {
          if (!mbar_wait(&free_[i % S], (i / S) & 1, kBudget, abort_flag)) {
            if (lane == 0) give_up(6, i);
            break;
          }
        }
      }
    }
  }

  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  if (warp == kMuIssueWarp) umma::tmem_dealloc(tmem, 512);
  if (tid == 0) {
    for (int i = 0; i < 2 * S + 5; ++i) mbar_inval(full + i);
  }
}

}  // namespace mdc
