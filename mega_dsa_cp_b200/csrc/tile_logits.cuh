// Indexer-logits tile: one thread block scores one chunk of one request's
// paged FP4 index-K cache against its 64 (x q_len) query heads and either
// writes the fp32 logits row or keeps the chunk's scores in shared memory and
// emits the exact local top-k.
//
// Data path.  Pages are contiguous in HBM (P x 64 B of packed E2M1 followed by
// the page's block scales), so one 1-D bulk copy (cp.async.bulk, mbarrier
// completion) moves a whole page into a ring of 128-token stages; eight warps
// consume a stage, 16 tokens per warp.  Per token the 64 x 128 query
// contraction runs on the tensor cores (mma.sync m16n8k16, fp16 operands, fp32
// accumulation): the K operand is decoded from FP4 straight into A fragments
// in registers (cvt.e2m1x2 -> f16x2, times the block scale, exact), the query
// fragments stay resident in registers for the whole chunk.  The contraction
// index is permuted so that a thread's A fragment for all eight k-steps comes
// from one 16-byte shared-memory load of its token row.
//
// Exactness.  K values (E2M1 x scale) are exact in fp16.  Query rows are
// rescaled per head by a power of two so that the largest element lands in
// [2^14, 2^15) before the fp16 conversion, and the head weight absorbs the
// inverse factor; relu commutes with a positive scale, so the logit is the
// same real number, accumulated in fp32.
#pragma once

#include "common.cuh"
#include "fp4.cuh"
#include "radix.cuh"

namespace mdc {

constexpr int kIdxDim = 128;
constexpr int kIdxHeads = 64;
constexpr int kTileTok = 128;  // tokens per pipeline stage
constexpr int kLogitStages = 8;

template <int FMT, int PAGE>
struct IdxPage {
  static constexpr int kData = PAGE * 64;
  static constexpr int kSf = PAGE * (FMT == MDC_FMT_MXFP4 ? 4 : 8);
  static constexpr int kBytes = kData + kSf;
  static constexpr int kTilePages = kTileTok / PAGE;
  static constexpr int kStageBytes = kTilePages * kBytes;
};

struct LogitsSmem {
  // byte offsets inside the tile's dynamic shared memory
  int ring, bars, page_ok, qh, wsc, sel, scores, total;
};

template <int FMT, int PAGE>
__host__ __device__ inline LogitsSmem logits_smem_layout(int q_len, int chunk_tokens, bool fused) {
  LogitsSmem L;
  int off = 0;
  L.ring = off;
  off += kLogitStages * IdxPage<FMT, PAGE>::kStageBytes;
  off = static_cast<int>(align_up(off, 128));
  L.bars = off;
  off += 2 * kLogitStages * 8;
  L.page_ok = off;
  off += kLogitStages * 4 * 4;
  off = static_cast<int>(align_up(off, 128));
  L.qh = off;
  off += q_len * kIdxHeads * kIdxDim * 2;
  L.wsc = off;
  off += q_len * kIdxHeads * 4;
  off = static_cast<int>(align_up(off, 16));
  L.sel = off;
  off += static_cast<int>(align_up(sizeof(SelectScratch), 16));
  L.scores = off;
  if (fused) off += q_len * chunk_tokens * 4;
  L.total = static_cast<int>(align_up(off, 128));
  return L;
}

// Prologue: stage the request's query rows as prescaled fp16 and the matching
// head weights.  Row r of the request = head r % 64 of query token r / 64.
template <int T>
__device__ inline void logits_stage_query(const mdc_logits_params& p, int b, __half* qh, float* wsc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  constexpr int N = T * kIdxHeads;
  for (int row = warp; row < N; row += kWarps) {
    float v[4];
    if (p.q_fmt == MDC_Q_BF16) {
      const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.q) +
                                 (static_cast<int64_t>(b) * N + row) * kIdxDim + 4 * lane;
      uint2 raw = *reinterpret_cast<const uint2*>(src);
      v[0] = __uint_as_float(raw.x << 16);
      v[1] = __uint_as_float(raw.x & 0xffff0000u);
      v[2] = __uint_as_float(raw.y << 16);
      v[3] = __uint_as_float(raw.y & 0xffff0000u);
    } else {
      const uint8_t* src = static_cast<const uint8_t*>(p.q) + (static_cast<int64_t>(b) * N + row) * 64 + 2 * lane;
      uint32_t two = *reinterpret_cast<const uint16_t*>(src);
      // atom-ordered scales: 512 B per block of 128 rows
      const uint8_t* sfb = p.q_sf + static_cast<int64_t>(b) * ceil_div(N, 128) * 512 + (row / 128) * 512;
      int r = row % 128;
      uint32_t e = sfb[(r % 32) * 16 + (r / 32) * 4 + lane / 8];
      float s = __uint_as_float(e << 23);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = e2m1_to_float((two >> (4 * i)) & 0xf) * s;
    }
    float m = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    m = warp_max(m);
    // power-of-two rescale: bring the largest magnitude to [2^14, 2^15)
    int ex = static_cast<int>((__float_as_uint(m) >> 23) & 0xff) - 127;
    int up = 14 - ex;
    up = max(-100, min(100, up));
    if (m == 0.f || !(m < 3.0e38f)) up = 0;
    float scale = __uint_as_float(static_cast<uint32_t>(127 + up) << 23);
    float inv = __uint_as_float(static_cast<uint32_t>(127 - up) << 23);
    __half2 h01 = __floats2half2_rn(v[0] * scale, v[1] * scale);
    __half2 h23 = __floats2half2_rn(v[2] * scale, v[3] * scale);
    uint2 out;
    out.x = *reinterpret_cast<uint32_t*>(&h01);
    out.y = *reinterpret_cast<uint32_t*>(&h23);
    *reinterpret_cast<uint2*>(qh + row * kIdxDim + 4 * lane) = out;
    if (lane == 0) wsc[row] = p.weights[static_cast<int64_t>(b) * N + row] * inv;
  }
}

// The tile.  smem: dynamic shared memory base (128 B aligned), laid out by
// logits_smem_layout.  All 256 threads of the block call it.
template <int FMT, int PAGE, int T>
__device__ void logits_tile(const mdc_logits_params& p, int b, int chunk, unsigned char* smem) {
  using PG = IdxPage<FMT, PAGE>;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, c = lane & 3;
  const bool fused = p.cand_v != nullptr;
  const int chunk_tokens = p.blocks_per_chunk * PAGE;
  const LogitsSmem L = logits_smem_layout<FMT, PAGE>(T, chunk_tokens, fused);

  unsigned char* ring = smem + L.ring;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* empty = full + kLogitStages;
  int32_t* page_ok = reinterpret_cast<int32_t*>(smem + L.page_ok);
  __half* qh = reinterpret_cast<__half*>(smem + L.qh);
  float* wsc = reinterpret_cast<float*>(smem + L.wsc);
  SelectScratch& sel = *reinterpret_cast<SelectScratch*>(smem + L.sel);
  float* scores = reinterpret_cast<float*>(smem + L.scores);

  const int blk0 = chunk * p.blocks_per_chunk;
  const int seq_len = p.seq_lens ? p.seq_lens[b] : p.max_pages * PAGE;
  const int limit = max(0, seq_len - p.window_exclude);
  // pages this block actually streams: the whole chunk when logits are
  // written out, only pages below the selection limit when fused
  int blk_end = min(blk0 + p.blocks_per_chunk, p.max_pages);
  if (fused) blk_end = min(blk_end, ceil_div(limit, PAGE));
  const int n_pages = max(0, blk_end - blk0);
  const int n_tiles = ceil_div(n_pages, PG::kTilePages);
  const int32_t* bt = p.block_table + static_cast<int64_t>(b) * p.max_pages;

  if (tid == 0) {
    for (int s = 0; s < kLogitStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kWarps);
    }
    mbar_fence_init();
  }
  logits_stage_query<T>(p, b, qh, wsc);
  __syncthreads();

  // producer step: one thread fills stage `tile % kLogitStages`
  auto issue = [&](int tile) {
    const int s = tile % kLogitStages;
    uint32_t bytes = 0;
    int32_t ids[PG::kTilePages];
#pragma unroll
    for (int pp = 0; pp < PG::kTilePages; ++pp) {
      int blk = blk0 + tile * PG::kTilePages + pp;
      int32_t id = -1;
      if (blk < blk_end) {
        id = bt[blk];
        if (id < 0 || id >= p.num_pages) {
          report_failure(p.status, MDC_DEV_BAD_INDEX, id, blk, 0, 0);
          id = -1;
        }
      }
      ids[pp] = id;
      page_ok[s * 4 + pp] = id >= 0;
      if (id >= 0) bytes += PG::kBytes;
    }
    if (bytes == 0) {
      mbar_arrive(&full[s]);
      return;
    }
    mbar_expect_tx(&full[s], bytes);
#pragma unroll
    for (int pp = 0; pp < PG::kTilePages; ++pp) {
      if (ids[pp] >= 0) {
        bulk_g2s(ring + s * PG::kStageBytes + pp * PG::kBytes,
                 p.kv_pages + static_cast<int64_t>(ids[pp]) * PG::kBytes, PG::kBytes, &full[s]);
      }
    }
  };

  if (tid == 0) {
    for (int t0 = 0; t0 < min(n_tiles, kLogitStages - 1); ++t0) issue(t0);
  }

  // query fragments and head weights of this warp's query token
  constexpr int kMtPerWarp = T;               // 8 m-tiles per stage, 8/T warps per query token
  const int tq = (T == 1) ? 0 : (warp >> 2);  // query token served by this warp
  const int mt0 = (T == 1) ? warp : (warp & 3);
  uint32_t bq[8][8][2];
  float wv[8][2];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
    const __half* row = qh + (tq * kIdxHeads + nt * 8 + g) * kIdxDim + 32 * c;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint2 v = *reinterpret_cast<const uint2*>(row + 4 * k);
      bq[nt][k][0] = v.x;
      bq[nt][k][1] = v.y;
    }
    wv[nt][0] = wsc[tq * kIdxHeads + nt * 8 + 2 * c];
    wv[nt][1] = wsc[tq * kIdxHeads + nt * 8 + 2 * c + 1];
  }

  bool failed = false;
  const float neg_inf = __int_as_float(0xff800000);
#pragma unroll 1
  for (int tile = 0; tile < n_tiles; ++tile) {
    const int s = tile % kLogitStages;
    if (!mbar_wait(&full[s], (tile / kLogitStages) & 1)) {
      if (lane == 0) report_failure(p.status, MDC_DEV_COPY_TIMEOUT, s, tile, 0, 0);
      failed = true;
      break;
    }
    const unsigned char* stage = ring + s * PG::kStageBytes;
#pragma unroll
    for (int mi = 0; mi < kMtPerWarp; ++mi) {
      const int mt = mt0 + mi * (8 / T);
      const int row_a = mt * 16 + g, row_b = row_a + 8;
      const int pp = (mt * 16) / PAGE;
      const bool ok = page_ok[s * 4 + pp] != 0;
      const unsigned char* pg = stage + pp * PG::kBytes;
      const int ta = row_a % PAGE, tb = row_b % PAGE;
      uint4 da = *reinterpret_cast<const uint4*>(pg + ta * 64 + 16 * c);
      uint4 db = *reinterpret_cast<const uint4*>(pg + tb * 64 + 16 * c);
      uint32_t sa_lo, sa_hi, sb_lo, sb_hi;
      if (FMT == MDC_FMT_NVFP4) {
        uint32_t xa = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(pg + PG::kData + ta * 8 + 2 * c));
        uint32_t xb = e4m3x2_to_f16x2(*reinterpret_cast<const uint16_t*>(pg + PG::kData + tb * 8 + 2 * c));
        sa_lo = bcast_lo(xa);
        sa_hi = bcast_hi(xa);
        sb_lo = bcast_lo(xb);
        sb_hi = bcast_hi(xb);
      } else {
        sa_lo = sa_hi = ue8m0_to_f16x2(pg[PG::kData + (ta % 32) * 16 + (ta / 32) * 4 + c]);
        sb_lo = sb_hi = ue8m0_to_f16x2(pg[PG::kData + (tb % 32) * 16 + (tb / 32) * 4 + c]);
      }
      float acc[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
      const uint32_t wa[4] = {da.x, da.y, da.z, da.w};
      const uint32_t wb[4] = {db.x, db.y, db.z, db.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint32_t ea[4], eb[4];
        e2m1x8_to_f16x2(wa[j], ea);
        e2m1x8_to_f16x2(wb[j], eb);
        const uint32_t sa = (j < 2) ? sa_lo : sa_hi;
        const uint32_t sb = (j < 2) ? sb_lo : sb_hi;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ea[i] = hmul2_u32(ea[i], sa);
          eb[i] = hmul2_u32(eb[i], sb);
        }
        const uint32_t a0[4] = {ea[0], eb[0], ea[1], eb[1]};
        const uint32_t a1[4] = {ea[2], eb[2], ea[3], eb[3]};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
          mma_f16_16816(acc[nt], a0, bq[nt][2 * j][0], bq[nt][2 * j][1]);
          mma_f16_16816(acc[nt], a1, bq[nt][2 * j + 1][0], bq[nt][2 * j + 1][1]);
        }
      }
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sum_a = fmaf(fmaxf(acc[nt][0], 0.f), wv[nt][0], sum_a);
        sum_a = fmaf(fmaxf(acc[nt][1], 0.f), wv[nt][1], sum_a);
        sum_b = fmaf(fmaxf(acc[nt][2], 0.f), wv[nt][0], sum_b);
        sum_b = fmaf(fmaxf(acc[nt][3], 0.f), wv[nt][1], sum_b);
      }
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1);
      sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
      sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
      if (c < 2) {
        const int row = (c == 0) ? row_a : row_b;
        const float val = ok ? ((c == 0) ? sum_a : sum_b) : neg_inf;
        const int local = tile * kTileTok + row;     // position inside the chunk
        if (local < n_pages * PAGE) {
          if (fused) {
            scores[tq * chunk_tokens + local] = val;
          } else {
            p.logits[(static_cast<int64_t>(b) * T + tq) * p.logits_stride + static_cast<int64_t>(blk0) * PAGE + local] = val;
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (tid == 0) {
      const int nxt = tile + kLogitStages - 1;
      if (nxt < n_tiles) {
        if (nxt >= kLogitStages) {
          // stage of tile-1: free once all eight warps have left it
          if (!mbar_wait(&empty[nxt % kLogitStages], ((nxt / kLogitStages) - 1) & 1)) {
            report_failure(p.status, MDC_DEV_COPY_TIMEOUT, nxt % kLogitStages, -nxt, 0, 0);
          }
        }
        issue(nxt);
      }
    }
  }
  // A failed wait means the copy engine never delivered; every warp saw the
  // same barrier, so every warp leaves.  Nothing else is in flight for a block
  // that completed its loop (each issued stage was waited on).
  __syncthreads();
  if (failed) return;

  if (fused) {
    const int n_local = n_pages * PAGE;
    const int base_pos = blk0 * PAGE;
    for (int t = 0; t < T; ++t) {
      const float* sc_row = scores + t * chunk_tokens;
      auto src = [&](int pos, bool& valid) -> uint32_t {
        valid = (base_pos + pos) < limit;
        return sortable_u32(sc_row[pos]);
      };
      Threshold<uint32_t> th = block_select_threshold<uint32_t>(src, n_local, p.top_k, sel);
      const int64_t slot0 = ((static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk) * p.top_k;
      int n = block_emit_selected<uint32_t>(src, n_local, th, sel, [&](int pos, int slot) {
        p.cand_v[slot0 + slot] = sc_row[pos];
        p.cand_i[slot0 + slot] = (base_pos + pos) * p.id_mul + p.id_add;
      });
      if (tid == 0) p.cand_c[(static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk] = n;
    }
  }
}

}  // namespace mdc
