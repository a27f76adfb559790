// Indexer-logits tile: one thread block scores one chunk of one request's
// paged FP4 index-K cache against its 64 (x q_len) query heads and either
// writes the fp32 logits row or keeps the chunk's scores in shared memory and
// emits the exact local top-k.
//
// The tile is a four-role pipeline over 128-token stages (14 warps):
//
//   copy warp (13)     one thread; a page is contiguous in HBM (P x 64 B of
//                      packed E2M1, then the page's block scales), so one 1-D
//                      bulk copy (cp.async.bulk + mbarrier) per page fills a
//                      ring of 8 raw stages in shared memory.
//   decode warps (0-7) thread i owns half of a token row of the stage (warp w:
//                      rows 32*(w%4).., dims 64*(w/4)..): reads its 32 B of
//                      codes and its scales, converts to fp16 with integer
//                      and fp16-multiply instructions only (see
//                      e2m1x8_pairs_f16; the conversion unit is far too slow
//                      for 16 K elements per stage), times the block scale,
//                      exact, and stores the row into TENSOR MEMORY
//                      (tcgen05.st) as the A operand of the next MMA; a ring
//                      of 4 A stages.
//   issue warp (12)    one thread issues eight tcgen05.mma (M=128 tokens,
//                      N=64*q_len heads, K=16, fp16 x fp16 -> fp32) per stage,
//                      A from tensor memory, B = the query block, staged once
//                      in shared memory in the K-major 128-byte-swizzle layout;
//                      two accumulator stages in tensor memory.
//   gate warps (8-11)  thread i reads accumulator row i (tcgen05.ld), applies
//                      relu and the head weights, reduces over heads and emits
//                      the token's score.
//
// Keeping A in tensor memory instead of shared memory matters: the decode
// output (32 KB per stage) and its re-read by the tensor core would otherwise
// triple the shared-memory traffic of a kernel that has to sustain one stage
// per ~400 cycles to follow HBM.
//
// Exactness.  K values (E2M1 x scale) are exact in fp16.  Query rows are
// rescaled per head by a power of two so that the largest element lands in
// [2^14, 2^15) before the fp16 conversion, and the head weight absorbs the
// inverse factor; relu commutes with a positive scale, so the logit is the
// same real number, accumulated in fp32.
//
// Every wait is bounded; a wait that runs out records MDC_DEV_COPY_TIMEOUT,
// raises a block-wide flag all roles poll, and the block leaves through the
// common exit (tensor memory is freed there).
#pragma once

#include "common.cuh"
#include "fp4.cuh"
#include "radix.cuh"
#include "radix_regs.cuh"
#include "umma.cuh"

namespace mdc {

#ifndef MDC_EXP
#define MDC_EXP 0
#endif
#ifdef MDC_TRACE
// Debug builds only: per-role timestamps of block (0,0), [role][tile][begin/end].
__device__ unsigned long long g_logits_trace[4 * 256 * 2];
#define MDC_TRACE_AT(role, tile, which)                                                        \
  do {                                                                                         \
    if (blockIdx.x == 0 && blockIdx.y == 0 && (tile) < 256)                                    \
      g_logits_trace[((role) * 256 + (tile)) * 2 + (which)] = global_timer_ns();               \
  } while (0)
#else
#define MDC_TRACE_AT(role, tile, which) do { } while (0)
#endif

constexpr int kIdxDim = 128;
constexpr int kIdxHeads = 64;
constexpr int kTileTok = 128;    // tokens per pipeline stage (= UMMA M)
constexpr int kRawStages = 8;    // raw page ring
constexpr int kAStages = 4;      // decoded-A ring in tensor memory
constexpr int kTmemCols = 512;
constexpr int kFusedRegE = 32;   // fused top-k keeps up to 256 * 32 scores per query token in registers
constexpr int kLogitsThreads = 480;  // 8 decode + 4 gate + 2 issue + 1 copy warps
constexpr int kGateWarp0 = 8, kIssueWarp = 12, kIssueWarps = 2, kCopyWarp = 14;

template <int FMT, int PAGE>
struct IdxPage {
  static constexpr int kData = PAGE * 64;
  static constexpr int kSf = PAGE * (FMT == MDC_FMT_MXFP4 ? 4 : 8);
  static constexpr int kBytes = kData + kSf;
  static constexpr int kTilePages = kTileTok / PAGE;
  static constexpr int kStageBytes = kTilePages * kBytes;
};

struct LogitsSmem {
  // byte offsets inside the tile's dynamic shared memory (base 1024 B aligned)
  int qb, ring, bars, misc, page_ok, wsc, sel, scores, total;
};

template <int FMT, int PAGE>
__host__ __device__ inline LogitsSmem logits_smem_layout(int q_len, int chunk_tokens, bool fused) {
  LogitsSmem L;
  int off = 0;
  L.qb = off;  // [2 K-halves][N rows][128 B], swizzled; needs 1024 B alignment
  off += 2 * q_len * kIdxHeads * 128;
  L.ring = off;
  off += kRawStages * IdxPage<FMT, PAGE>::kStageBytes;
  off = static_cast<int>(align_up(off, 128));
  L.bars = off;
  off += (2 * kRawStages + 2 * kAStages + 2 * 4) * 8;
  L.misc = off;  // [0] tensor-memory base, [1] abort flag
  off += 16;
  L.wsc = off;
  off += q_len * kIdxHeads * 4;
  off = static_cast<int>(align_up(off, 16));
  L.sel = off;
  off += static_cast<int>(align_up(sizeof(SelectScratch) > sizeof(RegSelectScratch<kFusedRegE>) ? sizeof(SelectScratch)
                                                                                             : sizeof(RegSelectScratch<kFusedRegE>), 16));
  L.page_ok = off;  // one byte per page of the chunk
  off += static_cast<int>(align_up(chunk_tokens / PAGE + 4, 16));
  L.scores = off;
  if (fused) off += q_len * chunk_tokens * 4;
  L.total = static_cast<int>(align_up(off, 128));
  return L;
}

// Prologue: the request's query rows as prescaled fp16 in the UMMA B layout,
// and the matching head weights (halved: the gate computes (x + |x|) * w/2).
// Row r of the request = head r % 64 of query token r / 64.  Called by warps
// 0..7; a half-warp stages one row, lane l of it the dims 8l..8l+7, stored in
// the order 0,4,1,5,2,6,3,7 -- the order in which the decode warps emit the
// elements of a packed 32-bit word (element i is paired with element i+4).
template <int T>
__device__ inline void logits_stage_query(const mdc_logits_params& p, int b, unsigned char* qb, float* wsc) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int hl = lane & 15, sub = lane >> 4;
  constexpr int N = T * kIdxHeads;
  for (int row0 = warp * 2; row0 < N; row0 += kWarps * 2) {
    const int row = row0 + sub;
    float v[8];
    if (p.q_fmt == MDC_Q_BF16) {
      const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(p.q) +
                                 (static_cast<int64_t>(b) * N + row) * kIdxDim + 8 * hl;
      uint4 raw = *reinterpret_cast<const uint4*>(src);
      const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[2 * i] = __uint_as_float(w4[i] << 16);
        v[2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
      }
    } else {
      const uint8_t* src = static_cast<const uint8_t*>(p.q) + (static_cast<int64_t>(b) * N + row) * 64 + 4 * hl;
      const uint32_t eight = *reinterpret_cast<const uint32_t*>(src);
      // atom-ordered scales: 512 B per block of 128 rows
      const uint8_t* sfb = p.q_sf + static_cast<int64_t>(b) * ceil_div(N, 128) * 512 + (row / 128) * 512;
      const int r = row % 128;
      const uint32_t e = sfb[(r % 32) * 16 + (r / 32) * 4 + hl / 4];
      const float sc = __uint_as_float(e << 23);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = e2m1_to_float((eight >> (4 * i)) & 0xf) * sc;
    }
    float m = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    // power-of-two rescale: bring the largest magnitude to [2^14, 2^15)
    int ex = static_cast<int>((__float_as_uint(m) >> 23) & 0xff) - 127;
    int up = 14 - ex;
    up = max(-100, min(100, up));
    if (m == 0.f || !(m < 3.0e38f)) up = 0;
    const float scale = __uint_as_float(static_cast<uint32_t>(127 + up) << 23);
    const float inv = __uint_as_float(static_cast<uint32_t>(127 - up) << 23);
    uint4 out;
    {
      __half2 h0 = __floats2half2_rn(v[0] * scale, v[4] * scale);
      __half2 h1 = __floats2half2_rn(v[1] * scale, v[5] * scale);
      __half2 h2 = __floats2half2_rn(v[2] * scale, v[6] * scale);
      __half2 h3 = __floats2half2_rn(v[3] * scale, v[7] * scale);
      out.x = *reinterpret_cast<uint32_t*>(&h0);
      out.y = *reinterpret_cast<uint32_t*>(&h1);
      out.z = *reinterpret_cast<uint32_t*>(&h2);
      out.w = *reinterpret_cast<uint32_t*>(&h3);
    }
    // dims 8*hl .. 8*hl+7: K-half = hl / 8, 16-byte chunk = hl % 8
    unsigned char* dst = qb + (hl >> 3) * (N * 128) + row * 128 + (((hl & 7) ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = out;
    // 0.5 for the (x + |x|) form of relu, 2^7 for the factor the decode warps leave out
    if (hl == 0) wsc[row] = 64.f * p.weights[static_cast<int64_t>(b) * N + row] * inv;
  }
}

// The tile.  smem: dynamic shared memory base (1024 B aligned), laid out by
// logits_smem_layout.  All kLogitsThreads threads of the block call it.
template <int FMT, int PAGE, int T>
__device__ void logits_tile(const mdc_logits_params& p, int b, int chunk, unsigned char* smem) {
  using PG = IdxPage<FMT, PAGE>;
  constexpr int N = T * kIdxHeads;
  // accumulator ring and MMA interleave: dependent MMAs on one accumulator are
  // latency bound at N = 64, so two stages are issued interleaved when q_len = 1
  constexpr int kAccStages = (T == 1) ? 4 : 2;
  constexpr uint32_t kAccBase = 0, kABase = kAccStages * N;  // tensor-memory columns
  static_assert(kABase + kAStages * 64 <= kTmemCols, "tensor memory over-subscribed");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool fused = p.cand_v != nullptr;
  const int chunk_tokens = p.blocks_per_chunk * PAGE;
  const LogitsSmem L = logits_smem_layout<FMT, PAGE>(T, chunk_tokens, fused);

  unsigned char* qb = smem + L.qb;
  unsigned char* ring = smem + L.ring;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* raw_empty = raw_full + kRawStages;
  uint64_t* a_full = raw_empty + kRawStages;
  uint64_t* a_empty = a_full + kAStages;
  uint64_t* acc_full = a_empty + kAStages;
  uint64_t* acc_empty = acc_full + 4;
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + L.misc);
  volatile uint32_t* abort_flag = misc + 1;
  uint8_t* page_ok = smem + L.page_ok;
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

  // ---------------- prologue
  if (tid == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 8);
    }
    for (int s = 0; s < kAStages; ++s) {
      mbar_init(&a_full[s], 8);
      mbar_init(&a_empty[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], 4);
    }
    misc[1] = 0;
    mbar_fence_init();
  }
  if (warp == kIssueWarp) umma::tmem_alloc(misc, kTmemCols);
  if (warp < kWarps) {
    logits_stage_query<T>(p, b, qb, wsc);
    fence_proxy_async_smem();  // the tensor core reads the query block through the async proxy
  }
  for (int i = tid; i < n_pages; i += kLogitsThreads) {
    const int32_t id = bt[blk0 + i];
    const bool ok = id >= 0 && id < p.num_pages;
    if (!ok) report_failure(p.status, MDC_DEV_BAD_INDEX, id, blk0 + i, 0, 0);
    page_ok[i] = ok;
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = misc[0];
  const float neg_inf = __int_as_float(0xff800000);

  auto give_up = [&](int what, int idx) {
    report_failure(p.status, MDC_DEV_COPY_TIMEOUT, what, idx, 0, 0);
    *abort_flag = 1;
  };

  if (warp == kCopyWarp) {
    // ---------------- copy warp
    if (lane == 0) {
      for (int tile = 0; tile < n_tiles && !*abort_flag; ++tile) {
        const int s = tile % kRawStages;
        if (tile >= kRawStages && !mbar_wait(&raw_empty[s], ((tile / kRawStages) - 1) & 1)) {
          give_up(0, tile);
          break;
        }
        MDC_TRACE_AT(0, tile, 0);
        uint32_t bytes = 0;
#pragma unroll
        for (int pp = 0; pp < PG::kTilePages; ++pp) {
          const int i = tile * PG::kTilePages + pp;
          if (i < n_pages && page_ok[i]) bytes += PG::kBytes;
        }
        if (bytes == 0 || MDC_EXP == 4) {
          mbar_arrive(&raw_full[s]);
          continue;
        }
        mbar_expect_tx(&raw_full[s], bytes);
#pragma unroll
        for (int pp = 0; pp < PG::kTilePages; ++pp) {
          const int i = tile * PG::kTilePages + pp;
          if (i < n_pages && page_ok[i]) {
            bulk_g2s(ring + s * PG::kStageBytes + pp * PG::kBytes,
                     p.kv_pages + static_cast<int64_t>(bt[blk0 + i]) * PG::kBytes, PG::kBytes, &raw_full[s]);
          }
        }
        MDC_TRACE_AT(0, tile, 1);
      }
    }
  } else if (warp >= kIssueWarp && warp < kIssueWarp + kIssueWarps) {
    // ---------------- issue warps (tiles are dealt round-robin to them): all lanes walk the loop together, one elected
    // lane issues (the tensor-core instructions take warp-uniform operands)
    constexpr uint32_t idesc = umma::idesc_f16(kTileTok, N, 0);
    const uint32_t qb_u = smem_u32(qb);
    uint64_t bdesc[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) bdesc[kk] = umma::smem_desc_sw128(qb_u + (kk >> 2) * (N * 128) + (kk & 3) * 32);
    for (int tile = warp - kIssueWarp; tile < n_tiles && !*abort_flag; tile += kIssueWarps) {
      const int a = tile % kAStages, c = tile % kAccStages;
      bool ok = mbar_wait(&a_full[a], (tile / kAStages) & 1);
      if (ok && tile >= kAccStages) ok = mbar_wait(&acc_empty[c], ((tile / kAccStages) - 1) & 1);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) give_up(1, tile);
        break;
      }
      umma::fence_after_sync();
      if (umma::elect_one()) {
        MDC_TRACE_AT(2, tile, 0);
        umma::mma_f16_ts_x8(tmem + kAccBase + c * N, tmem + kABase + a * 64, bdesc, idesc);
        umma::commit(&a_empty[a]);
        umma::commit(&acc_full[c]);
        MDC_TRACE_AT(2, tile, 1);
      }
      __syncwarp();
    }
  } else if (warp < kWarps) {
    // ---------------- decode warps: thread = half a token row of the stage
    const int quad = warp & 3, dh = warp >> 2;  // TMEM lane quadrant, dim half (0: dims 0..63)
    const int row = quad * 32 + lane;
    const int pp = row / PAGE, tok = row % PAGE;
    int prev_a = -1;
    for (int tile = 0; tile < n_tiles && !*abort_flag; ++tile) {
      const int s = tile % kRawStages, a = tile % kAStages;
      if (!mbar_wait(&raw_full[s], (tile / kRawStages) & 1)) {
        if (lane == 0) give_up(3, tile);
        break;
      }
      if (tile >= kAStages && !mbar_wait(&a_empty[a], ((tile / kAStages) - 1) & 1)) {
        if (lane == 0) give_up(4, tile);
        break;
      }
      umma::fence_after_sync();
      if (tid == 0) MDC_TRACE_AT(1, tile, 0);
      const unsigned char* pg = ring + s * PG::kStageBytes + pp * PG::kBytes;
      const int pidx = tile * PG::kTilePages + pp;
      const bool ok = pidx < n_pages && page_ok[pidx];
      uint32_t sc[4];  // fp16x2 block scale of each 16-dim group of this half row, times 2^7
      if (FMT == MDC_FMT_NVFP4) {
        const uint32_t raw = ok ? *reinterpret_cast<const uint32_t*>(pg + PG::kData + tok * 8 + 4 * dh) : 0u;
        const uint32_t x0 = hmul2_u32(e4m3x2_to_f16x2(static_cast<uint16_t>(raw & 0xffff)), kF16x2_2p7);
        const uint32_t x1 = hmul2_u32(e4m3x2_to_f16x2(static_cast<uint16_t>(raw >> 16)), kF16x2_2p7);
        sc[0] = bcast_lo(x0); sc[1] = bcast_hi(x0); sc[2] = bcast_lo(x1); sc[3] = bcast_hi(x1);
      } else {
        const uint32_t raw =
            ok ? *reinterpret_cast<const uint16_t*>(pg + PG::kData + (tok % 32) * 16 + (tok / 32) * 4 + 2 * dh) : 0u;
        sc[0] = sc[1] = ue8m0_to_f16x2_2p7(raw & 0xff);
        sc[2] = sc[3] = ue8m0_to_f16x2_2p7(raw >> 8);
      }
      const uint32_t t_row = tmem + (static_cast<uint32_t>(quad * 32) << 16) + kABase + a * 64 + 32 * dh;
      uint32_t out[2][16];
#pragma unroll
      for (int j = 0; j < 2; ++j) {  // 16-byte chunk j of the half row = 32 dims = 16 columns
        uint4 d = (ok && MDC_EXP != 2 && MDC_EXP != 3) ? *reinterpret_cast<const uint4*>(pg + tok * 64 + 32 * dh + 16 * j) : make_uint4(tile, 0, 0, 0);
        const uint32_t w4[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint32_t s16 = sc[2 * j + (q4 >> 1)];
          uint32_t e[4];
          if (MDC_EXP == 2 || MDC_EXP == 3) { e[0] = e[1] = e[2] = e[3] = w4[q4]; } else
          e2m1x8_pairs_f16(w4[q4], e);  // e[i] = elements (i, i+4) of the word, times 2^-14
#pragma unroll
          for (int i = 0; i < 4; ++i) out[j][4 * q4 + i] = hmul2_u32(e[i], s16);
        }
      }
      // the raw stage is consumed: hand it back before touching tensor memory
      __syncwarp();
      if (lane == 0) mbar_arrive(&raw_empty[s]);
      // stores of the previous stage were issued one iteration ago: retire them now
      if (prev_a >= 0) {
        umma::wait_st();
        umma::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&a_full[prev_a]);
      }
      if (MDC_EXP != 3) {
      umma::tmem_st16(t_row, out[0]);
      umma::tmem_st16(t_row + 16, out[1]);
      }
      prev_a = a;
      if (tid == 0) MDC_TRACE_AT(1, tile, 1);
    }
    if (prev_a >= 0) {
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[prev_a]);
    }
  } else {
    // ---------------- gate warps: thread = token row of the stage
    const int q = warp - kGateWarp0;
    const int row = q * 32 + lane;
    for (int tile = 0; tile < n_tiles && !*abort_flag; ++tile) {
      const int c = tile % kAccStages;
      if (!mbar_wait(&acc_full[c], (tile / kAccStages) & 1)) {
        if (lane == 0) give_up(5, tile);
        break;
      }
      umma::fence_after_sync();
      if (q == 0 && lane == 0) MDC_TRACE_AT(3, tile, 0);
      const uint32_t t_row = tmem + (static_cast<uint32_t>(q * 32) << 16) + kAccBase + c * N;
      float score[T];
#pragma unroll
      for (int t = 0; t < T && MDC_EXP != 1; ++t) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
        for (int hgrp = 0; hgrp < 2; ++hgrp) {
          uint32_t v[32];
          umma::tmem_ld32(t_row + t * kIdxHeads + hgrp * 32, v);
          umma::wait_ld();
          const float4* w4 = reinterpret_cast<const float4*>(wsc + t * kIdxHeads + hgrp * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 w = w4[i];
            const float x0 = __uint_as_float(v[4 * i + 0]), x1 = __uint_as_float(v[4 * i + 1]);
            const float x2 = __uint_as_float(v[4 * i + 2]), x3 = __uint_as_float(v[4 * i + 3]);
            // x + |x| is exactly 0 or 2x; the weighted sums run as packed fp32 pairs
            ffma2(s0, s1, x0 + fabsf(x0), x1 + fabsf(x1), w.x, w.y);
            ffma2(s2, s3, x2 + fabsf(x2), x3 + fabsf(x3), w.z, w.w);
          }
        }
        score[t] = (s0 + s1) + (s2 + s3);
      }
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[c]);
      if (q == 0 && lane == 0) MDC_TRACE_AT(3, tile, 1);
      const int local = tile * kTileTok + row;  // position inside the chunk
      if (local < n_pages * PAGE) {
        const bool ok = page_ok[local / PAGE];
#pragma unroll
        for (int t = 0; t < T; ++t) {
          const float val = ok ? score[t] : neg_inf;
          if (fused) {
            scores[t * chunk_tokens + local] = val;
          } else {
            p.logits[(static_cast<int64_t>(b) * T + t) * p.logits_stride + static_cast<int64_t>(blk0) * PAGE + local] = val;
          }
        }
      }
    }
  }

  // ---------------- common exit of the pipeline
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const bool failed = *abort_flag != 0;
  if (warp == kIssueWarp) umma::tmem_dealloc(tmem, kTmemCols);
  if (tid == 0) {  // the shared memory is reused by the next task of a persistent block
    for (int i = 0; i < 2 * kRawStages + 2 * kAStages + 2 * 4; ++i) mbar_inval(raw_full + i);
  }
  if (warp >= kWarps || failed) return;

  if (fused) {
    const int n_local = n_pages * PAGE;
    const int base_pos = blk0 * PAGE;
    for (int t = 0; t < T; ++t) {
      const float* sc_row = scores + t * chunk_tokens;
      auto src = [&](int pos, bool& valid) -> uint32_t {
        valid = (base_pos + pos) < limit;
        return sortable_u32(sc_row[pos]);
      };
      const int64_t slot0 = ((static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk) * p.top_k;
      int n;
      if (n_local <= kBlockThreads * kFusedRegE) {
        // register-resident select: one pass over shared memory, ties resolved by position
        RegSelectScratch<kFusedRegE>& rsel = *reinterpret_cast<RegSelectScratch<kFusedRegE>*>(smem + L.sel);
        uint32_t key[kFusedRegE];
#pragma unroll
        for (int it = 0; it < kFusedRegE; ++it) {
          const int pos = it * kBlockThreads + tid;
          key[it] = (pos < n_local && (base_pos + pos) < limit) ? max(sortable_u32(sc_row[pos]), 1u) : 0u;
        }
        const Threshold<uint32_t> th = block_select_regs<kFusedRegE>(key, p.top_k, rsel);
        const bool all = th.need_eq == 0x7fffffff;
        int slot[kFusedRegE];
        n = block_emit_regs<kFusedRegE>(
            all ? 0 : th.need_eq, rsel, [&](int it) { return all ? key[it] != 0u : key[it] > th.tau; },
            [&](int it) { return !all && key[it] == th.tau; }, slot);
#pragma unroll
        for (int it = 0; it < kFusedRegE; ++it) {
          if (slot[it] >= 0) {
            const int pos = it * kBlockThreads + tid;
            p.cand_v[slot0 + slot[it]] = sc_row[pos];
            p.cand_i[slot0 + slot[it]] = (base_pos + pos) * p.id_mul + p.id_add;
          }
        }
      } else {
        Threshold<uint32_t> th = block_select_threshold<uint32_t>(src, n_local, p.top_k, sel);
        n = block_emit_selected<uint32_t>(src, n_local, th, sel, [&](int pos, int slot) {
          p.cand_v[slot0 + slot] = sc_row[pos];
          p.cand_i[slot0 + slot] = (base_pos + pos) * p.id_mul + p.id_add;
        });
      }
      if (tid == 0) p.cand_c[(static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk] = n;
    }
  }
}

}  // namespace mdc
