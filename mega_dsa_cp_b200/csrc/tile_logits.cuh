// Indexer-logits tile: one thread block scores one chunk of one request's
// paged FP4 index-K cache against its 64 (x q_len) query heads and either
// writes the fp32 logits row or keeps the chunk's scores in shared memory and
// emits the exact local top-k.
//
// The tile is a four-role pipeline over 128-token stages:
//
//   copy warp          a page is contiguous in HBM (P x 64 B of packed E2M1,
//                      then the page's block scales), so one 1-D bulk copy
//                      (cp.async.bulk + mbarrier) per page fills a ring of 8
//                      raw stages in shared memory.  Lane l owns one page slot
//                      of the ring; the lanes poll the "empty" barriers of
//                      their stages together and refill whatever is free.
//   decode warps (0-7) two groups of four warps take the even and the odd
//                      stages.  Thread i of a group owns token row i: it reads
//                      the row's 64 B of codes (four 16-byte loads in an order
//                      rotated per lane pair, which makes them bank-conflict
//                      free) and its scales, converts with cvt.f16x2.e2m1x2,
//                      multiplies by the block scale (exact in fp16) and stores
//                      the row into TENSOR MEMORY (tcgen05.st) as the A operand
//                      of the stage's MMA; a ring of 4 A stages.
//   issue warp         one thread issues eight tcgen05.mma (M=128 tokens,
//                      N=64*q_len heads, K=16, fp16 x fp16 -> fp32) per stage,
//                      A from tensor memory, B = the query block, staged once
//                      in shared memory in the K-major 128-byte-swizzle layout;
//                      4 (q_len 1) or 2 accumulator stages in tensor memory.
//   gate warps         GG groups of four warps take stages round-robin; thread
//                      i reads accumulator row i (tcgen05.ld), applies relu and
//                      the head weights, reduces over heads and emits the
//                      token's score.
//
// Keeping A in tensor memory instead of shared memory matters: the decode
// output (32 KB per stage) and its re-read by the tensor core would otherwise
// triple the shared-memory traffic of a kernel that has to sustain one stage
// per ~400 cycles to follow HBM.
//
// What bounds the loop is not arithmetic but the latency of each hand-off
// (an mbarrier probe or a shared-memory atomic costs a warp 100-200 cycles
// even when it succeeds at once), so every role probes the barrier of its
// NEXT stage early, with a non-blocking test whose answer is read one
// iteration later, and signals with predicated instructions instead of
// divergent branches.
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

#include <cooperative_groups.h>

#include "common.cuh"
#include "events.cuh"
#include "fp4.cuh"
#include "radix.cuh"
#include "radix_regs.cuh"
#include "umma.cuh"

namespace mdc {

constexpr int kIdxDim = 128;
constexpr int kIdxHeads = 64;
constexpr int kTileTok = 128;    // tokens per pipeline stage (= UMMA M)
constexpr int kRawStages = 8;    // raw page ring
constexpr int kAStages = 6;      // decoded-A ring in tensor memory (at most)
constexpr int kTmemCols = 512;
constexpr int kFusedRegE = 32;   // fused top-k keeps up to 256 * 32 scores per query token in registers

// Warp layout for DG decode groups and GG gate groups: 4*DG decode, 4*GG gate, issue, copy.
constexpr int logits_threads(int dg, int gg) { return (4 * dg + 4 * gg + 2) * 32; }
constexpr int kLogitsDecodeGroups = 2, kLogitsGateGroups = 2;                      // the stand-alone kernel
constexpr int kLogitsThreads = logits_threads(kLogitsDecodeGroups, kLogitsGateGroups);  

template <int FMT, int PAGE>
struct IdxPage {
  static constexpr int kData = PAGE * 64;
  static constexpr int kSf = PAGE * (FMT == MDC_FMT_MXFP4 ? 4 : 8);
  static constexpr int kBytes = kData + kSf;
  static constexpr int kTilePages = kTileTok / PAGE;
  static constexpr int kStageBytes = kTilePages * kBytes;
};

// Scratch of the cluster-wide row select (read by the other blocks of the cluster).
struct RowSelectScratch {
  uint32_t hist[2][256];   // digit histograms of this block, double buffered over the radix passes
  int32_t cnt_gt, cnt_eq;  // this block's counts above / at the row threshold
  int32_t digit, excl;     // result of a pass: boundary digit, number of keys in higher bins
  int32_t bin_cnt, pad0;   // keys in the boundary bin
  int32_t wsum[kWarps];
};

struct LogitsSmem {
  // byte offsets inside the tile's dynamic shared memory (base 1024 B aligned)
  int qb, ring, bars, misc, page_ok, wsc, sel, row, scores, total;
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
  off += (2 * kRawStages + kAStages) * 8;
  L.misc = off;  // [0] tensor-memory base, [1] abort flag, [4..9] and [10..11] progress counters
  off += 64;
  L.wsc = off;
  off += q_len * kIdxHeads * 4;
  off = static_cast<int>(align_up(off, 16));
  L.sel = off;
  off += static_cast<int>(align_up(sizeof(SelectScratch) > sizeof(RegSelectScratch<kFusedRegE>) ? sizeof(SelectScratch)
                                                                                             : sizeof(RegSelectScratch<kFusedRegE>), 16));
  L.row = off;
  off += static_cast<int>(align_up(sizeof(RowSelectScratch), 16));
  L.page_ok = off;  // page id per page of the chunk (-1 = not usable)
  off += static_cast<int>(align_up((chunk_tokens / PAGE + 4) * 4, 16));
  L.scores = off;
  if (fused) off += q_len * chunk_tokens * 4;
  L.total = static_cast<int>(align_up(off, 128));
  return L;
}

// Prologue: the request's query rows as prescaled fp16 in the UMMA B layout,
// and the matching head weights (halved: the gate computes (x + |x|) * w/2).
// Row r of the request = head r % 64 of query token r / 64.  Called by warps
// 0..7; a half-warp stages one row, lane l of it the dims 8l..8l+7.
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
      __half2 h0 = __floats2half2_rn(v[0] * scale, v[1] * scale);
      __half2 h1 = __floats2half2_rn(v[2] * scale, v[3] * scale);
      __half2 h2 = __floats2half2_rn(v[4] * scale, v[5] * scale);
      __half2 h3 = __floats2half2_rn(v[6] * scale, v[7] * scale);
      out.x = *reinterpret_cast<uint32_t*>(&h0);
      out.y = *reinterpret_cast<uint32_t*>(&h1);
      out.z = *reinterpret_cast<uint32_t*>(&h2);
      out.w = *reinterpret_cast<uint32_t*>(&h3);
    }
    // dims 8*hl .. 8*hl+7: K-half = hl / 8, 16-byte chunk = hl % 8
    unsigned char* dst = qb + (hl >> 3) * (N * 128) + row * 128 + (((hl & 7) ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = out;
    // 0.5 for the (x + |x|) form of relu
    if (hl == 0) wsc[row] = 0.5f * p.weights[static_cast<int64_t>(b) * N + row] * inv;
  }
}

// Exact top-k of one chunk's scores (shared memory).  The scores become sortable keys in place
// (0 = not a candidate); search and position-ordered emit are rolled loops over them: code that a
// block executes once per task is bound by instruction fetch, so it is kept small.  Ties at the
// threshold go to the smaller position.  Returns the number of entries emitted.
template <typename Emit>
__device__ inline int fused_chunk_select(const float* sc_row, uint32_t* keys, int n_local, int base_pos, int limit, int top_k,
                                         SelectScratch& sel, Emit emit) {
  sync_workers();
  for (int pos = threadIdx.x; pos < n_local; pos += kBlockThreads)
    keys[pos] = (base_pos + pos) < limit ? max(sortable_u32(sc_row[pos]), 1u) : 0u;
  sync_workers();
  const Threshold<uint32_t> th = block_select_bits_smem(keys, n_local, top_k, sel);
  return block_emit_keys(keys, n_local, th, sel, emit);
}

// Row-threshold candidate filter (used by the persistent kernel, one query token).  The chunks of a
// request run as separate tasks on different blocks; instead of each emitting the exact top-k of its
// own chunk (a quarter of the chunk at k = 2048 of 8192: long lists, a tree of merges behind them),
// the tasks agree on a lower bound of the ROW's k-th largest score and emit only what reaches it:
//
//   1. every task adds the histogram of its scores (kThrBins bins = the top 12 bits of the sortable
//      key: sign, exponent, three mantissa bits) to the row's histogram in global memory and counts in;
//   2. it waits (bounded) until all n_chunks tasks of the row have counted in, reads the summed
//      histogram and takes the lowest bin B such that the bins >= B hold at least k scores: the
//      row's k-th largest score lies in bin B, so nothing below B can be selected;
//   3. it emits its scores in bins >= B, in position order: over the row about k plus one bin's worth.
//
// The one merge behind the tasks selects exactly.  Waiting on row mates inside a task cannot deadlock:
// tasks are dealt to the blocks in row-major order and every block runs its queue in order, so the
// lowest unfinished row always has all of its tasks running or next in line.  A wait that runs out
// is reported, and the task falls back to the exact top-k of its own chunk, which is always a valid
// candidate set; so does a chunk whose filtered set would not fit its list (heavily tied scores).
constexpr int kThrBins = MDC_THR_BINS, kThrShift = 32 - 12;   // sign, exponent, three mantissa bits
static_assert(kThrBins == 1 << (32 - kThrShift), "bins = the key's upper bits");

// Exact mode (RowThreshold::x set).  The chunk tasks of a row, on ALL ranks of a context-parallel group,
// settle the row's exact top-k between them, so that no merge has to run behind them:
//   a. the last task of a rank's row to count in stores the rank's row histogram into every rank's arena
//      and notifies the row's "histograms" cell there; every task waits for the cp histograms, sums them
//      and finds the boundary bin of the GLOBAL row (one rank: the local histogram is the global one);
//   b. every task stores a slot {scores above the bin, scores inside it, overflow flag, the keys inside
//      it} into every rank's arena and notifies the row's "keys" cell; it waits for all cp x n_chunks slots;
//   c. every task finds the exact threshold among the undecided keys of all slots (the same computation
//      on the same data everywhere), derives each slot's share (ties go to the lower rank, chunk,
//      position) and emits its own share: the gather list of this rank at its local offset, and the
//      selection list at its global offset on every rank.  Its candidate count is then -1 ("published").
// A slot that would overflow (heavily tied scores) makes every task of the row fall back to emitting
// candidates for the merge task, which always remains in the task graph.  All waits are bounded.
constexpr int kUndCap = 512;                      // boundary-bin keys one chunk contributes at most
constexpr int kUndRowCap = 4096;                  // ... and a whole row (the exact search's shared-memory list)
constexpr int kRowSlotBytes = 16 + kUndCap * 4;   // {n_above, n_und, overflow, 0} then the keys
constexpr int kRowHistBytes = MDC_THR_BINS * 4;
constexpr int kRowMaxSlots = 256;

struct RowExact {
  EventSet ev;
  int ev_hist, ev_keys;                        // the row's two cells
  unsigned long long hist_target, keys_target;  // cp and cp * n_chunks arrivals per step
  unsigned char* arena;                        // this rank's arena; rank d's is at arena + arena_offsets[d]
  const int64_t* arena_offsets;
  int64_t hist_off;                            // this step, this row: [cp][bins] u32 (unused with one rank)
  int64_t slot_off;                            // this step, this row: [cp * n_chunks] slots
  int64_t out_off;                             // several ranks: the row's candidate slices (slice 0 receives the
  int64_t slice_bytes;                         //   selection behind its 16-byte cell: [K f32][K i32]; every slice's cell: {-1, total})
  int cp, rank;                                // the ranks of the context-parallel group, and this one
  int pcp, prank;                              // the ranks that settle the row together: (cp, rank), or (1, 0): this rank's
                                               //   tasks settle the rank's own top-k and store it as the rank's candidate
                                               //   list (slice `rank` of the row, a plain count in its cell) on every rank
  float* out_v;                                // one rank: the row of the selection lists, written directly
  int32_t* out_i;
  int32_t* sel_c;
  int32_t* pt;                                 // the row of this rank's gather list (pool rows)
  int pt_cols;
  int32_t* k_valid;
  int row_base, win_slots;
};

struct RowThreshold {
  uint32_t* hist;       // (B, kThrBins) of this phase, zero when the step starts
  uint32_t* hist_next;  // the other phase's histogram: this step zeroes it for the next one
  uint32_t* done;       // (B,) tasks counted in, monotonic over the steps
  uint32_t target;      // value of done[b] when all n_chunks tasks of this step have counted in
  long long budget_ns;
  const RowExact* x;    // exact mode, or nullptr
};

// exclusive prefix sums of n <= 256 ints in shared memory, by one warp (eight consecutive per lane);
// out[n] receives the total
__device__ inline void warp_prefix256(const int* in, int* out, int n, int lane) {
  int c[8], sum = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    c[j] = lane * 8 + j < n ? in[lane * 8 + j] : 0;
    sum += c[j];
  }
  int total;
  int run = warp_excl_scan(sum, lane, &total);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (lane * 8 + j <= n) out[lane * 8 + j] = run;
    run += c[j];
  }
}

struct RowExactSmem {
  int32_t na[kRowMaxSlots], nu[kRowMaxSlots];     // slot headers
  int32_t g[kRowMaxSlots], e[kRowMaxSlots];       // per slot: selected above the threshold, tied at it
  int32_t take[kRowMaxSlots];
  int32_t uo[kRowMaxSlots + 1], eo[kRowMaxSlots + 1], to[kRowMaxSlots + 1];  // prefixes of nu, e, take
  int32_t overflow, my_n, ok, pad;
};

constexpr int kSurvCap = 2048;   // scores of one chunk at or above the row's boundary bin (more: the row falls back)

// Shared-memory scratch of the exact mode behind the chunk's histogram (all inside the idle raw ring).
// (hs, kThrBins words, then this struct: checked against the ring's size where the tile is instantiated)
struct RowExactScratch {
  uint32_t skey[kSurvCap];    // the chunk's survivors (keys in bins >= the boundary bin), in position order
  uint16_t spos[kSurvCap];    // ... and their positions inside the chunk
  uint32_t mylist[kUndCap];   // those inside the boundary bin: this chunk's slot
  uint32_t und[kUndRowCap];   // the undecided keys of the whole row
  RowExactSmem xs;
};

// Steps b and c of the exact mode, after the boundary bin `bin` of the global row is known (0: the row
// holds fewer than top_k scores, everything valid is selected).  n_pass: this chunk's scores in bins >= bin.
// hist2: 2048 words of shared memory for the threshold search (the chunk histogram's space, which is no longer
// needed).  Returns true when the row was published (this task emitted its share), false when the row falls back.
static __device__ __noinline__ bool chunk_publish_row_exact(const RowThreshold& rt, int32_t* status, int b, int chunk, int n_chunks,
                                               const uint32_t* keys, int n_local, int base_pos, int top_k, int id_mul,
                                               int id_add, uint32_t bin, int n_pass, SelectScratch& sel,
                                               RowExactScratch& rs, uint32_t* hist2) {
  const RowExact& x = *rt.x;
  RowExactSmem& xs = rs.xs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int J = x.pcp * n_chunks, me = x.prank * n_chunks + chunk;
  const bool local_only = x.pcp == 1;   // (slots, cells and counters on this rank only)
  const uint32_t floor_tau = bin ? (bin << kThrShift) - 1u : 0u;   // keys > floor_tau: the bins >= bin
  // ---- the chunk's survivors, compacted in position order: every later step works on this short list
  const bool fits = n_pass <= kSurvCap;
  int n_s = 0;
  if (fits) {
    Threshold<uint32_t> th;
    th.tau = floor_tau;
    th.need_eq = 0;
    th.n_sel = n_pass;
    n_s = block_emit_keys(keys, n_local, th, sel, [&](int pos, int slot) {
      if (slot < kSurvCap) {
        rs.skey[slot] = keys[pos];
        rs.spos[slot] = static_cast<uint16_t>(pos);
      }
    });
    n_s = min(n_s, kSurvCap);
  }
  const int n_s4 = (n_s + 3) & ~3;
  if (tid < n_s4 - n_s) rs.skey[n_s + tid] = 0u;
  if (tid == 0) xs.my_n = 0;
  sync_workers();
  // ---- b. this chunk's slot: how many above the bin, and the keys inside it
  int above = 0;
  for (int i0 = 0; i0 < n_s; i0 += kBlockThreads) {
    const int i = i0 + tid;
    const uint32_t v = i < n_s ? rs.skey[i] : 0u;
    const bool in = v != 0u && bin != 0u && (v >> kThrShift) == bin;
    above += v != 0u && !in;
    const uint32_t m = __ballot_sync(0xffffffffu, in);
    if (m != 0u) {
      int base = 0;
      if (lane == 0) base = atomicAdd(&xs.my_n, __popc(m));
      base = __shfl_sync(0xffffffffu, base, 0);
      const int slot = base + __popc(m & ((1u << lane) - 1u));
      if (in && slot < kUndCap) rs.mylist[slot] = v;
    }
  }
  above = __reduce_add_sync(0xffffffffu, above);
  if (lane == 0) sel.weq[warp] = above;
  sync_workers();
  int n_above = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) n_above += sel.weq[w];
  const int n_und = xs.my_n;
  const bool over = !fits || n_und > kUndCap;
  {
    const int n_keys = over ? 0 : n_und;
    const int64_t at = x.slot_off + static_cast<int64_t>(me) * kRowSlotBytes;
    for (int d = 0; d < x.pcp; ++d) {
      unsigned char* dst = x.arena + x.arena_offsets[local_only ? x.rank : d] + at;
      if (tid == 0) *reinterpret_cast<int4*>(dst) = make_int4(n_above, n_keys, over ? 1 : 0, 0);
      for (int i = tid; i < n_keys; i += kBlockThreads) reinterpret_cast<uint32_t*>(dst + 16)[i] = rs.mylist[i];
    }
    if (!local_only) __threadfence_system();
    else __threadfence();
    sync_workers();
    if (tid == 0) {
      for (int d = 0; d < x.pcp; ++d) x.ev.notify_1t(x.ev_keys, local_only ? x.rank : d);
      unsigned long long seen = 0;
      const bool ok = x.ev.poll_1t(x.ev_keys, x.keys_target, !local_only, rt.budget_ns, &seen, 64);
      if (!ok) report_failure(status, MDC_DEV_WAIT_TIMEOUT, -1000 - b, chunk, seen, x.keys_target);
      xs.ok = ok ? 1 : 0;
      xs.overflow = 0;
    }
    sync_workers();
    if (!xs.ok) return false;
  }
  // ---- c. all slots -> the exact threshold and every slot's share
  const unsigned char* slots = x.arena + x.slot_off;
  for (int j = tid; j < J; j += kBlockThreads) {
    const uint4 h = ld_sys_u4(reinterpret_cast<const uint4*>(slots + static_cast<int64_t>(j) * kRowSlotBytes));
    xs.na[j] = static_cast<int>(h.x);
    xs.nu[j] = min(max(static_cast<int>(h.y), 0), kUndCap);
    if (h.z != 0u) xs.overflow = 1;
  }
  sync_workers();
  if (warp == 0) warp_prefix256(xs.nu, xs.uo, J, lane);
  if (warp == 1) warp_prefix256(xs.na, xs.to, J, lane);   // (to: scratch here, its total is the count above the bin)
  sync_workers();
  const int U = xs.uo[J], A = xs.to[J];
  if (xs.overflow != 0 || U > kUndRowCap) return false;
  uint32_t* und = rs.und;
  for (int i0 = tid; i0 < U; i0 += 4 * kBlockThreads) {   // (independent loads: four in flight per thread)
    const float* src[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = min(i0 + u * kBlockThreads, U - 1);
      int lo = 0, hi = J;   // the slot j with uo[j] <= i < uo[j + 1]
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (xs.uo[mid] <= i) lo = mid;
        else hi = mid;
      }
      src[u] = reinterpret_cast<const float*>(slots + static_cast<int64_t>(lo) * kRowSlotBytes + 16) + (i - xs.uo[lo]);
    }
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) v[u] = ld_sys_f32(src[u]);
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i0 + u * kBlockThreads < U) und[i0 + u * kBlockThreads] = __float_as_uint(v[u]);
  }
  const int U4 = (U + 3) & ~3;
  if (tid < U4 - U) und[U + tid] = 0u;
  sync_workers();
  uint32_t tau = floor_tau;   // bin == 0, or the whole bin is taken: everything above the floor
  int need_eq = 0;
  if (bin != 0u) {
    const int need = top_k - A;   // 1 <= need <= U by the choice of the bin
    if (need > 0 && need < U) {
      const Threshold<uint32_t> th = block_select_hist_smem(und, U4, need, sel, hist2);
      if (th.need_eq != 0x7fffffff) {
        tau = th.tau;
        need_eq = th.need_eq;
      }
    }
  }
  // per slot: keys above the threshold and tied at it (one warp per slot in turn)
  for (int j = warp; j < J; j += kWarps) {
    int g = 0, e = 0;
    const int n = xs.nu[j], o = xs.uo[j];
    for (int i = lane; i < n; i += 32) {
      const uint32_t v = und[o + i];
      g += v > tau;
      e += v == tau;
    }
    g = __reduce_add_sync(0xffffffffu, g);
    e = __reduce_add_sync(0xffffffffu, e);
    if (lane == 0) {
      xs.g[j] = xs.na[j] + g;
      xs.e[j] = need_eq > 0 ? e : 0;
    }
  }
  sync_workers();
  if (warp == 0) warp_prefix256(xs.e, xs.eo, J, lane);
  sync_workers();
  for (int j = tid; j < J; j += kBlockThreads) xs.take[j] = xs.g[j] + min(xs.e[j], max(0, need_eq - xs.eo[j]));
  sync_workers();
  if (warp == 0) warp_prefix256(xs.take, xs.to, J, lane);
  sync_workers();
  const int my_eq = min(xs.e[me], max(0, need_eq - xs.eo[me]));
  const int off_g = xs.to[me], off_l = xs.to[me] - xs.to[x.prank * n_chunks];
  const int total = xs.to[J], local_total = xs.to[(x.prank + 1) * n_chunks] - xs.to[x.prank * n_chunks];
  const bool as_list = local_only && x.cp > 1;   // the result is this rank's candidate list, not the selection
  const int64_t out_at = x.out_off + (as_list ? static_cast<int64_t>(x.rank) * x.slice_bytes : 0);
  // ---- this chunk's share, from its survivor list (position order)
  Threshold<uint32_t> th;
  th.tau = tau;
  th.need_eq = my_eq;
  th.n_sel = xs.take[me];
  const int K = top_k;
  block_emit_keys(rs.skey, n_s4, th, sel, [&](int idx, int slot) {
    const uint32_t kv = rs.skey[idx];
    const int pos = rs.spos[idx];
    const float v = __uint_as_float((kv & 0x80000000u) ? (kv ^ 0x80000000u) : ~kv);
    const int id = (base_pos + pos) * id_mul + id_add;
    if (!as_list && off_l + slot < x.pt_cols) x.pt[off_l + slot] = x.row_base + base_pos + pos;
    const int o = off_g + slot;
    if (o < K) {
      if (x.cp == 1) {
        x.out_v[o] = v;
        x.out_i[o] = id;
      } else {
        for (int d = 0; d < x.cp; ++d) {
          unsigned char* dst = x.arena + x.arena_offsets[d] + out_at;   // slice: [cell 16 B][K f32][K i32]
          reinterpret_cast<float*>(dst + 16)[o] = v;
          reinterpret_cast<int32_t*>(dst + 16 + static_cast<int64_t>(K) * 4)[o] = id;
        }
      }
    }
  });
  if (tid == 0) {
    if (chunk == 0 && !as_list) {
      *x.k_valid = x.win_slots + min(local_total, x.pt_cols);
      if (x.cp == 1) *x.sel_c = min(total, K);
    }
    if (as_list) {   // the rank's list on every rank: its length, by the row's first task
      if (chunk == 0)
        for (int d = 0; d < x.cp; ++d)
          *reinterpret_cast<int4*>(x.arena + x.arena_offsets[d] + out_at) = make_int4(min(total, K), 0, 0, 0);
    } else if (x.cp > 1) {  // this task's slice on every rank: "published", and the length of the selection
      for (int d = 0; d < x.cp; ++d)
        *reinterpret_cast<int4*>(x.arena + x.arena_offsets[d] + x.out_off + static_cast<int64_t>(me) * x.slice_bytes) =
            make_int4(-1, min(total, K), 0, 0);
    }
  }
  return true;
}

template <typename Emit>
__device__ inline int chunk_emit_above_row_threshold(const RowThreshold& rt, int32_t* status, int b, int chunk, int n_chunks,
                                                     const float* sc_row, uint32_t* keys, int n_local, int base_pos, int limit,
                                                     int top_k, SelectScratch& sel, uint32_t* hs, Emit emit, int id_mul = 1,
                                                     int id_add = 0) {
  constexpr int PER = kThrBins / kBlockThreads;   // bins a thread owns in the scan from the top
  static_assert(kThrBins % (4 * kBlockThreads) == 0, "the bin scan reads whole 16-byte pieces");
  const int tid = threadIdx.x;
  sync_workers();
  for (int i = tid; i < kThrBins; i += kBlockThreads) hs[i] = 0u;
  sync_workers();
  for (int pos = tid; pos < n_local; pos += kBlockThreads) {
    const uint32_t k = (base_pos + pos) < limit ? max(sortable_u32(sc_row[pos]), 1u) : 0u;
    keys[pos] = k;
    if (k) atomicAdd(&hs[k >> kThrShift], 1u);   // (a __match_any_sync aggregation per warp was measured: 2.4x slower)
  }
  sync_workers();
  uint32_t* gh = rt.hist + static_cast<int64_t>(b) * kThrBins;
  for (int i = tid; i < kThrBins; i += kBlockThreads) {
    const uint32_t h = hs[i];
    if (h) atomicAdd(&gh[i], h);
  }
  {  // this task's slice of the next step's histogram
    const int per = ceil_div(kThrBins, n_chunks);
    uint32_t* gn = rt.hist_next + static_cast<int64_t>(b) * kThrBins;
    for (int i = chunk * per + tid; i < min(kThrBins, (chunk + 1) * per); i += kBlockThreads) gn[i] = 0u;
  }
  __threadfence();
  sync_workers();
  const RowExact* x = rt.x;
  const bool many = x != nullptr && x->pcp > 1;   // the ranks settle the row together: the histograms are exchanged
  if (tid == 0) {
    const uint32_t before = atomicAdd(&rt.done[b], 1u);
    sel.hist_bnd = (before + 1u == rt.target) ? 1 : 0;   // the last task of this rank's row to count in
    bool ok = true;
    if (!many) {
      const unsigned long long t0 = global_timer_ns();
      while (static_cast<int32_t>(*reinterpret_cast<volatile uint32_t*>(&rt.done[b]) - rt.target) < 0) {
        nanosleep(64);
        if (static_cast<long long>(global_timer_ns() - t0) > rt.budget_ns) {
          ok = false;
          break;
        }
      }
      __threadfence();
      if (!ok) report_failure(status, MDC_DEV_WAIT_TIMEOUT, -1 - b, chunk, rt.done[b], rt.target);
    }
    sel.bnd = ok ? 0 : -1;
  }
  sync_workers();
  if (many) {
    if (sel.hist_bnd) {  // this rank's row histogram is complete: it goes to every rank, then one notify each
      __threadfence();
      const int64_t at = x->hist_off + static_cast<int64_t>(x->rank) * kRowHistBytes;
      for (int i = tid; i < kThrBins / 4; i += kBlockThreads) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(gh) + i);
        for (int d = 0; d < x->cp; ++d) reinterpret_cast<uint4*>(x->arena + x->arena_offsets[d] + at)[i] = v;
      }
      __threadfence_system();
      sync_workers();
      if (tid == 0)
        for (int d = 0; d < x->cp; ++d) x->ev.notify_1t(x->ev_hist, d);
    }
    if (tid == 0) {
      unsigned long long seen = 0;
      const bool ok = x->ev.poll_1t(x->ev_hist, x->hist_target, true, rt.budget_ns, &seen, 64);
      if (!ok) report_failure(status, MDC_DEV_WAIT_TIMEOUT, -500 - b, chunk, seen, x->hist_target);
      sel.bnd = ok ? 0 : -1;
    }
    sync_workers();
  }
  bool use_filter = sel.bnd >= 0;
  sync_workers();
  if (use_filter) {
    // thread t owns the bins kThrBins-1-PER*t .. kThrBins-PER-PER*t, scanned from the top
    uint32_t c[PER];
    int local = 0;
#pragma unroll
    for (int j = 0; j < PER; ++j) c[j] = 0u;
    const int first = kThrBins - PER - PER * tid;   // lowest bin of this thread, a multiple of 4
    for (int r = 0; r < (many ? x->cp : 1); ++r) {
      const uint4* src = many ? reinterpret_cast<const uint4*>(x->arena + x->hist_off + static_cast<int64_t>(r) * kRowHistBytes)
                              : reinterpret_cast<const uint4*>(gh);
      src += first / 4;
#pragma unroll
      for (int q = 0; q < PER / 4; ++q) {
        const uint4 v = many ? ld_sys_u4(src + q) : __ldcg(src + q);   // bins first + 4q .. first + 4q + 3, ascending
        c[PER - 1 - 4 * q] += v.x;
        c[PER - 2 - 4 * q] += v.y;
        c[PER - 3 - 4 * q] += v.z;
        c[PER - 4 - 4 * q] += v.w;
      }
    }
#pragma unroll
    for (int j = 0; j < PER; ++j) local += static_cast<int>(c[j]);
    const int lane = tid & 31, warp = tid >> 5;
    int wtot;
    int cum = warp_excl_scan(local, lane, &wtot);
    if (lane == 0) sel.wgt[warp] = wtot;
    sync_workers();
    for (int w = 0; w < warp; ++w) cum += sel.wgt[w];
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (cum < top_k && cum + static_cast<int>(c[j]) >= top_k) sel.bnd = kThrBins - 1 - PER * tid - j;  // (one thread at most)
      cum += static_cast<int>(c[j]);
    }
    sync_workers();
    const uint32_t bin = static_cast<uint32_t>(sel.bnd);   // 0 when the row holds fewer than k scores: everything passes
    // this chunk's scores in the bins >= bin
    int mine = 0;
    for (int i = tid; i < kThrBins; i += kBlockThreads) mine += static_cast<uint32_t>(i) >= bin ? static_cast<int>(hs[i]) : 0;
    mine = __reduce_add_sync(0xffffffffu, mine);
    sync_workers();
    if (lane == 0) sel.weq[warp] = mine;
    sync_workers();
    int n_pass = 0;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) n_pass += sel.weq[w];
    sync_workers();
    if (x != nullptr) {
      if (chunk_publish_row_exact(rt, status, b, chunk, n_chunks, keys, n_local, base_pos, top_k, id_mul, id_add, bin, n_pass,
                                  sel, *reinterpret_cast<RowExactScratch*>(hs + kThrBins), hs))
        return -1;
      sync_workers();
    }
    if (n_pass <= top_k) {   // the chunk's share fits its list
      Threshold<uint32_t> th;
      th.tau = bin ? (bin << kThrShift) - 1u : 0u;
      th.need_eq = 0;
      th.n_sel = n_pass;
      return block_emit_keys(keys, n_local, th, sel, emit);
    }
  }
  const Threshold<uint32_t> th = block_select_bits_smem(keys, n_local, top_k, sel);
  return block_emit_keys(keys, n_local, th, sel, emit);
}

// Exact top-k of a whole request row across the blocks of a thread-block
// cluster (block rank = chunk).  Every block holds its chunk's scores in shared
// memory; the k-th largest key of the row is found by a 4-pass byte radix
// search whose histograms are summed over the cluster through distributed
// shared memory (every block computes the same sums, so no result has to be
// sent back), then each block emits its selected entries in position order at
// the offset given by the lower ranks' counts.  Ties at the threshold go to the
// smaller position.  The number of cluster barriers is fixed (6 per query
// token) and does not depend on the data.  Called by the 256 worker threads of
// every block of the cluster; n_local = 0 for a block that has nothing to offer.
template <int T>
__device__ void logits_row_select(const mdc_logits_params& p, int b, int chunk, int n_local, int base_pos, int limit,
                                  int chunk_tokens, const float* scores, RegSelectScratch<kFusedRegE>& rsel,
                                  RowSelectScratch& rs) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int nr = static_cast<int>(cluster.num_blocks());
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  constexpr int E = kFusedRegE;
  for (int t = 0; t < T; ++t) {
    const float* sc_row = scores + t * chunk_tokens;
    uint32_t key[E];
#pragma unroll
    for (int it = 0; it < E; ++it) {
      const int pos = it * kBlockThreads + tid;
      key[it] = (pos < n_local && (base_pos + pos) < limit) ? max(sortable_u32(sc_row[pos]), 1u) : 0u;
    }
    uint32_t prefix = 0u;
    int kk = p.top_k;
    bool all = false;
    int low_bits = 0;  // undecided low bits when the search stopped early (the boundary bin is taken whole)
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass, buf = pass & 1;
      rs.hist[buf][tid] = 0u;
      sync_workers();
      // run-length over this thread's keys: equal digits in a row cost one atomic
      uint32_t run_d = 0xffffffffu, run_n = 0u;
#pragma unroll
      for (int it = 0; it < E; ++it) {
        const bool in = key[it] != 0u && (pass == 0 || (key[it] >> (shift + 8)) == prefix);
        const uint32_t d = in ? (key[it] >> shift) & 255u : 0xffffffffu;
        if (d != run_d) {
          if (run_n) atomicAdd(&rs.hist[buf][run_d], run_n);
          run_d = d;
          run_n = 0u;
        }
        run_n += in;
      }
      if (run_n) atomicAdd(&rs.hist[buf][run_d], run_n);
      cluster.sync();
      // thread tid owns bin 255 - tid, summed over the cluster
      const int bin = 255 - tid;
      uint32_t g = 0u;
      for (int r = 0; r < nr; ++r) g += cluster.map_shared_rank(&rs.hist[buf][0], r)[bin];
      // inclusive scan over tid = number of keys in bins >= bin
      uint32_t inc = g;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += y;
      }
      if (lane == 31) rs.wsum[warp] = static_cast<int32_t>(inc);
      if (tid == 0) rs.digit = -1;
      sync_workers();
      uint32_t before = 0u, total = 0u;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        if (w < warp) before += static_cast<uint32_t>(rs.wsum[w]);
        total += static_cast<uint32_t>(rs.wsum[w]);
      }
      inc += before;
      const uint32_t exc = inc - g;
      if (!all && static_cast<int>(exc) < kk && kk <= static_cast<int>(inc)) {
        rs.digit = bin;
        rs.excl = static_cast<int32_t>(exc);
        rs.bin_cnt = static_cast<int32_t>(g);
      }
      sync_workers();
      if (pass == 0 && static_cast<int>(total) <= kk) all = true;  // fewer valid entries than k: take all
      if (all) break;  // (every block of the cluster sees the same sums and takes the same exit)
      prefix = (prefix << 8) | static_cast<uint32_t>(rs.digit);
      kk -= rs.excl;
      if (rs.bin_cnt == kk && shift > 0) {  // the whole boundary bin is selected: no finer digit needed
        low_bits = shift;
        break;
      }
    }
    // Threshold key: entries above it are selected outright, kk of those equal to it in position
    // order.  After an early stop everything at or above prefix << low_bits is selected.
    uint32_t tau = all ? 0u : prefix;
    if (low_bits > 0) {
      tau = (prefix << low_bits) - 1u;
      kk = 0;
      if ((prefix << low_bits) == 0u) all = true;
    }
    int c_gt = 0, c_eq = 0;
#pragma unroll
    for (int it = 0; it < E; ++it) {
      c_gt += all ? key[it] != 0u : key[it] > tau;
      c_eq += !all && key[it] == tau;
    }
    c_gt = __reduce_add_sync(0xffffffffu, c_gt);
    c_eq = __reduce_add_sync(0xffffffffu, c_eq);
    if (tid == 0) rs.cnt_gt = rs.cnt_eq = 0;
    sync_workers();
    if (lane == 0) {
      atomicAdd(&rs.cnt_gt, c_gt);
      atomicAdd(&rs.cnt_eq, c_eq);
    }
    cluster.sync();
    int gt_before = 0, eq_before = 0, gt_all = 0, eq_all = 0, eq_mine = 0;
    for (int r = 0; r < nr; ++r) {
      const RowSelectScratch* o = cluster.map_shared_rank(&rs, r);
      const int g1 = o->cnt_gt, e1 = o->cnt_eq;
      if (r < chunk) {
        gt_before += g1;
        eq_before += e1;
      }
      if (r == chunk) eq_mine = e1;
      gt_all += g1;
      eq_all += e1;
    }
    const int need_row = all ? 0 : kk;
    const int need = max(0, min(need_row - eq_before, eq_mine));   // ties this block contributes
    const int base = gt_before + min(eq_before, need_row);         // entries selected in lower chunks
    // position-ordered emit as a rolled loop over the scores (compact code: it runs once per block)
    const int64_t out0 = (static_cast<int64_t>(b) * T + t) * p.top_k;
    Threshold<uint32_t> th;
    th.tau = tau;
    th.need_eq = need;
    th.n_sel = 0;
    block_emit_selected<uint32_t>(
        [&](int pos, bool& valid) {
          valid = (base_pos + pos) < limit;
          return max(sortable_u32(sc_row[pos]), 1u);
        },
        n_local, th, *reinterpret_cast<SelectScratch*>(&rsel),
        [&](int pos, int slot) {
          const int o = base + slot;
          if (o < p.top_k) {
            p.row_v[out0 + o] = sc_row[pos];
            p.row_i[out0 + o] = (base_pos + pos) * p.id_mul + p.id_add;
          }
        });
    if (chunk == 0 && tid == 0) p.row_c[static_cast<int64_t>(b) * T + t] = min(p.top_k, gt_all + min(eq_all, need_row));
    cluster.sync();  // counts and histograms are reused by the next query token; nobody leaves while a peer may read
  }
}

// The tile.  smem: dynamic shared memory base (1024 B aligned), laid out by
// logits_smem_layout.  All logits_threads(GG) threads of the block call it.
template <int FMT, int PAGE, int T, int DG, int GG, bool ROWK = false>
__device__ void logits_tile(const mdc_logits_params& p, int b, int chunk, unsigned char* smem, const RowThreshold* rt = nullptr) {
  using PG = IdxPage<FMT, PAGE>;
  constexpr int N = T * kIdxHeads;
  constexpr int kThreads = logits_threads(DG, GG);
  constexpr int kGateWarp0 = 4 * DG, kIssueWarp = kGateWarp0 + 4 * GG, kCopyWarp = kIssueWarp + 1;
  // Tensor memory: two accumulator stages of N columns (a gate warp frees its stage as soon as
  // the row is in registers), then kASt decoded-A stages of 64 columns (128 fp16 per row):
  // 512 columns for q_len 1 and 2.
  constexpr int kAccSt = 2;
  constexpr int kASt = (T == 1) ? 6 : 4;
  constexpr uint32_t kAccBase = 0, kABase = kAccSt * N;
  static_assert(kABase + kASt * 64 <= kTmemCols && kASt <= kAStages && kASt > DG, "tensor memory over-subscribed");
  // A group probes the barriers of its next stage one iteration early with a parity test; the
  // answer is only unambiguous if the stage's previous user was the same group.
  static_assert(kRawStages % DG == 0 && kASt % DG == 0 && kASt % GG == 0, "ring sizes must be multiples of the group counts");
  static_assert(kRawStages * PG::kTilePages <= 32, "one copy-warp lane per page of the raw ring");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const bool row_mode = ROWK && p.row_v != nullptr;
  const bool fused = p.cand_v != nullptr || row_mode;
  const int chunk_tokens = p.blocks_per_chunk * PAGE;
  const LogitsSmem L = logits_smem_layout<FMT, PAGE>(T, chunk_tokens, fused);

  unsigned char* qb = smem + L.qb;
  unsigned char* ring = smem + L.ring;
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(smem + L.bars);
  uint64_t* raw_empty = raw_full + kRawStages;
  uint64_t* mma_done = raw_empty + kRawStages;  // [kAStages]: stage t % 4 finished on the tensor core
  uint32_t* misc = reinterpret_cast<uint32_t*>(smem + L.misc);
  volatile uint32_t* abort_flag = misc + 1;
  uint32_t* a_cnt = misc + 4;    // [kAStages] decode warps that finished writing the A stage (monotonic)
  uint32_t* acc_cnt = misc + 10;  // [kAccSt] gate warps that finished reading the accumulator stage (monotonic)
  int32_t* page_id = reinterpret_cast<int32_t*>(smem + L.page_ok);
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
  const int n_tiles = ceil_div(n_pages, PG::kTilePages);  // pipeline stages of this block
  const int32_t* bt = p.block_table + static_cast<int64_t>(b) * p.max_pages;
  constexpr long long kBudget = 1ll << 31;  // clock cycles a role waits before it gives up

  // ---------------- prologue
  if (tid == 0) {
    for (int s = 0; s < kRawStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], 4);
    }
    for (int s = 0; s < kAStages; ++s) mbar_init(&mma_done[s], 1);
    for (int i = 1; i < 16; ++i) misc[i] = 0;
    mbar_fence_init();
  }
  if (warp == kIssueWarp) umma::tmem_alloc(misc, kTmemCols);
  if (warp < kWarps) {
    logits_stage_query<T>(p, b, qb, wsc);
    fence_proxy_async_smem();  // the tensor core reads the query block through the async proxy
  }
  for (int i = tid; i < n_pages + 4; i += kThreads) {  // (+4: the slots behind the last page read as unusable)
    int32_t id = -1;
    if (i < n_pages) {
      id = bt[blk0 + i];
      if (id < 0 || id >= p.num_pages) {
        report_failure(p.status, MDC_DEV_BAD_INDEX, id, blk0 + i, 0, 0);
        id = -1;
      }
    }
    page_id[i] = id;
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
    // ---------------- copy warp: lane l owns page l % kTilePages of raw stage l / kTilePages.
    // The lanes poll their stages' "empty" barriers together without blocking and every lane
    // whose stage is free issues its page's bulk copy in the same instruction, so the ring is
    // refilled in whatever order the decode warps release it and no single thread serialises
    // the address arithmetic of all pages.
    const int s = lane / PG::kTilePages, pp = lane % PG::kTilePages;
    int tile = (s < kRawStages) ? s : n_tiles;
    const uint64_t stream_policy = l2_policy_evict_first();  // the index cache is read once per step
    long long t_last = clock64();
    while (__any_sync(0xffffffffu, tile < n_tiles) && !*abort_flag) {
      bool ready = false;
      if (tile < n_tiles) ready = tile < kRawStages || mbar_test(&raw_empty[s], ((tile / kRawStages) - 1) & 1);
      ready = __shfl_sync(0xffffffffu, ready, lane - pp);  // the lanes of a stage act on one answer
      if (ready) {
        const int i0 = tile * PG::kTilePages;
        if (pp == 0) {
          uint32_t bytes = 0;
#pragma unroll
          for (int k = 0; k < PG::kTilePages; ++k) bytes += page_id[i0 + k] >= 0 ? PG::kBytes : 0;
          if (bytes == 0) mbar_arrive(&raw_full[s]);
          else mbar_expect_tx(&raw_full[s], bytes);
        }
        const int32_t id = page_id[i0 + pp];
        if (id >= 0) {
          bulk_g2s_hint(ring + s * PG::kStageBytes + pp * PG::kBytes, p.kv_pages + static_cast<int64_t>(id) * PG::kBytes,
                        PG::kBytes, &raw_full[s], stream_policy);
        }
        tile += kRawStages;
      }
      if (__any_sync(0xffffffffu, ready)) {
        t_last = clock64();
        continue;
      }
      __nanosleep(200);  // nothing to refill: do not spin hot beside the decode warps
      if (clock64() - t_last > kBudget) {
        if (lane == 0) give_up(0, tile);
        break;
      }
    }
  } else if (warp == kIssueWarp) {
    // ---------------- issue warp: all lanes walk the loop together, one elected lane issues
    // (the tensor-core instructions take warp-uniform operands)
    constexpr uint32_t idesc = umma::idesc_f16(kTileTok, N, 0);
    const uint32_t qb_u = smem_u32(qb);
    uint64_t bdesc[8];
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) bdesc[kk] = umma::smem_desc_sw128(qb_u + (kk >> 2) * (N * 128) + (kk & 3) * 32);
    for (int tile = 0; tile < n_tiles; ++tile) {
      const int a = tile % kASt, c = tile % kAccSt;
      // progress counters instead of mbarriers here: an mbarrier wait costs this
      // thread ~150 cycles even when the phase is long complete
      bool ok = counter_wait(&a_cnt[a], 4u * (tile / kASt + 1), kBudget, abort_flag);
      if (ok && tile >= kAccSt) ok = counter_wait(&acc_cnt[c], 4u * (tile / kAccSt), kBudget, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) give_up(1, tile);
        break;
      }
      umma::fence_after_sync();
      if (umma::elect_one()) {
        umma::mma_f16_ts_x8(tmem + kAccBase + c * N, tmem + kABase + a * 64, bdesc, idesc);
        umma::commit(&mma_done[a]);
      }
      __syncwarp();
    }
  } else if (warp < kGateWarp0) {
    // ---------------- decode warps: thread = token row; group g (warps 4g..4g+3) takes the stages g, g + DG, ...
    const int quad = warp & 3, grp = warp >> 2;  // TMEM lane quadrant, group
    const int row = quad * 32 + lane;
    const int pp = row / PAGE, tok = row % PAGE;
    const int rot = (lane >> 1) & 3;  // chunk rotation: lanes 2m, 2m+1 start at chunk m (no bank conflicts)
    const uint32_t t_row = tmem + (static_cast<uint32_t>(quad * 32) << 16) + kABase;
    // answers of the early probes for the next stage (true = known complete)
    bool raw_ok = false, a_ok = true;
    for (int tile = grp; tile < n_tiles; tile += DG) {
      const int s = tile % kRawStages, a = tile % kASt;
      if (!raw_ok && !mbar_wait(&raw_full[s], (tile / kRawStages) & 1, kBudget, abort_flag)) {
        if (lane == 0) give_up(3, tile);
        break;
      }
      const unsigned char* pg = ring + s * PG::kStageBytes + pp * PG::kBytes;
      const bool ok = page_id[tile * PG::kTilePages + pp] >= 0;
      uint4 d[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        d[j] = ok ? *reinterpret_cast<const uint4*>(pg + tok * 64 + 16 * ((j + rot) & 3)) : make_uint4(0, 0, 0, 0);
      uint2 raw_sf = make_uint2(0u, 0u);  // the row's block scales
      if (ok) {
        if (FMT == MDC_FMT_NVFP4) raw_sf = *reinterpret_cast<const uint2*>(pg + PG::kData + tok * 8);
        else raw_sf.x = *reinterpret_cast<const uint32_t*>(pg + PG::kData + (tok % 32) * 16 + (tok / 32) * 4);
      }
      // probe the barriers of this group's next stage now; the answers are read at the top of the next iteration
      const int nt = tile + DG;
      bool n_raw = false, n_a = true;
      if (nt < n_tiles) {
        n_raw = mbar_test(&raw_full[nt % kRawStages], (nt / kRawStages) & 1);
        if (nt >= kASt) n_a = mbar_test(&mma_done[nt % kASt], ((nt / kASt) - 1) & 1);
      }
      if (!a_ok && !mbar_wait(&mma_done[a], ((tile / kASt) - 1) & 1, kBudget, abort_flag)) {
        if (lane == 0) give_up(4, tile);
        break;
      }
      umma::fence_after_sync();
      // the raw stage is in registers: hand it back to the copy warp
      __syncwarp();
      mbar_arrive_if(&raw_empty[s], lane == 0);
      // undo the rotation in registers (the tensor-memory store takes one column address per
      // warp, so chunk k has to sit in the same register of every lane): two select stages
      if (rot & 1) {
        const uint4 t = d[3];
        d[3] = d[2]; d[2] = d[1]; d[1] = d[0]; d[0] = t;
      }
      if (rot & 2) {
        uint4 t = d[0]; d[0] = d[2]; d[2] = t;
        t = d[1]; d[1] = d[3]; d[3] = t;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // 16-byte chunk j = 32 dims = 16 columns
        uint32_t s_lo, s_hi;  // fp16x2 block scale of dims 0-15 and 16-31 of the chunk
        if (FMT == MDC_FMT_NVFP4) {
          const uint32_t two = (j & 2 ? raw_sf.y : raw_sf.x) >> (16 * (j & 1));  // scale bytes 2j, 2j+1
          const uint32_t x = e4m3x2_to_f16x2(static_cast<uint16_t>(two & 0xffff));
          s_lo = bcast_lo(x);
          s_hi = bcast_hi(x);
        } else {
          s_lo = s_hi = ue8m0_to_f16x2((raw_sf.x >> (8 * j)) & 0xff);
        }
        const uint32_t w4[4] = {d[j].x, d[j].y, d[j].z, d[j].w};
        uint32_t out[16];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          uint32_t e[4];
          e2m1x8_to_f16x2(w4[q4], e);  // e[i] = elements (2i, 2i+1) of the word
#pragma unroll
          for (int i = 0; i < 4; ++i) out[4 * q4 + i] = hmul2_u32(e[i], q4 < 2 ? s_lo : s_hi);
        }
        umma::tmem_st16(t_row + a * 64 + 16 * j, out);
      }
      // publish the stage as soon as the stores have landed: the tensor core works on it while
      // this group decodes its next stage into another A stage
      umma::wait_st();
      umma::fence_before_sync();
      __syncwarp();
      red_release_cta_shared_inc_if(&a_cnt[a], lane == 0);
      raw_ok = n_raw;
      a_ok = n_a;
    }
  } else {
    // ---------------- gate warps: group gg takes the stages gg, gg + GG, ...; thread = token row
    const int q = (warp - kGateWarp0) & 3, gg = (warp - kGateWarp0) >> 2;
    const uint32_t t_base = tmem + (static_cast<uint32_t>(q * 32) << 16) + kAccBase;
    bool done_ok = false;
    for (int tile = gg; tile < n_tiles; tile += GG) {
      const int c = tile % kAccSt;
      if (!done_ok && !mbar_wait(&mma_done[tile % kASt], (tile / kASt) & 1, kBudget, abort_flag)) {
        if (lane == 0) give_up(5, tile);
        break;
      }
      umma::fence_after_sync();
      const int nt = tile + GG;
      bool n_done = false;
      if (nt < n_tiles) n_done = mbar_test(&mma_done[nt % kASt], (nt / kASt) & 1);
      float score[T];
#pragma unroll
      for (int t = 0; t < T; ++t) {
        uint32_t v0[32], v1[32];
        umma::tmem_ld32(t_base + c * N + t * kIdxHeads, v0);
        umma::tmem_ld32(t_base + c * N + t * kIdxHeads + 32, v1);
        umma::wait_ld();
        if (t == T - 1) {  // the row is in registers: the accumulator stage can be overwritten
          umma::fence_before_sync();
          __syncwarp();
          red_release_cta_shared_inc_if(&acc_cnt[c], lane == 0);
        }
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        const float4* w4 = reinterpret_cast<const float4*>(wsc + t * kIdxHeads);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float4 w = w4[i];
          const uint32_t* v = i < 8 ? v0 + 4 * i : v1 + 4 * (i - 8);
          const float x0 = __uint_as_float(v[0]), x1 = __uint_as_float(v[1]);
          const float x2 = __uint_as_float(v[2]), x3 = __uint_as_float(v[3]);
          // x + |x| is exactly 0 or 2x; the weighted sums run as packed fp32 pairs
          ffma2(s0, s1, x0 + fabsf(x0), x1 + fabsf(x1), w.x, w.y);
          ffma2(s2, s3, x2 + fabsf(x2), x3 + fabsf(x3), w.z, w.w);
        }
        score[t] = (s0 + s1) + (s2 + s3);
      }
      const int local = tile * kTileTok + q * 32 + lane;  // position inside the chunk
      if (local < n_pages * PAGE) {
        const bool ok = page_id[local / PAGE] >= 0;
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
      done_ok = n_done;
    }
  }

  // ---------------- common exit of the pipeline
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const bool failed = *abort_flag != 0;
  if (warp == kIssueWarp) umma::tmem_dealloc(tmem, kTmemCols);
  if (tid == 0) {  // the shared memory is reused by the next task of a persistent block
    for (int i = 0; i < 2 * kRawStages + kAStages; ++i) mbar_inval(raw_full + i);
  }
  if (warp >= kWarps) return;
  if (ROWK && row_mode) {
    // every block of the cluster walks the same barriers, also one whose pipeline gave up
    logits_row_select<T>(p, b, chunk, failed ? 0 : n_pages * PAGE, blk0 * PAGE, limit, chunk_tokens, scores,
                         *reinterpret_cast<RegSelectScratch<kFusedRegE>*>(smem + L.sel),
                         *reinterpret_cast<RowSelectScratch*>(smem + L.row));
    return;
  }
  if (failed) return;

  if (fused) {
    const int n_local = n_pages * PAGE;
    const int base_pos = blk0 * PAGE;
    for (int t = 0; t < T; ++t) {
      const float* sc_row = scores + t * chunk_tokens;
      const int64_t slot0 = ((static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk) * p.top_k;
      uint32_t* keys = reinterpret_cast<uint32_t*>(scores + t * chunk_tokens);
      auto emit = [&](int pos, int slot) {
        const uint32_t kv = keys[pos];
        p.cand_v[slot0 + slot] = __uint_as_float((kv & 0x80000000u) ? (kv ^ 0x80000000u) : ~kv);
        p.cand_i[slot0 + slot] = (base_pos + pos) * p.id_mul + p.id_add;
      };
      int n;
      if (rt && T == 1)  // (the raw ring is idle by now: it holds the chunk's histogram)
        n = chunk_emit_above_row_threshold(*rt, p.status, b, chunk, p.n_chunks, sc_row, keys, n_local, base_pos, limit, p.top_k,
                                           sel, reinterpret_cast<uint32_t*>(ring), emit, p.id_mul, p.id_add);
      else
        n = fused_chunk_select(sc_row, keys, n_local, base_pos, limit, p.top_k, sel, emit);
      if (tid == 0) p.cand_c[(static_cast<int64_t>(b) * T + t) * p.n_chunks + chunk] = n;
    }
  }
}

}  // namespace mdc
