// Persistent decode megakernel: one block per SM walks its static task queue;
// every task waits on its events, runs one tile (indexer logits, candidate
// merges, sparse attention, LSE merge, or a test op) and posts its notifies.
// Cross-rank payload travels by direct stores / bulk copies into the peers'
// symmetric arena, followed by a system-scope release notify.
//
// Block shape: 15 warps.  Warps 0..7 are the workers every tile is written
// for; the indexer tile additionally uses warps 8..14 (gate, issue, copy).
// Blocks wait on each other, so the grid must be co-resident (<= one block per
// SM; the launcher checks it).  Every wait has a time budget; a block that
// runs out records the event in the status block, which all blocks check at
// each task boundary, and the grid drains.
#include "comm.cuh"
#include "events.cuh"
#include "sched.cuh"
#include "tile_compress.cuh"
#include "tile_logits.cuh"
#include "tile_lse_merge.cuh"
#include "tile_merge.cuh"
#include "tile_mla.cuh"
#include "tile_mla_umma.cuh"

namespace mdc {

constexpr int kMegaGate = 1;  // gate groups of the indexer tile inside the persistent kernel
constexpr int kMegaThreads = logits_threads(2, kMegaGate);
static_assert(kMegaThreads >= kMuThreads, "the block must hold the attention tile's warps (its roles go by warp index; extra warps only join the barriers)");
constexpr int kStagedWords = 128;  // queue rows up to this length are staged in shared memory
constexpr int kMegaTileSmem = MlaUmmaSmem<576>::kTotal > MlaSmem<576>::kTotal ? MlaUmmaSmem<576>::kTotal : MlaSmem<576>::kTotal;  // the largest tile

// The merge ops keep their scratch (MergeSmem) at the base of the tile's shared memory and stage the
// lists behind it.
constexpr int kMergeHdr = (static_cast<int>(sizeof(MergeSmem)) + 1023) / 1024 * 1024;
static_assert(kMergeHdr + 16384 * 8 <= kMegaTileSmem, "a row of 16384 staged candidates must fit behind the merge scratch");

struct MegaShared {
  int32_t row[kStagedWords];
  int32_t fail;
  int32_t next;   // dynamic scheduling: index of the task this block pulled
  unsigned long long phase;
};

__device__ inline int64_t phase_offset(const mdc_mega_params& p, unsigned long long phase) {
  return static_cast<int64_t>(phase % static_cast<unsigned long long>(max(p.layer.phases, 1))) * p.layer.phase_bytes;
}
// One candidate slice of the arena: [count cell, 16 bytes][top_k f32 logits][top_k i32 ids].  The cell comes first so
// that a list of n entries leaves as ONE bulk copy of the slice's head (cell, all logits, the first n ids).
__device__ inline int cand_slice_bytes(const mdc_layer_params& L) { return L.top_k * 8 + 16; }
constexpr int kSliceV = 16;
__device__ __host__ inline int64_t slice_i_off(int K) { return 16 + static_cast<int64_t>(K) * 4; }
__device__ inline int inbox_slice_bytes(const mdc_layer_params& L) { return L.H * kMlaDv * 2 + L.H * 4; }
// Lists each rank contributes to a row's candidate region.
__device__ __host__ inline int cand_lists_per_rank(const mdc_layer_params& L) { return L.cand_direct && L.cp > 1 ? L.n_chunks : 1; }
// First KV pool row of batch entry b: kv_group consecutive entries share one sequence's rows.
__device__ inline int64_t kv_row_base(const mdc_layer_params& L, int b) {
  return static_cast<int64_t>(L.kv_group > 1 ? b / L.kv_group : b) * L.kv_seq_stride;
}

// Ordered compaction by the 256 workers: keeps ids[i] (i < n) with
// ids[i] % cp == rank and writes row_base + ids[i] / cp to out in input order.  Returns the count.
// A warp fetches its whole segment in batches of eight independent loads per lane (the ids were just
// written to global memory: one dependent load per step of the scan would cost an L2 round trip each).
__device__ inline int compact_local_ids(const int32_t* ids, int n, int cp, int rank, int row_base, int32_t* out,
                                        int out_cap, SelectScratch& sc) {
  constexpr int U = 8;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = ceil_div(ceil_div(n, kWarps), 32) * 32;
  const int lo = warp * seg, hi = min(n, lo + seg);
  const uint32_t lt = (1u << lane) - 1u;
  int cnt = 0;
  for (int base = lo; base < hi; base += 32 * U) {
    int32_t id[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + 32 * u + lane;
      id[u] = i < hi ? ids[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) cnt += __popc(__ballot_sync(0xffffffffu, id[u] >= 0 && (id[u] % cp) == rank));
  }
  sync_workers();
  if (lane == 0) sc.wgt[warp] = cnt;
  sync_workers();
  int before = 0, total = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) before += sc.wgt[w];
    total += sc.wgt[w];
  }
  for (int base = lo; base < hi; base += 32 * U) {
    int32_t id[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i = base + 32 * u + lane;
      id[u] = i < hi ? ids[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const bool keep = id[u] >= 0 && (id[u] % cp) == rank;
      const uint32_t m = __ballot_sync(0xffffffffu, keep);
      const int slot = before + __popc(m & lt);
      if (keep && slot < out_cap) out[slot] = row_base + id[u] / cp;
      before += __popc(m);
    }
  }
  sync_workers();
  return min(total, out_cap);
}

// ------------------------------------------------------------------ layer ops
// Byte sizes of one sequence's query arrays and the q region's sub-offsets (arrays over all B sequences).
__device__ __host__ inline int64_t q_idx_bytes() { return 64 * 128 * 2; }
__device__ __host__ inline int64_t q_w_bytes() { return 64 * 4; }
__device__ __host__ inline int64_t q_mla_bytes(const mdc_layer_params& L) { return static_cast<int64_t>(L.H) * L.mla.d_qk * 2; }

// Owner of sequence b: its query block from the staging buffer -> the q region of every rank's arena.
// Each array goes through shared memory as bulk copies: one global -> shared, then one shared -> (peer)
// global per destination rank (own arena included), all issued by one thread and carried by the copy
// engine; 16-byte loads and stores by the threads took 20 us per task at eight ranks.
// One SM moves about 45 GB/s this way, so the big array is cut into slices that run as separate tasks.
// part 0: the indexer's share (q_idx, weights: 16.6 KB, what the LOGITS tasks wait for); part 1 + s:
// slice s of n_slices of the attention query (147 KB in all, needed only once the selection is done).
// The step's attention query may still be on its way from the host: thread 0 polls the flag the host's copy
// stream writes behind it (bounded), the caller's barrier publishes the result.
__device__ inline void wait_host_query(const mdc_mega_params& p, unsigned long long phase) {
  const unsigned long long* flag = p.layer.q_host_flag;
  if (flag == nullptr || threadIdx.x != 0) return;
  const unsigned long long want = phase + 1ull, t0 = global_timer_ns();
  unsigned long long seen = ld_acquire_sys_u64(flag);
  while (seen < want) {
    nanosleep(128);
    seen = ld_acquire_sys_u64(flag);
    if (seen < want && static_cast<long long>(global_timer_ns() - t0) > p.wait_budget_ns) {
      report_failure(p.status, MDC_DEV_WAIT_TIMEOUT, -2000, 0, seen, want);
      break;
    }
  }
}

__device__ __noinline__ void op_qpath(const mdc_mega_params& p, int b, int part, int n_slices, unsigned long long phase,
                                unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  if (!L.q_stage || b % L.cp != L.rank) return;
  if (part >= 1 && L.q_host_flag) {
    wait_host_query(p, phase);
    sync_workers();
  }
  const PeerBuffer arena{static_cast<unsigned char*>(p.arena.base), p.arena.offsets, p.arena.my_rank, p.arena.world,
                         p.arena.mc_base};
  const int n_owned = ceil_div(L.B - L.rank, L.cp), j = b / L.cp;
  const unsigned char* st = static_cast<const unsigned char*>(L.q_stage);
  const int64_t src_off[3] = {j * q_idx_bytes(), n_owned * q_idx_bytes() + j * q_w_bytes(),
                              n_owned * (q_idx_bytes() + q_w_bytes()) + j * q_mla_bytes(L)};
  const int64_t base = phase_offset(p, phase) + L.q_off;
  const int64_t dst_off[3] = {base + b * q_idx_bytes(), base + L.B * q_idx_bytes() + b * q_w_bytes(),
                              base + L.B * (q_idx_bytes() + q_w_bytes()) + b * q_mla_bytes(L)};
  int64_t len[3] = {q_idx_bytes(), q_w_bytes(), q_mla_bytes(L)};
  int64_t skip = 0;
  if (part >= 1) {  // a 16-byte aligned slice of the attention query
    n_slices = max(1, n_slices);
    const int64_t per = (len[2] / n_slices + 15) / 16 * 16;
    skip = min(len[2], static_cast<int64_t>(part - 1) * per);
    len[2] = max(static_cast<int64_t>(0), min(per, len[2] - skip));
  }
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem);
  unsigned char* buf = smem + 128;
  if (threadIdx.x == 0) {
    // all arrays of the part in flight together: global -> shared (one barrier), then every shared ->
    // (peer) global copy, one wait at the end (a wait per array would pay the NVLink write round trip each time)
    const int a0 = part >= 1 ? 2 : 0, a1 = part == 0 ? 2 : 3;
    mbar_init(bar, 1);
    mbar_fence_init();
    uint32_t total = 0;
    for (int a = a0; a < a1; ++a) total += static_cast<uint32_t>(len[a]);
    if (total > 0) {
      mbar_expect_tx(bar, total);
      uint32_t at_smem = 0;
      for (int a = a0; a < a1; ++a) {
        if (len[a] > 0) bulk_g2s(buf + at_smem, st + src_off[a] + (a == 2 ? skip : 0), static_cast<uint32_t>(len[a]), bar);
        at_smem += static_cast<uint32_t>(len[a]);
      }
      if (mbar_wait(bar, 0)) {
        at_smem = 0;
        for (int a = a0; a < a1; ++a) {
          if (len[a] > 0)
            for (int dst = 0; dst < L.cp; ++dst)
              bulk_s2g(arena.peer_ptr(dst_off[a] + (a == 2 ? skip : 0), dst), buf + at_smem, static_cast<uint32_t>(len[a]));
          at_smem += static_cast<uint32_t>(len[a]);
        }
        bulk_commit();
        bulk_wait_all();
        fence_proxy_async_global();
      } else {
        report_failure(p.status, MDC_DEV_COPY_TIMEOUT, b, part, 0, 0);
      }
    }
    mbar_inval(bar);
  }
  sync_workers();
}

// The step's new token of sequence b: on the rank that owns its position, the index-K record is
// quantised into the paged cache, the KV row is copied into the pool and the rank-local length grows
// by one; every rank then (optionally) advances its copy of the global length.
__device__ __noinline__ void op_kvwrite(const mdc_mega_params& p, int b) {
  const mdc_layer_params& L = p.layer;
  if (!L.kvw_glen) return;
  const mdc_logits_params& lp = L.logits;
  const int tid = threadIdx.x;
  const int t = L.kvw_glen[b];
  if (t >= 0 && t % L.cp == L.rank) {
    const int slot = t / L.cp, P = lp.page_tokens;
    const int blk = slot / P, tok = slot % P;
    const int32_t page = blk < lp.max_pages ? lp.block_table[static_cast<int64_t>(b) * lp.max_pages + blk] : -1;
    if (page < 0 || page >= lp.num_pages || slot >= L.kv_seq_stride) {
      if (tid == 0) report_failure(p.status, MDC_DEV_BAD_INDEX, page, slot, 0, 0);
    } else {
      if (tid < 32) {  // one warp: 128 fp32 -> 64 code bytes + block scales of the cache format
        const float4 v = reinterpret_cast<const float4*>(L.kvw_k_idx + static_cast<int64_t>(b) * 128)[tid];
        const float x[4] = {v.x, v.y, v.z, v.w};
        const int sf_per_tok = lp.fmt == MDC_FMT_MXFP4 ? 4 : 8;
        uint8_t* pg = const_cast<uint8_t*>(lp.kv_pages) + static_cast<int64_t>(page) * (P * 64 + P * sf_per_tok);
        uint8_t* sf = lp.fmt == MDC_FMT_MXFP4 ? pg + P * 64 + (tok % 32) * 16 + (tok / 32) * 4 : pg + P * 64 + tok * 8;
        fp4_quant_warp(x, pg + tok * 64, sf, lp.fmt);
      }
      const int row_bytes = L.mla.d_qk * (L.mla.kv_dtype == MDC_DT_E4M3 ? 1 : 2);
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(L.kvw_kv) + static_cast<int64_t>(b) * row_bytes);
      uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(const_cast<void*>(L.mla.kv_cmp)) +
                                            (kv_row_base(L, b) + slot) * row_bytes);
      for (int i = tid; i < row_bytes / 16; i += kBlockThreads) dst[i] = src[i];
      if (tid == 0) const_cast<int32_t*>(lp.seq_lens)[b] = slot + 1;
    }
  }
  sync_workers();
  if (tid == 0 && L.kvw_advance) L.kvw_glen[b] = t + 1;
}

// the tiles' parameters with the query pointers redirected to this phase's q region of the own arena
__device__ inline void redirect_q(const mdc_mega_params& p, unsigned long long phase, mdc_logits_params* lp,
                                  mdc_sparse_mla_params* mp) {
  const mdc_layer_params& L = p.layer;
  if (!L.q_stage) return;
  const unsigned char* base = static_cast<const unsigned char*>(p.arena.base) + phase_offset(p, phase) + L.q_off;
  if (lp) {
    lp->q = base;
    lp->weights = reinterpret_cast<const float*>(base + L.B * q_idx_bytes());
  }
  if (mp) mp->q = base + L.B * (q_idx_bytes() + q_w_bytes());
}

template <int FMT, int PAGE>
__device__ __noinline__ void op_logits(const mdc_mega_params& p, int b, int chunk, unsigned long long phase, unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  mdc_logits_params lp = L.logits;
  redirect_q(p, phase, &lp, nullptr);
  if (L.thr_hist && L.thr_done) {
    const int64_t half = static_cast<int64_t>(L.B) * kThrBins;
    RowThreshold rt;
    rt.hist = L.thr_hist + (phase & 1ull) * half;
    rt.hist_next = L.thr_hist + ((phase + 1ull) & 1ull) * half;
    rt.done = L.thr_done;
    rt.target = static_cast<uint32_t>(static_cast<unsigned long long>(L.n_chunks) * (phase + 1ull));
    rt.budget_ns = p.wait_budget_ns;
    rt.x = nullptr;
    RowExact x;
    static_assert(kThrBins * 4 + sizeof(RowExactScratch) <= kRawStages * IdxPage<FMT, PAGE>::kStageBytes,
                  "the exact selection's scratch lives in the idle raw ring");
    if (L.thr_exact) {
      const int C = L.n_chunks, K = L.top_k;
      x.ev = EventSet{static_cast<unsigned char*>(p.events.base), p.events.offsets, p.events.my_rank, p.events.world};
      x.ev_hist = L.thr_ev_base + b;
      x.ev_keys = L.thr_ev_base + L.B + b;
      const bool local_only = L.thr_exact == 2 && L.cp > 1;   // each rank settles its own list
      x.pcp = local_only ? 1 : L.cp;
      x.prank = local_only ? 0 : L.rank;
      x.hist_target = static_cast<unsigned long long>(x.pcp) * (phase + 1ull);
      x.keys_target = static_cast<unsigned long long>(x.pcp) * C * (phase + 1ull);
      x.arena = static_cast<unsigned char*>(p.arena.base);
      x.arena_offsets = p.arena.offsets;
      const int64_t row_bytes = static_cast<int64_t>(L.cp) * (kRowHistBytes + static_cast<int64_t>(C) * kRowSlotBytes);
      x.hist_off = phase_offset(p, phase) + L.thr_off + b * row_bytes;
      x.slot_off = x.hist_off + static_cast<int64_t>(L.cp) * kRowHistBytes;
      x.slice_bytes = cand_slice_bytes(L);
      x.out_off = phase_offset(p, phase) + L.cand_off + static_cast<int64_t>(b) * L.cp * cand_lists_per_rank(L) * x.slice_bytes;
      x.cp = L.cp;
      x.rank = L.rank;
      x.out_v = L.sel_v + static_cast<int64_t>(b) * K;
      x.out_i = L.sel_i + static_cast<int64_t>(b) * K;
      x.sel_c = L.sel_c + b;
      x.pt = const_cast<int32_t*>(L.mla.pt_cmp) + static_cast<int64_t>(b) * L.mla.pt_cols;
      x.pt_cols = L.mla.pt_cols;
      x.k_valid = const_cast<int32_t*>(L.mla.k_valid) + b;
      x.row_base = static_cast<int>(kv_row_base(L, b));
      x.win_slots = kWinSlots;
      rt.x = &x;
    }
    logits_tile<FMT, PAGE, 1, 2, kMegaGate>(lp, b, chunk, smem, &rt);
  } else {
    logits_tile<FMT, PAGE, 1, 2, kMegaGate>(lp, b, chunk, smem);
  }
  if (L.cand_direct && L.cp > 1 && threadIdx.x < kBlockThreads) {
    // The chunk's list goes to every rank's candidate region (slot rank * n_chunks + chunk of the
    // row) as bulk copies of the filled part only: stage it in the tile's idle raw ring first.  The
    // pipeline's warps have left the tile; the worker threads wrote the list and are all here.
    const PeerBuffer arena{static_cast<unsigned char*>(p.arena.base), p.arena.offsets, p.arena.my_rank, p.arena.world,
                           p.arena.mc_base};
    const int K = L.top_k, C = L.n_chunks;
    __threadfence();
    sync_workers();
    const int64_t row = static_cast<int64_t>(b) * C + chunk;
    int n = lp.cand_c[row];
    if (n < 0) return;   // (uniform over the block) the row was published by the tasks themselves, cells included
    n = min(n, K);
    const int n4 = (n + 3) & ~3;   // K is a multiple of 4 here: the rounded part stays inside the slice
    // staged with the slice's own layout, so that one bulk copy per rank carries cell, logits and ids
    unsigned char* stage = smem + logits_smem_layout<FMT, PAGE>(1, lp.blocks_per_chunk * PAGE, true).ring;
    int32_t* sc = reinterpret_cast<int32_t*>(stage);
    uint32_t* sv = reinterpret_cast<uint32_t*>(stage + kSliceV);
    uint32_t* si = reinterpret_cast<uint32_t*>(stage + slice_i_off(K));
    const uint32_t* gv = reinterpret_cast<const uint32_t*>(lp.cand_v + row * K);
    const uint32_t* gi = reinterpret_cast<const uint32_t*>(lp.cand_i + row * K);
    for (int i = threadIdx.x; i < n4; i += kBlockThreads) {
      sv[i] = i < n ? __ldcg(gv + i) : 0u;
      si[i] = i < n ? __ldcg(gi + i) : 0u;
    }
    if (threadIdx.x < 4) sc[threadIdx.x] = threadIdx.x == 0 ? n : 0;
    fence_proxy_async_smem();
    sync_workers();
    if (threadIdx.x < L.cp) {
      const int64_t off = phase_offset(p, phase) + L.cand_off +
                          ((static_cast<int64_t>(b) * L.cp + L.rank) * C + chunk) * cand_slice_bytes(L);
      unsigned char* dst = arena.peer_ptr(off, threadIdx.x);
      bulk_s2g(dst, stage, n4 > 0 ? static_cast<uint32_t>(slice_i_off(K) + n4 * 4) : 16u);
      bulk_commit();
      bulk_wait_all();
      fence_proxy_async_global();
    }
    sync_workers();
  }
}

// first level of a two-level local merge: the chunk lists of group g of sequence b -> one list
__device__ __noinline__ void op_merge_l1a(const mdc_mega_params& p, int b, int g, unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  MergeSmem& sm = *reinterpret_cast<MergeSmem*>(smem);
  const int K = L.top_k, C = L.n_chunks, G = max(1, L.l1_groups);
  const int per = ceil_div(C, G);
  const int c0 = min(max(g, 0), G - 1) * per, n = max(0, min(per, C - c0));
  MergeLists ls;
  ls.v = L.logits.cand_v + (static_cast<int64_t>(b) * C + c0) * K;
  ls.i = L.logits.cand_i + (static_cast<int64_t>(b) * C + c0) * K;
  ls.c = L.logits.cand_c + static_cast<int64_t>(b) * C + c0;
  ls.stride = K;
  ls.c_stride = 1;
  const int64_t o = static_cast<int64_t>(b) * G + g;
  merge_lists_auto<false>(ls, n, K, K, L.mid_v + o * K, L.mid_i + o * K, L.mid_c + o, nullptr, sm, smem + kMergeHdr,
                          kMegaTileSmem - kMergeHdr);
}

// chunk (or group) candidate lists of sequence b -> this rank's top-k, written into the
// own slice of the candidate region and copied to every peer's arena
__device__ __noinline__ void op_merge_l1(const mdc_mega_params& p, int b, unsigned long long phase, unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  MergeSmem& sm = *reinterpret_cast<MergeSmem*>(smem);
  const PeerBuffer arena{static_cast<unsigned char*>(p.arena.base), p.arena.offsets, p.arena.my_rank, p.arena.world,
                         p.arena.mc_base};
  const int K = L.top_k;
  const bool two_level = L.l1_groups > 1 && L.mid_v != nullptr;
  const int C = two_level ? L.l1_groups : L.n_chunks;  // lists to merge: the groups' lists, or the chunks'
  MergeLists ls;
  ls.v = (two_level ? L.mid_v : L.logits.cand_v) + static_cast<int64_t>(b) * C * K;
  ls.i = (two_level ? L.mid_i : L.logits.cand_i) + static_cast<int64_t>(b) * C * K;
  ls.c = (two_level ? L.mid_c : L.logits.cand_c) + static_cast<int64_t>(b) * C;
  ls.stride = K;
  ls.c_stride = 1;
  if (L.thr_exact && !two_level && (L.cp == 1 || L.thr_exact == 2)) {
    // the LOGITS tasks of the row published the selection and the gather list themselves: nothing to do
    int pub = 0;
    if (threadIdx.x < 32) {
      int all = 1;
      for (int c = threadIdx.x; c < C; c += 32) all &= __ldcg(ls.c + c) < 0;
      pub = __all_sync(0xffffffffu, all);
      if (threadIdx.x == 0) sm.sel.bnd = pub;
    }
    sync_workers();
    pub = sm.sel.bnd;
    sync_workers();
    if (pub) return;
  }
  const int64_t off = phase_offset(p, phase) + L.cand_off + (static_cast<int64_t>(b) * L.cp + L.rank) * cand_slice_bytes(L);
  unsigned char* slice = arena.local_ptr(off);
  merge_lists_auto<false>(ls, C, K, K, reinterpret_cast<float*>(slice + kSliceV), reinterpret_cast<int32_t*>(slice + slice_i_off(K)),
                          reinterpret_cast<int32_t*>(slice), nullptr, sm, smem + kMergeHdr, kMegaTileSmem - kMergeHdr);
  if (L.cp == 1) {
    // one rank: this list IS the selection; publish it and the gather list here (no MERGE_L2 task)
    __threadfence();
    sync_workers();
    const int n = *reinterpret_cast<const int32_t*>(slice);
    const float* sv = reinterpret_cast<const float*>(slice + kSliceV);
    const int32_t* si = reinterpret_cast<const int32_t*>(slice + slice_i_off(K));
    for (int i = threadIdx.x; i < n; i += kBlockThreads) {
      L.sel_v[static_cast<int64_t>(b) * K + i] = sv[i];
      L.sel_i[static_cast<int64_t>(b) * K + i] = si[i];
    }
    if (threadIdx.x == 0) L.sel_c[b] = n;
    int32_t* pt = const_cast<int32_t*>(L.mla.pt_cmp) + static_cast<int64_t>(b) * L.mla.pt_cols;
    const int mine = compact_local_ids(si, n, 1, 0, static_cast<int>(kv_row_base(L, b)), pt, L.mla.pt_cols, sm.sel);
    if (threadIdx.x == 0) const_cast<int32_t*>(L.mla.k_valid)[b] = kWinSlots + mine;
  }
  if (L.cp > 1) {
    // The slice goes to every peer as ONE bulk copy each (the copy engine keeps NVLink busy with
    // large packets; thousands of 16-byte stores per task do not): stage it in shared memory first.
    __threadfence();
    sync_workers();
    unsigned char* stage = smem + kMergeHdr;
    const int n16 = cand_slice_bytes(L) / 16;
    for (int i = threadIdx.x; i < n16; i += kBlockThreads)
      reinterpret_cast<uint4*>(stage)[i] = reinterpret_cast<const uint4*>(slice)[i];
    fence_proxy_async_smem();
    sync_workers();
    if (threadIdx.x < L.cp && static_cast<int>(threadIdx.x) != L.rank) {
      bulk_s2g(arena.peer_ptr(off, threadIdx.x), stage, cand_slice_bytes(L));
      bulk_commit();
      bulk_wait_all();
      fence_proxy_async_global();
    }
    sync_workers();  // the staging area is reused by the block's next task
  }
}

// cp candidate lists of sequence b (one per rank, in the own arena) -> global
// top-k (identical on every rank) and this rank's gather list for attention
template <bool SYS>
__device__ __noinline__ void op_merge_l2(const mdc_mega_params& p, int b, unsigned long long phase, unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  MergeSmem& sm = *reinterpret_cast<MergeSmem*>(smem);
  const int K = L.top_k;
  const int64_t off = phase_offset(p, phase) + L.cand_off +
                      static_cast<int64_t>(b) * L.cp * cand_lists_per_rank(L) * cand_slice_bytes(L);
  const unsigned char* first = static_cast<const unsigned char*>(p.arena.base) + off;
  MergeLists ls;
  ls.v = reinterpret_cast<const float*>(first + kSliceV);
  ls.i = reinterpret_cast<const int32_t*>(first + slice_i_off(K));
  ls.c = reinterpret_cast<const int32_t*>(first);
  ls.stride = cand_slice_bytes(L) / 4;
  ls.c_stride = cand_slice_bytes(L) / 4;
  int32_t* sel_i = L.sel_i + static_cast<int64_t>(b) * K;
  if (L.thr_exact == 1 && L.cand_direct) {
    // published by the LOGITS tasks of all ranks (every slice's cell holds {-1, length}): the selection lies
    // in slice 0 of the row; the gather list and its length are already in place
    const int J = L.cp * L.n_chunks;
    if (threadIdx.x < 32) {
      int all = 1;
      for (int j = threadIdx.x; j < J; j += 32)
        all &= __float_as_int(ld_sys_f32(reinterpret_cast<const float*>(first + static_cast<int64_t>(j) * cand_slice_bytes(L)))) < 0;
      const int pub = __all_sync(0xffffffffu, all);
      if (threadIdx.x == 0) sm.sel.bnd = pub;
    }
    sync_workers();
    const int pub = sm.sel.bnd;
    sync_workers();
    if (pub) {
      const int n = min(max(__float_as_int(ld_sys_f32(reinterpret_cast<const float*>(first + 4))), 0), K);
      const int n4 = (n + 3) >> 2;
      float* ov = L.sel_v + static_cast<int64_t>(b) * K;
      for (int i = threadIdx.x; i < n4; i += kBlockThreads) {
        const uint4 v = ld_sys_u4(reinterpret_cast<const uint4*>(first + kSliceV) + i);
        const uint4 d = ld_sys_u4(reinterpret_cast<const uint4*>(first + slice_i_off(K)) + i);
        reinterpret_cast<uint4*>(ov)[i] = v;
        reinterpret_cast<uint4*>(sel_i)[i] = d;
      }
      if (threadIdx.x == 0) L.sel_c[b] = n;
      return;
    }
  }
  // The selected ids land in shared memory (the tail of the staging area): the gather list is compacted from
  // there, without a fence and two round trips to the copy in global memory.
  const int sid_bytes = (K * 4 + 15) & ~15;
  int32_t* sid = reinterpret_cast<int32_t*>(smem + kMegaTileSmem - sid_bytes);
  const int n = merge_lists_auto<SYS>(ls, L.cp * cand_lists_per_rank(L), K, K, L.sel_v + static_cast<int64_t>(b) * K, sid, L.sel_c + b, nullptr, sm,
                                     smem + kMergeHdr, kMegaTileSmem - kMergeHdr - sid_bytes);
  sync_workers();
  for (int i = threadIdx.x; i < n; i += kBlockThreads) sel_i[i] = sid[i];
  int32_t* pt = const_cast<int32_t*>(L.mla.pt_cmp) + static_cast<int64_t>(b) * L.mla.pt_cols;
  const int mine = compact_local_ids(sid, n, L.cp, L.rank, static_cast<int>(kv_row_base(L, b)), pt, L.mla.pt_cols, sm.sel);
  if (threadIdx.x == 0) const_cast<int32_t*>(L.mla.k_valid)[b] = kWinSlots + mine;
}

// attention of sequence b over this rank's share of the selection; the normalised partial
// (bf16) and its log2-LSE go straight into the owner's inbox.  With bf16 operands and heads in
// blocks of 128 a task is 128 heads x 128 output columns on the tcgen05 tile (task index =
// 4 * head block + column block, all threads take part); otherwise 64 heads x 256 columns on
// the mma.sync tile (task index = 2 * head block + column half, worker threads only).
__device__ __noinline__ void op_attn(const mdc_mega_params& p, int b, int hbv, int split, unsigned long long phase,
                               unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  const PeerBuffer arena{static_cast<unsigned char*>(p.arena.base), p.arena.offsets, p.arena.my_rank, p.arena.world,
                         p.arena.mc_base};
  const int owner = b % L.cp;
  const int ns = max(1, L.attn_splits);
  split = min(max(split, 0), ns - 1);
  const int64_t off = phase_offset(p, phase) + L.inbox_off +
                      ((static_cast<int64_t>(b / L.cp) * L.cp + L.rank) * ns + split) * inbox_slice_bytes(L);
  unsigned char* slot = arena.peer_ptr(off, owner);
  float* lse_row = reinterpret_cast<float*>(slot + static_cast<int64_t>(L.H) * kMlaDv * 2);
  // The tiles seed the attention sink in split 0; across ranks exactly one partial may carry it
  // (the owner's), or the merged denominator would count the sink cp times.
  mdc_sparse_mla_params mp = L.mla;
  if (L.rank != owner) mp.attn_sink = nullptr;
  redirect_q(p, phase, nullptr, &mp);
  if (L.q_host_flag && !L.q_stage) {   // (with QPATH tasks they have waited for it)
    wait_host_query(p, phase);
    __syncthreads();
  }
  if (mp.kv_dtype == MDC_DT_BF16 && L.H % kMuHeads == 0) {
    if (mp.d_qk == 576) mla_umma_tile<576>(mp, b, hbv >> 2, hbv & 3, split, ns, smem, slot, lse_row, true);
    else mla_umma_tile<512>(mp, b, hbv >> 2, hbv & 3, split, ns, smem, slot, lse_row, true);
    return;
  }
  if (threadIdx.x >= kBlockThreads) return;
  const int hb = hbv >> 1, dv0 = (hbv & 1) * 256;
  if (mp.d_qk == 576 && mp.kv_dtype == MDC_DT_BF16) mla_tile<576, MDC_DT_BF16, 256>(mp, b, hb, split, ns, smem, slot, lse_row, dv0, true);
  else if (mp.d_qk == 512 && mp.kv_dtype == MDC_DT_BF16) mla_tile<512, MDC_DT_BF16, 256>(mp, b, hb, split, ns, smem, slot, lse_row, dv0, true);
  else if (mp.d_qk == 576) mla_tile<576, MDC_DT_E4M3, 256>(mp, b, hb, split, ns, smem, slot, lse_row, dv0, true);
  else mla_tile<512, MDC_DT_E4M3, 256>(mp, b, hb, split, ns, smem, slot, lse_row, dv0, true);
}

// owner of sequence b: cp inbox slices -> merged output
// (task = head group hq of n_groups: the merge of one sequence is spread over several blocks)
template <bool SYS>
__device__ __noinline__ void op_lse_merge(const mdc_mega_params& p, int b, int hq, int n_groups, unsigned long long phase,
                                    unsigned char* smem) {
  const mdc_layer_params& L = p.layer;
  n_groups = max(1, min(n_groups, L.H));
  const int nh = ceil_div(L.H, n_groups);
  const int h0 = min(max(hq, 0), n_groups - 1) * nh;
  const int n_heads = max(0, min(nh, L.H - h0));
  const int ns = max(1, L.attn_splits);
  const int64_t off = phase_offset(p, phase) + L.inbox_off + static_cast<int64_t>(b / L.cp) * L.cp * ns * inbox_slice_bytes(L);
  LseSrc src;
  src.o = static_cast<const unsigned char*>(p.arena.base) + off;
  src.lse = reinterpret_cast<const float*>(src.o + static_cast<int64_t>(L.H) * kMlaDv * 2);
  src.o_stride = inbox_slice_bytes(L);
  src.lse_stride = inbox_slice_bytes(L) / 4;
  const int osz = (L.out_dtype == MDC_DT_F32) ? 4 : 2;
  lse_merge_rows<SYS>(src, L.cp * ns, L.H, kMlaDv, MDC_DT_BF16, L.out_dtype,
                      static_cast<unsigned char*>(L.out) + static_cast<int64_t>(b / L.cp) * L.H * kMlaDv * osz,
                      L.out_lse ? L.out_lse + static_cast<int64_t>(b / L.cp) * L.H : nullptr, h0, n_heads,
                      reinterpret_cast<float*>(smem));
}

// KV compressor of sequence b (layer.cmp): the step appends this rank's new record and, on a closing
// step, pushes this rank's statistics to the entry's owner; the finalize runs on the owner after all
// cp statistics have arrived (the task's wait edge) and writes the pools.  Off the critical path:
// the new entry becomes visible to the next step.
__device__ __noinline__ void op_cmp(const mdc_mega_params& p, int b, bool finalize, unsigned long long phase, unsigned char* smem) {
  mdc_compress_params c = p.layer.cmp;
  c.arena = p.arena;
  c.stats_off += phase_offset(p, phase);
  c.status = p.status;
  if (b < 0 || b >= c.B) return;
  if (c.ratio == 4) {
    if (finalize) csa_finalize_tile<false>(c, b, *reinterpret_cast<FinalizeSmem*>(smem));
    else csa_step_tile<false>(c, b, reinterpret_cast<float*>(smem));
  } else {
    if (finalize) online_finalize_tile<false>(c, b, *reinterpret_cast<FinalizeSmem*>(smem));
    else online_step_tile<false>(c, b, reinterpret_cast<float*>(smem));
  }
}

// ------------------------------------------------------------------ test ops
__device__ inline uint32_t test_pattern(int src_rank, int slot, unsigned long long phase, int i) {
  return 0x9e3779b9u * static_cast<uint32_t>(i + 1) + static_cast<uint32_t>(src_rank) * 0x01000193u +
         static_cast<uint32_t>(slot) * 7919u + static_cast<uint32_t>(phase) * 104729u;
}
// stage a pattern in shared memory and bulk-push it into slot (my rank, slot) of rank dst
__device__ inline void op_push(const mdc_mega_params& p, int dst, int slot, unsigned long long phase, unsigned char* smem) {
  const PeerBuffer arena{static_cast<unsigned char*>(p.arena.base), p.arena.offsets, p.arena.my_rank, p.arena.world,
                         p.arena.mc_base};
  uint32_t* stage = reinterpret_cast<uint32_t*>(smem);
  const int words = p.test_slot_bytes / 4;
  for (int i = threadIdx.x; i < words; i += kBlockThreads) stage[i] = test_pattern(arena.my_rank, slot, phase, i);
  fence_proxy_async_smem();
  sync_workers();
  if (threadIdx.x == 0) {
    const int64_t off = p.test_off + (static_cast<int64_t>(slot) * arena.world + arena.my_rank) * p.test_slot_bytes;
    push_start(arena.peer_ptr(off, dst), stage, p.test_slot_bytes);
    push_finish();
  }
}
__device__ inline void op_verify(const mdc_mega_params& p, int src_rank, int slot, unsigned long long phase) {
  const int words = p.test_slot_bytes / 4;
  const int64_t off = p.test_off + (static_cast<int64_t>(slot) * p.arena.world + src_rank) * p.test_slot_bytes;
  const float* data = reinterpret_cast<const float*>(static_cast<const unsigned char*>(p.arena.base) + off);
  for (int i = threadIdx.x; i < words; i += kBlockThreads) {
    const uint32_t got = __float_as_uint(ld_sys_f32(data + i));
    if (got != test_pattern(src_rank, slot, phase, i)) report_failure(p.status, MDC_DEV_BAD_INDEX, slot, i, got, 0);
  }
}

}  // namespace mdc

namespace mdc {

__global__ void __launch_bounds__(kMegaThreads, 1) mega_kernel(const __grid_constant__ mdc_mega_params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  __shared__ MegaShared sh;
  const int tid = threadIdx.x, warp = tid >> 5;
  const bool worker = warp < kWarps;

  const bool dyn = p.dyn_task_off != nullptr;   // one shared row, tasks pulled with an atomic counter
  const int32_t* row_g = p.queue + (dyn ? 0 : static_cast<int64_t>(blockIdx.x) * p.row_words);
  const bool staged = !dyn && p.row_words <= kStagedWords;
  if (staged) {
    for (int i = tid; i < p.row_words; i += kMegaThreads) sh.row[i] = row_g[i];
  }
  if (tid == 0) sh.fail = 0;
  __syncthreads();

  Cursor cur;
  cur.row = staged ? sh.row : row_g;
  cur.scalars = reinterpret_cast<const unsigned long long*>(p.scalars);
  cur.arity = p.arity;
  cur.scopes = p.scopes;
  // The phase is read once per launch.  With phase_ctl set the kernel advances it by itself: every
  // block counts in after its read, and the last one to do so (nobody can read after it) stores
  // phase + 1 for the next launch, so a captured graph replays without a host-side update.
  if (tid == 0) {
    const unsigned long long ph = ld_acquire_gpu_u64(cur.scalars);
    sh.phase = ph;
    if (p.phase_ctl) {
      __threadfence();
      if (atomicAdd(p.phase_ctl, 1ull) + 1ull == static_cast<unsigned long long>(gridDim.x)) {
        *p.phase_ctl = 0ull;
        *const_cast<volatile unsigned long long*>(cur.scalars) = ph + 1ull;
      }
    }
  }
  __syncthreads();
  cur.phase = sh.phase;
  const EventSet ev{static_cast<unsigned char*>(p.events.base), p.events.offsets, p.events.my_rank, p.events.world};
  const mdc_layer_params& L = p.layer;

  TaskInfo t_end;
  t_end.op = kOpEnd;
  auto pull = [&]() -> TaskInfo {   // dynamic: the next task of the shared row, or the end marker
    if (tid == 0) sh.next = static_cast<int32_t>(atomicAdd(p.dyn_ctl, 1u));
    __syncthreads();
    const int idx = sh.next;
    __syncthreads();
    return idx >= 0 && idx < p.dyn_n_tasks ? cur.read(p.dyn_task_off[idx]) : t_end;
  };
  for (TaskInfo t = dyn ? pull() : cur.read(0); t.valid(); t = dyn ? pull() : cur.advance(t)) {
    unsigned long long tr0 = 0, tr1 = 0;
    if (p.trace && tid == 0) tr0 = global_timer_ns();
    // ---- waits: thread 0 polls, the barrier publishes
    if (tid == 0) {
      if (p.status && *reinterpret_cast<volatile int32_t*>(p.status) != 0) sh.fail = 1;
      for (int i = 0; i < t.n_waits && !sh.fail; ++i) {
        const int e = cur.wait_event(t, i);
        unsigned long long seen = 0;
        const bool bad_id = e < 0 || e >= p.n_events;
        if (bad_id || !ev.poll_1t(e, cur.target(e), cur.scopes[e] != 0, p.wait_budget_ns, &seen)) {
          report_failure(p.status, bad_id ? MDC_DEV_BAD_OP : MDC_DEV_WAIT_TIMEOUT, e, t.op, seen, bad_id ? 0 : cur.target(e));
          sh.fail = 1;
        }
      }
    }
    __syncthreads();
    if (sh.fail) break;
    if (p.trace && tid == 0) tr1 = global_timer_ns();

    // ---- the task body
    const bool layer_op = t.op >= MDC_OP_LOGITS && t.op <= MDC_OP_KVWRITE;
    if (layer_op && (L.B <= 0 || t.c0 < 0 || t.c0 >= L.B)) {  // no (validated) layer behind this queue
      if (tid == 0) report_failure(p.status, MDC_DEV_BAD_OP, t.op, t.c0, 0, 0);
    } else
    switch (t.op) {
      case MDC_OP_NOP:
        break;
      case MDC_OP_LOGITS:
        if (L.logits.fmt == MDC_FMT_MXFP4) op_logits<MDC_FMT_MXFP4, 128>(p, t.c0, t.c1, cur.phase, smem);
        else if (L.logits.page_tokens == 64) op_logits<MDC_FMT_NVFP4, 64>(p, t.c0, t.c1, cur.phase, smem);
        else op_logits<MDC_FMT_NVFP4, 128>(p, t.c0, t.c1, cur.phase, smem);
        break;
      case MDC_OP_QPATH:
        if (worker) op_qpath(p, t.c0, t.c1, t.c2, cur.phase, smem);
        break;
      case MDC_OP_KVWRITE:
        if (worker) op_kvwrite(p, t.c0);
        break;
      case MDC_OP_MERGE_L1:
        if (worker) op_merge_l1(p, t.c0, cur.phase, smem);
        break;
      case MDC_OP_MERGE_L1A:
        if (worker && L.mid_v && L.mid_i && L.mid_c) op_merge_l1a(p, t.c0, t.c1, smem);
        break;
      case MDC_OP_MERGE_L2:
        if (worker) {
          if (L.cp > 1) op_merge_l2<true>(p, t.c0, cur.phase, smem);
          else op_merge_l2<false>(p, t.c0, cur.phase, smem);
        }
        break;
      case MDC_OP_ATTN:
        op_attn(p, t.c0, t.c1, t.c2, cur.phase, smem);
        break;
      case MDC_OP_LSE_MERGE:
        if (worker) {
          if (L.cp > 1) op_lse_merge<true>(p, t.c0, t.c1, t.c2, cur.phase, smem);
          else op_lse_merge<false>(p, t.c0, t.c1, t.c2, cur.phase, smem);
        }
        break;
      case MDC_OP_CMP_STEP:
      case MDC_OP_CMP_FIN:
        if (worker) op_cmp(p, t.c0, t.op == MDC_OP_CMP_FIN, cur.phase, smem);
        break;
      case MDC_OP_SLEEP:
        if (tid == 0) {
          const unsigned long long t0 = global_timer_ns();
          const unsigned long long want = static_cast<unsigned long long>(min(max(t.c1, 0), 100000000));
          while (global_timer_ns() - t0 < want) nanosleep(256);
        }
        break;
      case MDC_OP_LOG:
        if (tid == 0 && p.log) {
          const int slot = atomicAdd(p.log, 1);
          if (slot + 1 < p.log_cap) p.log[slot + 1] = t.c0;
          __threadfence();
        }
        break;
      case MDC_OP_PUSH:
        if (worker) op_push(p, t.c1, t.c2, cur.phase, smem);
        break;
      case MDC_OP_VERIFY:
        if (worker) op_verify(p, t.c1, t.c2, cur.phase);
        break;
      default:
        if (tid == 0) report_failure(p.status, MDC_DEV_BAD_OP, t.op, t.pos, 0, 0);
        break;
    }

    // ---- notifies: everything this block wrote is released first
    // (threads that issued bulk copies have completed them and fenced the async proxy inside the
    // op; the barrier orders every thread's writes before thread 0's fence, which is cumulative, so
    // ONE fence releases the whole block's payload: system scope only when a peer is notified)
    if (t.n_notifies > 0) {
      __syncthreads();
      if (tid == 0) {
        bool remote = false;
        for (int i = 0; i < t.n_notifies; ++i) remote |= (cur.notify_word(t, i) & 0xFF) != ev.my_rank;
        if (remote) fence_acq_rel_sys();
        else fence_acq_rel_gpu();
        for (int i = 0; i < t.n_notifies; ++i) {
          const int w = cur.notify_word(t, i);
          const int e = w >> 8, dst = w & 0xFF;
          if (e >= 0 && e < p.n_events && dst < ev.world) ev.notify_1t_fenced(e, dst);
          else report_failure(p.status, MDC_DEV_BAD_OP, e, dst, 0, 0);
        }
      }
    }
    if (p.trace && tid == 0) {
      const unsigned long long slot = atomicAdd(p.trace, 1ull);
      if (slot < static_cast<unsigned long long>(p.trace_cap)) {
        unsigned long long* e = p.trace + 4 + 4 * slot;
        e[0] = (static_cast<unsigned long long>(blockIdx.x) << 32) | (static_cast<unsigned long long>(t.op & 0xff) << 24) |
               (static_cast<unsigned long long>(t.c0 & 0xfff) << 12) | static_cast<unsigned long long>(t.c1 & 0xfff);
        e[1] = tr0;
        e[2] = tr1;
        e[3] = global_timer_ns();
      }
    }
    __syncthreads();
  }
  if (dyn && tid == 0) {   // the last block to finish rewinds the counters for the next launch
    __threadfence();
    if (atomicAdd(p.dyn_ctl + 1, 1u) + 1u == gridDim.x) {
      p.dyn_ctl[0] = 0u;
      p.dyn_ctl[1] = 0u;
      __threadfence();
    }
  }
}

}  // namespace mdc

extern "C" int mdc_megakernel_smem_bytes(void) { return mdc::kMegaTileSmem + 1024; }
extern "C" int mdc_megakernel_threads(void) { return mdc::kMegaThreads; }

int mdc_attrs_megakernel(cudaFuncAttributes* a) { return static_cast<int>(cudaFuncGetAttributes(a, mdc::mega_kernel)); }

namespace mdc {
int logits_check(const mdc_logits_params* p);
int mla_check(const mdc_sparse_mla_params* p);
int compress_check(const mdc_compress_params* p, bool finalize);

// Everything a layer op dereferences or sizes shared memory with, checked on the host: a bad
// configuration comes back as an error code, it never reaches the device.  B == 0 means "no
// layer" (test queues); the kernel then refuses layer ops.
static int layer_check(const mdc_mega_params& p) {
  const mdc_layer_params& L = p.layer;
  if (L.B == 0) return MDC_OK;
  if (L.B < 0 || L.cp < 1 || L.rank < 0 || L.rank >= L.cp || L.top_k < 1 || L.n_chunks < 1) return MDC_ERR_BAD_SHAPE;
  if (L.cp != p.arena.world || L.rank != p.arena.my_rank || L.cp != p.events.world) return MDC_ERR_BAD_SHAPE;
  if (!p.arena.base || !p.arena.offsets) return MDC_ERR_NULL;
  int rc = logits_check(&L.logits);
  if (rc != MDC_OK) return rc;
  rc = mla_check(&L.mla);
  if (rc != MDC_OK) return rc;
  if (!L.logits.cand_v || L.logits.row_v || L.logits.q_len != 1 || L.mla.q_len != 1) return MDC_ERR_BAD_SHAPE;
  if (L.logits.B != L.B || L.mla.B != L.B || L.logits.top_k != L.top_k || L.logits.n_chunks != L.n_chunks)
    return MDC_ERR_BAD_SHAPE;
  if (L.H != L.mla.H || L.H % 64 != 0 || L.mla.n_splits != 1) return MDC_ERR_BAD_SHAPE;
  if ((L.top_k * 8 + 16) % 16 != 0) return MDC_ERR_BAD_ALIGN;  // candidate slices travel as 16-byte bulk copies
  if (L.mla.pt_cols < 1 || L.kv_seq_stride < 1 || L.phases < 1 || L.phase_bytes < 0 || L.kv_group < 0) return MDC_ERR_BAD_SHAPE;
  {  // the gather list holds 32-bit pool rows
    const long long groups = L.kv_group > 1 ? (L.B + L.kv_group - 1) / L.kv_group : L.B;
    if (groups * L.kv_seq_stride > 0x7fffffffLL) return MDC_ERR_TOO_LARGE;
  }
  if (!L.sel_v || !L.sel_i || !L.sel_c || !L.out) return MDC_ERR_NULL;
  if (L.out_dtype != MDC_DT_F32 && L.out_dtype != MDC_DT_BF16) return MDC_ERR_BAD_FORMAT;
  if (L.l1_groups > 1 && (!L.mid_v || !L.mid_i || !L.mid_c)) return MDC_ERR_NULL;
  if (L.l1_groups < 0 || L.l1_groups > L.n_chunks) return MDC_ERR_BAD_SHAPE;
  if (L.cand_direct && L.cp > 1 && (L.l1_groups > 1 || L.cp * L.n_chunks > 256)) return MDC_ERR_BAD_SHAPE;  // the merge takes 256 lists
  if (L.cand_direct && L.cp > 1 && L.top_k % 4 != 0) return MDC_ERR_BAD_ALIGN;   // the ids start on a 16-byte boundary of the slice
  if (L.thr_exact) {
    if (!L.thr_hist || !L.thr_done || L.thr_ev_base < p.n_events || (L.thr_off & 15)) return MDC_ERR_BAD_SHAPE;
    if (L.thr_exact != 1 && L.thr_exact != 2) return MDC_ERR_BAD_SHAPE;
    if (L.cp * L.n_chunks > kRowMaxSlots || L.l1_groups > 1) return MDC_ERR_BAD_SHAPE;
    if (L.cp > 1 && (L.thr_exact == 1) != (L.cand_direct != 0)) return MDC_ERR_BAD_SHAPE;   // 1: with the chunk lists' layout, 2: one list per rank
    if (L.top_k % 4 != 0) return MDC_ERR_BAD_ALIGN;   // the published selection is copied in 16-byte pieces
  }
  if (static_cast<long long>(L.cp) * (L.attn_splits > 1 ? L.attn_splits : 1) > kLseMaxSlices) return MDC_ERR_TOO_LARGE;
  // the chunk's scores stay in shared memory: the tile's layout must fit the kernel's allocation
  const int ct = L.logits.blocks_per_chunk * L.logits.page_tokens;
  int need;
  if (L.logits.fmt == MDC_FMT_MXFP4) need = logits_smem_layout<MDC_FMT_MXFP4, 128>(1, ct, true).total;
  else if (L.logits.page_tokens == 64) need = logits_smem_layout<MDC_FMT_NVFP4, 64>(1, ct, true).total;
  else need = logits_smem_layout<MDC_FMT_NVFP4, 128>(1, ct, true).total;
  if (need > kMegaTileSmem) return MDC_ERR_TOO_LARGE;
  if (L.q_stage && ((reinterpret_cast<uintptr_t>(L.q_stage) | static_cast<uintptr_t>(L.q_off)) & 15)) return MDC_ERR_BAD_ALIGN;
  if (L.q_stage && (L.logits.q_fmt != MDC_Q_BF16 || L.mla.kv_dtype != MDC_DT_BF16)) return MDC_ERR_BAD_FORMAT;
  if (L.kvw_glen) {
    if (!L.kvw_k_idx || !L.kvw_kv || !L.logits.seq_lens) return MDC_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(L.kvw_k_idx) | reinterpret_cast<uintptr_t>(L.kvw_kv)) & 15) return MDC_ERR_BAD_ALIGN;
    if (L.mla.page_cmp != 1) return MDC_ERR_BAD_SHAPE;   // the new row goes to pool row b * kv_seq_stride + slot
    if (L.kv_group > 1) return MDC_ERR_BAD_SHAPE;        // entries that share KV rows would write the same slot
  }
  if (L.cmp.B != 0) {  // compressor tasks: the tiles' own checks, with the fields the kernel fills in
    mdc_compress_params c = L.cmp;
    c.arena = p.arena;
    c.events = p.events;
    c.wait_budget_ns = p.wait_budget_ns;
    if (c.B != L.B || c.cp != L.cp || c.rank != L.rank) return MDC_ERR_BAD_SHAPE;
    rc = compress_check(&c, false);
    if (rc != MDC_OK) return rc;
    rc = compress_check(&c, true);
    if (rc != MDC_OK) return rc;
  }
  return MDC_OK;
}
}  // namespace mdc

extern "C" int mdc_megakernel_check(const mdc_mega_params* p) {
  using namespace mdc;
  if (!p || !p->queue || !p->scalars || !p->arity || !p->scopes || !p->events.base || !p->events.offsets)
    return MDC_ERR_NULL;
  if (p->n_ctas < 1 || p->row_words < 1 || p->n_events < 0) return MDC_ERR_BAD_SHAPE;
  if (p->dyn_task_off && (!p->dyn_ctl || p->dyn_n_tasks < 0)) return MDC_ERR_NULL;
  if (p->wait_budget_ns <= 0) return MDC_ERR_BAD_SHAPE;
  return layer_check(*p);
}

extern "C" int mdc_megakernel_launch(const mdc_mega_params* p, void* stream) {
  using namespace mdc;
  const int rc = mdc_megakernel_check(p);
  if (rc != MDC_OK) return rc;
  const int smem = mdc_megakernel_smem_bytes();
  MDC_CUDA_OK(cudaFuncSetAttribute(mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  // the blocks wait on each other: all of them must be resident at once
  int dev = 0, sms = 0, per_sm = 0;
  MDC_CUDA_OK(cudaGetDevice(&dev));
  MDC_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  MDC_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mega_kernel, kMegaThreads, smem));
  if (per_sm < 1 || p->n_ctas > sms * per_sm) return MDC_ERR_TOO_LARGE;
  mega_kernel<<<p->n_ctas, kMegaThreads, smem, static_cast<cudaStream_t>(stream)>>>(*p);
  MDC_CUDA_OK(cudaGetLastError());
  return MDC_OK;
}

