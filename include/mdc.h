/*
 * mdc.h -- C ABI of libmdc.so: sm_100a CUDA kernels for the context-parallel
 * DeepSeek-sparse-attention decode path (indexer logits, top-k selection and
 * merge, sparse MLA attention, LSE merge, KV compressor, event / comm /
 * scheduler device layer, persistent decode megakernel).
 *
 * Conventions
 *   - Every pointer is a device pointer unless stated otherwise; the caller
 *     owns all memory, the library allocates nothing (borrowed for the
 *     duration of the stream-ordered launch).
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous.
 *   - Return value: MDC_OK or a negative MDC_ERR_* code; nothing aborts.
 *   - Device-side failures (a wait that ran out of its budget, an id out of
 *     range) are written to the caller's 8-word `status` block (may be NULL):
 *     [0]=MDC_DEV_* code, [1]=block, [2..3]=detail, [4..5]=seen, [6..7]=wanted.
 *
 * Each entry point cites the interface of the reference project
 * (ultism/mega-dsa-cp, paths relative to its root) that it replaces.
 */
#ifndef MDC_H_
#define MDC_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MDC_ABI_VERSION 3

/* host-side return codes */
#define MDC_OK 0
#define MDC_ERR_BAD_SHAPE (-1)   /* unsupported size / count            */
#define MDC_ERR_BAD_ALIGN (-2)   /* pointer or stride not 16 B aligned  */
#define MDC_ERR_BAD_FORMAT (-3)  /* unknown format / dtype enum         */
#define MDC_ERR_NULL (-4)        /* required pointer missing            */
#define MDC_ERR_CUDA (-5)        /* CUDA runtime error, see mdc_last_cuda_error */
#define MDC_ERR_TOO_LARGE (-6)   /* exceeds a stated capacity           */

/* device-side status codes (status[0]) */
#define MDC_DEV_OK 0
#define MDC_DEV_WAIT_TIMEOUT 1   /* event wait gave up: [2]=event id            */
#define MDC_DEV_COPY_TIMEOUT 2   /* staged copy never completed: [2]=stage      */
#define MDC_DEV_BAD_INDEX 3      /* page / entry id out of range: [2]=id        */
#define MDC_DEV_BAD_OP 4         /* unknown task op code: [2]=op                */
#define MDC_DEV_ABORTED 5        /* left early because another block failed     */

/* index-K cache formats (E2M1 values, two per byte, even element low nibble) */
#define MDC_FMT_MXFP4 0 /* UE8M0 scale per 32 elements; page = [P x 64 B][atom-ordered scales] */
#define MDC_FMT_NVFP4 1 /* UE4M3 scale per 16 elements; page = [P x 64 B][P x 8 B scales]      */

/* query formats of the indexer */
#define MDC_Q_FP4 0  /* (B, N, 64) packed E2M1 + (B, N*4) atom-ordered UE8M0 scales */
#define MDC_Q_BF16 1 /* (B, N, 128) bf16                                             */

/* element types of attention operands / partial outputs */
#define MDC_DT_F32 0
#define MDC_DT_BF16 1
#define MDC_DT_E4M3 2

int mdc_abi_version(void);
const char* mdc_status_string(int code);
int mdc_last_cuda_error(void);
/* registers / static smem / max dynamic smem of a kernel, for co-residency
 * checks (the probe planned in docs/phase1.4-comm-tasks.md:14-16).
 * kernel ids: MDC_K_* below.  Needs a CUDA device. */
int mdc_kernel_attrs(int kernel_id, int* regs, int* static_smem, int* max_dynamic_smem);
#define MDC_K_LOGITS 0
#define MDC_K_MERGE_TOPK 1
#define MDC_K_LSE_MERGE 2
#define MDC_K_SPARSE_MLA 3
#define MDC_K_MEGAKERNEL 4
#define MDC_K_COUNT 5

/* ------------------------------------------------------------------------
 * FP4 paged MQA indexer logits (+ optional fused exact local top-k).
 * Replaces run_fp4_paged_mqa_logits, mega_dsa_cp/tiles/logits.py:1054-1145
 * (kernel Fp4PagedMQALogits.kernel, logits.py:421-870; candidate heap
 * logits.py:886-1042).
 *
 *   logits[(b*q_len+t), pos] = sum_h w[b, t*heads+h] * relu(q[b, t*heads+h] . k[pos])
 *   k[pos] = dequantised row (pos % page_tokens) of page block_table[b, pos / page_tokens]
 *
 * One thread block per (chunk, b); a chunk is `blocks_per_chunk` consecutive
 * page-table entries.  With cand_v == NULL the fp32 logits row is written.
 * With cand_v != NULL the block keeps its scores on chip and emits the exact
 * top_k of the chunk positions pos < seq_lens[b] - window_exclude under the
 * total order (logit descending, position ascending), in position order:
 *   cand_v/cand_i (B, q_len, n_chunks, top_k), cand_c (B, q_len, n_chunks),
 *   cand_i = pos * id_mul + id_add   (global token id under token-interleaved
 *   context parallelism: id_mul = cp, id_add = rank).
 * Page ids outside [0, num_pages) produce -inf scores and MDC_DEV_BAD_INDEX.
 * ------------------------------------------------------------------------ */
typedef struct {
  const uint8_t* kv_pages;   /* (num_pages, page_bytes) fused pages, 16 B aligned */
  int32_t num_pages;
  int32_t page_tokens;       /* 64 or 128 (MXFP4: 128 only)                       */
  int32_t fmt;               /* MDC_FMT_*                                          */
  int32_t q_fmt;             /* MDC_Q_*                                            */
  const void* q;             /* see MDC_Q_*; N = q_len*heads rows per request      */
  const uint8_t* q_sf;       /* MDC_Q_FP4 only: (B, N*4) atom-ordered scales        */
  const float* weights;      /* (B, N) head-gate weights                           */
  const int32_t* block_table;/* (B, max_pages)                                     */
  int32_t max_pages;
  const int32_t* seq_lens;   /* (B,) rank-local token counts; NULL = max_pages*page_tokens */
  float* logits;             /* (B*q_len, logits_stride) or NULL when fused        */
  int64_t logits_stride;
  float* cand_v;             /* fused top-k outputs, or NULL                        */
  int32_t* cand_i;
  int32_t* cand_c;
  int32_t top_k;             /* multiple of 32, <= 2048 (fused only)                */
  int32_t B;
  int32_t q_len;             /* 1 or 2                                              */
  int32_t heads;             /* 64                                                  */
  int32_t blocks_per_chunk;
  int32_t n_chunks;
  int32_t window_exclude;    /* reference: 128 (sliding-window tokens skipped)      */
  int32_t id_mul, id_add;
  int32_t* status;           /* 8 words or NULL                                     */
  /* Row mode (ABI 2, no counterpart in the reference): when row_v is set, the n_chunks blocks
   * of a request run as one thread-block cluster (n_chunks in {1,2,4,8}, chunk <= 8192 tokens)
   * and select the exact top_k of the WHOLE row across their chunks, written in position order:
   * the same result as fused candidates followed by mdc_merge_topk_launch, in one launch.
   * cand_* are ignored in this mode. */
  float* row_v;              /* (B, q_len, top_k) or NULL                           */
  int32_t* row_i;            /* (B, q_len, top_k)                                   */
  int32_t* row_c;            /* (B, q_len)                                          */
} mdc_logits_params;
int mdc_logits_fp4_launch(const mdc_logits_params* p, void* stream);
/* dynamic shared memory the launch above will request (bytes), or <0 */
int mdc_logits_fp4_smem_bytes(const mdc_logits_params* p);

/* ------------------------------------------------------------------------
 * Exact top-k over L candidate lists per (b, t); deterministic input-order
 * emit.  Replaces run_merge_topk, mega_dsa_cp/tiles/merge.py:347-379 (kernel
 * MergeTopK.kernel, merge.py:147-323).  Total order: logit descending (bit
 * level, so -0.0 < +0.0), then id ascending (as signed int32 ids >= 0).
 * dbg (>= 1 word, may be NULL): [0] += 1 per (b,t) whose emitted count
 * differs from min(total, top_k).
 * ------------------------------------------------------------------------ */
typedef struct {
  const float* cand_v;    /* (B, q_len, L, maxK) */
  const int32_t* cand_i;  /* (B, q_len, L, maxK) */
  const int32_t* cand_c;  /* (B, q_len, L)       */
  float* out_v;           /* (B, q_len, top_k)   */
  int32_t* out_i;         /* (B, q_len, top_k)   */
  int32_t* out_c;         /* (B, q_len)          */
  int32_t* dbg;
  int32_t B, q_len, L, maxK, top_k;
} mdc_merge_topk_params;
int mdc_merge_topk_launch(const mdc_merge_topk_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Merge of per-rank (or per-split) normalised attention partials by their
 * log2-domain LSE.  Replaces run_lse_merge, mega_dsa_cp/tiles/lse_merge.py:175-197
 * (kernel LseMerge.kernel, lse_merge.py:77-142):
 *   g = max_i l_i; glse = g + log2(sum_i 2^(l_i-g)); O = sum_i O_i * 2^(l_i-glse);
 *   all-empty heads give O = 0, glse = -inf.
 * Partials: acc_o (rows, n_slices_max, H, D) in acc_dtype, acc_lse (rows,
 * n_slices_max, H) fp32, rows = B*q_len; the first n_slices slices are merged.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* acc_o;
  const float* acc_lse;
  void* o;               /* (rows, H, D) in out_dtype */
  float* lse;            /* (rows, H) or NULL         */
  int32_t rows, H, D;
  int32_t n_slices, n_slices_max;
  int32_t acc_dtype;     /* MDC_DT_F32 | MDC_DT_BF16  */
  int32_t out_dtype;     /* MDC_DT_F32 | MDC_DT_BF16  */
} mdc_lse_merge_params;
int mdc_lse_merge_launch(const mdc_lse_merge_params* p, void* stream);

/* ------------------------------------------------------------------------
 * Sparse MLA decode attention over a window pool plus a gathered pool.
 * Replaces run_hca_fp8, mega_dsa_cp/tiles/hca.py:3160-3270 (kernel
 * HcaFp8Forward.attention_kernel, hca.py:694-1206).
 *
 * Row r = b*q_len + t attends to slots [0,128) = kv_win[pt_win[r]] (valid
 * below win_valid[r]) and slots [128, k_valid[r]) = gathered rows
 * kv_cmp[id] for id = pt_cmp[r, slot-128] (page_cmp == 1) or entry
 * (slot-128) % page_cmp of page pt_cmp[r, (slot-128)/page_cmp].  V is the
 * first d_v columns of K.  attn_sink[h] (-inf = off) adds a zero-valued
 * logit.  Output is normalised; lse = log2(sum) + scale*log2(e)*max, or
 * -inf with O = 0 when nothing is valid.
 *
 * n_splits > 1 splits the slot range; partials go to `ws_o` (rows, n_splits,
 * H, d_v) fp32 and `ws_lse` (rows, n_splits, H) and are merged into o / lse
 * by a second kernel launched by the same call.  Workspace is caller-owned.
 * fp8_p != 0 rounds the probabilities through e4m3 before P.V, as the
 * reference kernel does.
 * ------------------------------------------------------------------------ */
typedef struct {
  const void* q;            /* (B, q_len, H, d_qk) kv_dtype                  */
  const void* kv_win;       /* (pages_win, 128, d_qk) or NULL                */
  const void* kv_cmp;       /* (pages_cmp, page_cmp, d_qk)                   */
  const int32_t* pt_win;    /* (rows,) window page per row, or NULL          */
  const int32_t* pt_cmp;    /* (rows, pt_cols)                               */
  const int32_t* k_valid;   /* (rows,) includes the 128 window slots         */
  const int32_t* win_valid; /* (rows,) or NULL (= 0)                         */
  const float* attn_sink;   /* (H,) or NULL                                  */
  void* o;                  /* (rows, H, d_v) out_dtype, row stride o_stride */
  float* lse;               /* (rows, H), row stride lse_stride, or NULL     */
  int64_t o_stride;         /* elements between consecutive rows of o        */
  int64_t lse_stride;
  float* ws_o;              /* split workspace (n_splits > 1)                */
  float* ws_lse;
  int32_t B, q_len, H;      /* H multiple of 64                              */
  int32_t d_qk, d_v;        /* (576,512) or (512,512)                        */
  int32_t pages_win, pages_cmp, page_cmp, pt_cols;
  int32_t kv_dtype;         /* MDC_DT_BF16 | MDC_DT_E4M3                     */
  int32_t out_dtype;        /* MDC_DT_F32 | MDC_DT_BF16                      */
  int32_t n_splits;
  int32_t fp8_p;
  float softmax_scale;
  float output_scale;
  int32_t* status;
} mdc_sparse_mla_params;
int mdc_sparse_mla_launch(const mdc_sparse_mla_params* p, void* stream);
int mdc_sparse_mla_smem_bytes(const mdc_sparse_mla_params* p);

/* Same launch, but the split workspace is a fixed block inside the library's own
 * device data (p->ws_o / p->ws_lse are ignored), so the call enters no allocator.
 * No counterpart in the reference: it exists for callers that cannot allocate
 * at launch time (all device memory already given to a cache pool; a thread that
 * must not take the allocator's lock).  Capacity: B * q_len * n_splits * H <=
 * MDC_STATIC_WS_MAX_SLOTS, else MDC_ERR_TOO_LARGE and nothing is launched.  The
 * first call on a device is a warm-up: it loads the library's device data segment
 * (8 MiB + 16 KiB, held until the process exits) and looks the block's address up
 * once.  Make it at start-up: before the application commits the remaining device
 * memory to its pool (later it could fail with MDC_ERR_CUDA / out of memory) and
 * before any stream capture begins.  One block per device: calls whose kernels
 * may overlap race on it.  Nothing has to be cleared between calls; a call whose
 * status block comes back non-zero leaves o / lse undefined. */
#define MDC_STATIC_WS_MAX_SLOTS 4096
int mdc_sparse_mla_launch_static_ws(const mdc_sparse_mla_params* p, void* stream);


/* ------------------------------------------------------------------------
 * Event / comm / scheduler device layer and the persistent decode megakernel.
 *
 * mdc_event_set replaces the device view EventSet (mega_dsa_cp/events/core.py:40-62):
 * 128-byte cells of u64 counters, `offsets[r]` = byte offset of rank r's cells
 * from `base`.  mdc_peer_buffer replaces PeerBuffer (comm/device.py:11-44).
 * ------------------------------------------------------------------------ */
typedef struct {
  void* base;
  const int64_t* offsets; /* device, [world] */
  int32_t my_rank;
  int32_t world;
} mdc_event_set;

typedef struct {
  void* base;
  const int64_t* offsets; /* device, [world] */
  int32_t my_rank;
  int32_t world;
  int64_t mc_base;        /* NVLS multicast address or 0 */
} mdc_peer_buffer;

/* ------------------------------------------------------------------------
 * KV compressor: softmax-gated pooling of token records into compressed
 * entries, context-parallel (per-rank partial statistics -> pushed to the
 * entry's owner rank -> owner merges, normalises, rotates, quantises and
 * writes its pools).  Replaces the four kernels and launchers of
 * mega_dsa_cp/tiles/compress.py:120-250 (csa step), :284-523 (csa finalize),
 * :564-640 (c128 step), :669-792 (c128 finalize) and the micro kernel :828-889.
 *
 * ratio == 4 : overlapping 8-slot window machine, two streams (attention 512
 *              channels, indexer 128 channels), records (B, 4*hd) =
 *              [kv_overlap | kv_normal | score_overlap | score_normal]; rings
 *              (B, ring_slots, 4*hd), slot of local record l = l % ring_slots.
 * ratio == 64 / 128 : online machine, one stream of 512 channels, records
 *              (B, 2*512) = [kv | score], running state (B, 3, 512) = [m | l | kv].
 * A step covers global positions seq_len[b] .. seq_len[b] + q_len - 1; this
 * rank owns the position p with p % cp == rank (q_len <= cp).  Entry n is
 * owned by rank n % cp and stored at its local slot n / cp.
 * Statistics region: (B, cp, stats_bytes) at arena offset stats_off with
 * stats_bytes = 7696 (ratio 4) or 6160 (online); event cell ev_base_id + b is
 * bumped once per rank per step on every rank (arity cp).
 * ------------------------------------------------------------------------ */
typedef struct {
  int32_t B, cp, rank, q_len, ratio;
  int32_t phase;               /* finalize: waits for cell value cp * (phase + 1)        */
  const int32_t* seq_len;      /* (B,) global length before the step                     */
  float* ring_attn;            /* ratio 4: (B, 8, 4*512) ring of this rank's records     */
  float* ring_idx;             /* ratio 4: (B, 8, 4*128)                                 */
  const float* new_attn;       /* ratio 4: (B, 4*512); online: (B, 2*512)                */
  const float* new_idx;        /* ratio 4: (B, 4*128)                                    */
  const float* ape_attn;       /* ratio 4: (8, 512) slot bias; online: (ratio, 512)      */
  const float* ape_idx;        /* ratio 4: (8, 128)                                      */
  float* state;                /* online: (B, 3, 512)                                    */
  mdc_peer_buffer arena;
  int64_t stats_off;
  mdc_event_set events;
  int32_t ev_base_id;
  int32_t do_push;             /* 0 skips the payload push (bisecting aid)               */
  int64_t wait_budget_ns;
  const float* norm_w_attn;    /* (512,)                                                 */
  const float* norm_w_idx;     /* (128,)                                                 */
  const float* freqs;          /* (freq_rows, 64) rope table [cos0, sin0, cos1, ...]     */
  int32_t freq_rows;
  float norm_eps;
  float inv_fp8_scale;
  int32_t attn_pool_dtype;     /* MDC_DT_E4M3 | MDC_DT_BF16                              */
  void* attn_pool;             /* (B, max_entries, 512)                                  */
  uint8_t* idx_pool;           /* ratio 4: (B, max_entries / idx_page_tokens, page bytes) */
  int32_t idx_fmt;             /* MDC_FMT_*                                              */
  int32_t idx_page_tokens;
  int32_t max_entries;
  int32_t ring_slots;          /* ratio 4: slots of ring_attn / ring_idx per sequence, >= ceil(8 / cp); 0 = 8.  The reference's ring holds 4 (cp = 2, compress.py:43) */
  int32_t* k_valid;            /* (B,) entries held by this rank                         */
  float* dbg_attn;             /* (B, max_entries, 512) merged fp32 before the norm, or NULL */
  float* dbg_idx;              /* (B, max_entries, 128) or NULL                          */
  int32_t* status;
} mdc_compress_params;
int mdc_compress_step_launch(const mdc_compress_params* p, void* stream);
int mdc_compress_finalize_launch(const mdc_compress_params* p, void* stream);
/* staged 128-point Hadamard + MXFP4 quantisation of n rows: x (n, 128) fp32 ->
 * out (n, 68) = 64 B packed codes + 4 B UE8M0 (compress.py:828-889) */
int mdc_hadamard_quant_launch(const float* x, uint8_t* out, int32_t n, void* stream);


/* Latency probe of the event layer: a ping-pong over two event cells, timed on the pinging side with
 * %globaltimer (replaces pingpong_kernel / waitoverhead_kernel of tests/bench_notify_latency.py:49-143).
 * role 0 pings (notify ev_ping at `peer`, wait for the own ev_pong), role 1 pongs; launched on two GPUs,
 * one block each.  role 2 runs both roles as two blocks of ONE launch on one GPU (peer = own rank).
 * Cells are monotonic: `base` = value of both cells before the launch.  out_ns (pinging side):
 * rounds round-trip times in ns, then one more entry = mean cost of a wait that is already satisfied. */
typedef struct {
  mdc_event_set events;
  int32_t role, peer, ev_ping, ev_pong, rounds;
  uint64_t base;
  int64_t wait_budget_ns;
  unsigned long long* out_ns;  /* rounds + 1 entries, or NULL (pong side) */
  int32_t* status;
} mdc_pingpong_params;
int mdc_test_pingpong_launch(const mdc_pingpong_params* p, void* stream);

/* task op codes understood by mdc_megakernel_launch */
#define MDC_OP_NOP 0
#define MDC_OP_LOGITS 1     /* c0 = b, c1 = chunk                                  */
#define MDC_OP_MERGE_L1 2   /* c0 = b: chunk lists -> local top-k -> every rank    */
#define MDC_OP_MERGE_L2 3   /* c0 = b: cp lists -> global top-k + local gather list */
#define MDC_OP_ATTN 4       /* c0 = b, c1 = head/column block (see megakernel.cu), c2 = slot split: partial -> owner inbox */
#define MDC_OP_MERGE_L1A 6  /* c0 = b, c1 = group: chunk lists of the group -> mid list              */
#define MDC_OP_LSE_MERGE 5  /* c0 = b (owned), c1 = head group of c2 groups: inbox slices -> output */
#define MDC_OP_CMP_STEP 7   /* c0 = b: compressor step of layer.cmp (record append, statistics push to the entry owner)  */
#define MDC_OP_CMP_FIN 8    /* c0 = b: entry owner merges the cp statistics and writes its pools                       */
#define MDC_OP_QPATH 9      /* c0 = b (owned), c1 = part (0: indexer q + weights; 1 + s: slice s of c2 slices of the attention q): this step's query block of sequence b -> every rank's arena */
#define MDC_OP_KVWRITE 10   /* c0 = b: the step's new token of sequence b -> index-K page and KV row of its owner (kv_written[b]) */
#define MDC_OP_SLEEP 16     /* c1 = nanoseconds (test op)                          */
#define MDC_OP_LOG 17       /* appends c0 to the execution log (test op)           */
#define MDC_OP_PUSH 18      /* c1 = dst rank, c2 = slot: bulk push a pattern (test op) */
#define MDC_OP_VERIFY 19    /* c1 = src rank, c2 = slot: check a pushed pattern (test op) */

/* One decode layer-step of context-parallel sparse attention, one query token
 * per sequence (the composition planned in docs/phase1.4-comm-tasks.md:37-117
 * of the reference).  Rank r holds tokens t with t % cp == r at local index
 * t / cp.  All buffers are per rank; the arena regions are per phase.
 *   cand region : (B, cp, cand_slice) with cand_slice = top_k*8 + 16 bytes:
 *                 [i32 count, pad to 16 bytes][top_k f32 logits][top_k i32 global ids]
 *   inbox region: (B_owned, cp, H*512*2 + H*4) bytes, owner(b) = b % cp,
 *                 owned index b / cp: [H x 512 bf16 partial O][H f32 log2-LSE]  */
#define MDC_THR_BINS 4096  /* bins of the row histogram: the upper 12 bits of the order-preserving u32 image of a score */

typedef struct {
  int32_t cp, rank, B, top_k, H;
  int32_t n_chunks;             /* chunks per sequence in `logits`             */
  int32_t kv_seq_stride;        /* KV pool row of local token l of sequence b = b*kv_seq_stride + l (see kv_group) */
  int32_t attn_splits;          /* ATTN tasks per (b, block) over the slot range (0 or 1 = no split); inbox holds cp * attn_splits slices per sequence */
  mdc_logits_params logits;     /* fused mode; cand_* = chunk candidate scratch */
  mdc_sparse_mla_params mla;    /* local KV pool; pt_cmp/k_valid = local gather list written by MERGE_L2 */
  int64_t cand_off, inbox_off;  /* byte offsets of the regions inside one phase */
  int64_t phase_bytes;          /* arena bytes per phase                         */
  int32_t phases;
  float* sel_v;                 /* (B, top_k) merged logits                      */
  int32_t* sel_i;               /* (B, top_k) global ids, identical on every rank */
  int32_t* sel_c;               /* (B,)                                          */
  void* out;                    /* (ceil(B/cp), H, 512) merged attention output of the owned sequences: row b / cp for b % cp == rank */
  float* out_lse;               /* (ceil(B/cp), H)                               */
  int32_t out_dtype;            /* MDC_DT_F32 | MDC_DT_BF16                      */
  /* two-level local merge: with l1_groups > 1 MERGE_L1A tasks first merge the chunk lists of one
   * group (ceil(n_chunks / l1_groups) lists each) into mid_*, and MERGE_L1 merges the groups */
  int32_t l1_groups;
  float* mid_v;                 /* (B, l1_groups, top_k)                         */
  int32_t* mid_i;               /* (B, l1_groups, top_k)                         */
  int32_t* mid_c;               /* (B, l1_groups)                                */
  /* KV compressor of the layer as CMP_STEP / CMP_FIN tasks (docs/phase1.4-comm-tasks.md:37-38,52,67 of the
   * reference: ops of the layer DAG, event cmp_stats_arrived[b] with arity cp, arena region cmp_stats).
   * cmp.B == 0: the layer has no compressor tasks.  The tasks' wait / notify edges replace the event
   * fields of cmp (events, ev_base_id, phase, wait_budget_ns are not used); cmp.stats_off is the offset
   * of the statistics region inside ONE phase of the arena (the kernel adds the phase rotation). */
  mdc_compress_params cmp;
  /* Query path (the reference's QPATH_STUB task and q_ready event, docs/phase1.4-comm-tasks.md:37,48,117:
   * "the host supplies q").  q_stage == NULL: logits.q / logits.weights / mla.q are read as given
   * (replicated on every rank by the caller).  Else the owner of sequence b (b % cp) holds that
   * sequence's per-step block in q_stage, laid out over its owned sequences j = b / cp as
   *   [ (n_owned, 64, 128) bf16 indexer q | (n_owned, 64) f32 gate weights | (n_owned, H, d_qk) bf16 attention q ],
   * and QPATH(b) stores it into the q region of EVERY rank's arena (offset q_off inside a phase, same
   * three arrays over all B sequences); the indexer and attention tiles then read q from the arena.
   * Each rank receives 1/cp of the bytes from its host instead of all of them. */
  const void* q_stage;
  int64_t q_off;
  /* New-token write (the reference's KVWRITE task and kv_written event, docs/phase1.4-comm-tasks.md:37,49,
   * 114-116: "host-supplied new token KV / index records are written into the pools, the valid counters
   * updated").  kvw_glen == NULL: no KVWRITE tasks.  Else every rank runs KVWRITE(b): with t = kvw_glen[b]
   * (global length before the step, the same on every rank), the rank with t % cp == rank quantises
   * kvw_k_idx[b] to the cache format and writes it into slot t / cp of its index-K cache (page
   * block_table[b][slot / page_tokens], which must be allocated), copies kvw_kv[b] to KV pool row
   * b * kv_seq_stride + slot, and sets logits.seq_lens[b] = slot + 1 (seq_lens is written here).  The
   * indexer tasks of b wait for kv_written[b]: the new token takes part in this step's selection.
   * kvw_advance != 0: the task then adds 1 to kvw_glen[b], so a replayed launch writes the next token. */
  const float* kvw_k_idx;       /* (B, 128) fp32, replicated on every rank       */
  const void* kvw_kv;           /* (B, d_qk) elements of mla.kv_dtype, replicated */
  int32_t* kvw_glen;            /* (B,)                                          */
  int32_t kvw_advance;
  /* Row-threshold candidate filter (no counterpart in the reference, whose chunk tasks emit exact chunk
   * top-k lists).  thr_hist != NULL: the LOGITS tasks of a sequence sum an MDC_THR_BINS-bin histogram of their
   * scores in thr_hist, wait for each other (bounded), and emit only the scores in the bins that can
   * still hold the row's top_k: about top_k candidates per sequence instead of top_k per chunk, one
   * MERGE_L1 behind them (l1_groups = 1).  thr_hist: (2, B, MDC_THR_BINS) u32, zero before the first step (the
   * kernel keeps the two halves zeroed in turn); thr_done: (B,) u32, zero before the first step. */
  uint32_t* thr_hist;
  uint32_t* thr_done;
  /* Batch entries that share one sequence's KV rows (chunked prefill: the query tokens of a tile are
   * batch entries with their own causal lengths): the KV pool row of local token l of entry b is
   * (b / kv_group) * kv_seq_stride + l.  0 or 1: every entry is its own sequence (decode). */
  int32_t kv_group;
  /* cp > 1 only.  1: the LOGITS tasks store their chunk lists into every rank's cand region themselves
   * (the region then holds (B, cp, n_chunks, cand_slice): rank-major, chunk-minor) and MERGE_L2 merges
   * cp * n_chunks lists; no MERGE_L1 task may be queued.  0: MERGE_L1 stores one exact list per rank. */
  int32_t cand_direct;
  /* Exact row selection inside the LOGITS tasks (needs thr_hist / thr_done; no counterpart in the
   * reference).  thr_exact = 1: the chunk tasks of a row, on all ranks, agree on the row's exact top-k
   * through a histogram exchange and a short list of undecided keys, write the selection and the gather
   * lists themselves and mark their candidate counts -1; the merge task of the row (MERGE_L1 with one
   * rank, MERGE_L2 with several and cand_direct = 1, which it requires there) then only passes the result
   * on.  Heavily tied rows fall back to the merge.  thr_exact = 2 (several ranks, cand_direct = 0): the chunk
   * tasks of a rank settle the RANK's exact top-k the same way, without any exchange between ranks, and store
   * it as the rank's candidate list on every rank; MERGE_L1 then only passes on, MERGE_L2 merges cp lists.  thr_off: byte offset inside one arena phase of
   * (B, cp * 4 * MDC_THR_BINS + cp * n_chunks * 2064) bytes of exchange space (histograms per rank, then one slot per
   * rank and chunk); thr_ev_base: first of 2 * B extra event cells (beyond the queue's events) of the
   * event buffer: cell thr_ev_base + b counts histogram arrivals, thr_ev_base + B + b slot arrivals. */
  int32_t thr_exact, thr_ev_base;
  int64_t thr_off;
  /* Optional: the attention query of the step (mla.q without q_stage, the q_mla part of q_stage with it)
   * arrives by a host copy that may still be in flight when the launch starts.  The tasks that read it first
   * (ATTN, or QPATH parts >= 1) then wait, bounded by wait_budget_ns, until *q_host_flag >= phase + 1; the
   * host writes that value with a copy queued behind the query's copy on the same stream.  The wait is on
   * a DMA, not on another kernel.  NULL: the query is in place when the launch starts. */
  const unsigned long long* q_host_flag;
} mdc_layer_params;

/* Persistent kernel: block i walks queue row i (format of
 * mega_dsa_cp/schedule/codegen.py:3-11), executes each task's inline waits,
 * dispatches on the op code, executes its notifies.  Replaces the scheduler
 * device loop of schedule/device.py:35-129 and the skeleton kernel of
 * tests/test_skeleton_cp2.py:144-240.  n_ctas must not exceed the number of
 * blocks that can be co-resident (one per SM): tasks wait on each other. */
typedef struct {
  const int32_t* queue;        /* (n_ctas, row_words) */
  int32_t row_words, n_ctas;
  const uint64_t* scalars;     /* [0] = phase, [1..] dynamic extents */
  const int32_t* arity;        /* per event: notifies per phase into this rank's cell */
  const int32_t* scopes;       /* per event: 0 local, 1 sys */
  int32_t n_events;
  mdc_event_set events;
  mdc_peer_buffer arena;
  int64_t wait_budget_ns;      /* every event wait gives up after this long */
  int32_t* status;             /* 8 words, see top of file */
  int32_t* log;                /* [0] = entries used, then entries; or NULL */
  int32_t log_cap;
  int64_t test_off;            /* arena offset of the test region (PUSH / VERIFY) */
  int32_t test_slot_bytes;
  mdc_layer_params layer;
  /* Optional task timeline (NULL = off): trace[0] counts entries; entry i occupies the four
   * words trace[4+4i..]: (block << 32 | op << 24 | (c0 & 0xfff) << 12 | (c1 & 0xfff)),
   * globaltimer ns at task start, after its waits, at its end (after the notifies). */
  unsigned long long* trace;
  int32_t trace_cap;           /* entries                                        */
  /* Device-side phase counter (docs/event-system.md:32-36 of the reference: "a step counter kept on
   * the device, +1 per replay", so that a captured CUDA graph replays without host updates).
   * NULL: the host writes scalars[0] before every launch.  Else one u64, zero at start: every block
   * counts in after reading scalars[0]; the last one stores scalars[0] + 1 for the next launch and
   * clears the counter (scalars must then be writable). */
  unsigned long long* phase_ctl;
  /* Dynamic scheduling (the reference plans a dynamic scheduler, docs/event-system.md:27,110; its code has
   * the static queues only).  dyn_task_off != NULL: `queue` holds ONE row (row_words words) with all of this
   * rank's tasks in dependency order; dyn_task_off[i] is the word offset of task i, dyn_n_tasks their number;
   * the n_ctas blocks pull the next task with an atomic counter instead of walking a row of their own.  A task's
   * producers come earlier in the row, so they are always running or done when it is pulled.  dyn_ctl: two
   * u32 words, zero before the first launch (next task, finished blocks); the last block to finish clears
   * them, so a launch can be replayed. */
  const int32_t* dyn_task_off;
  int32_t dyn_n_tasks;
  uint32_t* dyn_ctl;
} mdc_mega_params;
int mdc_megakernel_launch(const mdc_mega_params* p, void* stream);
/* The host-side validation of a launch alone (no GPU needed): the return code mdc_megakernel_launch
 * would give for these parameters before it touches the device.  With layer.B != 0 it covers the
 * layer: both tiles' own checks, counts that size on-chip arrays (cp * attn_splits <= 16 LSE
 * slices, the chunk's scores within the kernel's shared memory), strides and required pointers. */
int mdc_megakernel_check(const mdc_mega_params* p);
int mdc_megakernel_smem_bytes(void);
int mdc_megakernel_threads(void);

#ifdef __cplusplus
}
#endif
#endif /* MDC_H_ */
