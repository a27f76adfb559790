"""One decode layer-step of context-parallel DeepSeek sparse attention as a
single persistent-kernel launch per rank.

Per rank r of cp ranks (token t lives on rank t % cp at local index t // cp):

    LOGITS(b, c)   indexer logits + exact local top-k of chunk c     (x B x C)
    MERGE_L1A(b,g) (more than 8 chunks only) the chunk lists of group g -> one list
    MERGE_L1(b)    chunk (or group) lists -> rank-local top-k, stored into every rank's arena
    MERGE_L2(b)    cp lists -> global top-k (bit-identical on all ranks) and
                   this rank's gather list (ids with id % cp == r)
    ATTN(b, j)     sparse MLA over the local share, 64 heads x 256 columns per
                   task; bf16 partial + log2-LSE stored into the owner's inbox
    LSE_MERGE(b)   on owner b % cp: cp (x attention splits) partials -> output row,
                   8 tasks of 16 heads

wired by events l1[b], cand[b], topk[b], part[b] (docs/phase1.4-comm-tasks.md
section 3 of the reference; its design never got assembled there).  The task
graph is validated and turned into per-block queues by schedule.codegen; the
device side is csrc/megakernel.cu.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _native as N
from .comm.buffers import alloc_arena
from .events import SCOPE_LOCAL, SCOPE_SYS, EventSpec, NotifyEdge, TaskSpec, WaitEdge
from .events.symm import alloc_event_buffer
from .schedule.codegen import codegen_schedule
from .schedule.device import launch_megakernel, upload_schedule

D_V = 512
LSE_GROUPS = 8
QPATH_SLICES = 8
THR_BINS = 4096   # MDC_THR_BINS of include/mdc.h
THR_HIST_BYTES, THR_SLOT_BYTES = THR_BINS * 4, 16 + 512 * 4   # exchange space of the exact row selection


def l1_groups_for(n_chunks: int) -> int:
    """Groups of the two-level local merge: up to 8 chunk lists (16384 candidates, the largest row the
    register search takes) are merged directly; beyond that, first-level tasks of at most 4 lists
    (measured: 4 x 4 beats 2 x 8 at 16 chunks)."""
    return 1 if n_chunks <= 8 else -(-n_chunks // 4)


def build_layer_dag(B: int, n_chunks: int, cp: int, heads: int = 128, attn_splits: int = 1, l1_groups: int = 1,
                    compressor: bool = False, qpath: bool = False, kvwrite: bool = False, cand_direct: bool = False):
    """Tasks / events of one layer-step for ALL ranks, plus op codes by task name.  With `cand_direct`
    (cp > 1, one merge level) the LOGITS tasks store their chunk lists into every rank's arena
    themselves and notify cand[b] there (arity cp x n_chunks); no MERGE_L1 task runs.  With `compressor`
    every rank also runs CMP_STEP(b) (record append + statistics push, notifies cmp_stats[b] on all
    ranks) and CMP_FIN(b) (entry owner, waits for the cp statistics); they are listed last, so the
    queues hold them behind the attention path (docs/phase1.4-comm-tasks.md:37-38,52 of the reference)."""
    cross = SCOPE_SYS if cp > 1 else SCOPE_LOCAL
    cand_direct = cand_direct and cp > 1
    assert not (cand_direct and l1_groups > 1)
    events, tasks, ops = [], [], {}
    for b in range(B):
        if l1_groups > 1:
            events += [EventSpec(f"l1a[{b},{g}]", SCOPE_LOCAL) for g in range(l1_groups)]
        if qpath or not cand_direct:    # (direct: only the held-back attention-query slices wait for it)
            events += [EventSpec(f"l1[{b}]", SCOPE_LOCAL)]
        events += [EventSpec(f"cand[{b}]", cross)] if cp > 1 else []
        events += [EventSpec(f"topk[{b}]", SCOPE_LOCAL), EventSpec(f"part[{b}]", cross)]
    n_attn = 2 * (heads // 64)
    per = -(-n_chunks // l1_groups)
    if qpath:   # QPATH(b, part) on the owner of b: the step's query block -> every rank's arena; the small indexer
        # part first (q_ready[b] releases the LOGITS tasks), the attention query behind it (qm_ready[b])
        events += [EventSpec(f"q_ready[{b}]", cross) for b in range(B)]
        events += [EventSpec(f"qm_ready[{b}]", cross) for b in range(B)]
    if kvwrite:  # KVWRITE(b) on every rank (the owner of the new position acts); the indexer of b waits for it
        events += [EventSpec(f"kv_written[{b}]", SCOPE_LOCAL) for b in range(B)]
    for r in range(cp):
        if kvwrite:
            for b in range(B):
                name = f"kvwrite[{r},{b}]"
                tasks.append(TaskSpec(name, r, (), (NotifyEdge(f"kv_written[{b}]", r),), (b, 0, 0)))
                ops[name] = N.OP_KVWRITE
        if qpath:
            for b in range(r, B, cp):
                name = f"qpath_idx[{r},{b}]"
                tasks.append(TaskSpec(name, r, (), tuple(NotifyEdge(f"q_ready[{b}]", d) for d in range(cp)), (b, 0, 0)))
                ops[name] = N.OP_QPATH

        for b in range(B):
            for c in range(n_chunks):
                name = f"logits[{r},{b},{c}]"
                ev = f"l1a[{b},{c // per}]" if l1_groups > 1 else f"l1[{b}]"
                waits = ((WaitEdge(f"q_ready[{b}]"),) if qpath else ()) + ((WaitEdge(f"kv_written[{b}]"),) if kvwrite else ())
                # (direct: l1[b] only gates the owner's held-back attention-query slices)
                out = (NotifyEdge(ev, r),) if not cand_direct or (qpath and b % cp == r) else ()
                if cand_direct:
                    out += tuple(NotifyEdge(f"cand[{b}]", d) for d in range(cp))
                tasks.append(TaskSpec(name, r, waits, out, (b, c, 0)))
                ops[name] = N.OP_LOGITS
        if qpath:
            # The attention query in slices (one SM moves only ~45 GB/s), held back until the owner's own
            # indexer tasks of the row are through (they wait for l1[b] / the row's first-level event): the
            # attention needs it much later, and nothing is queued ahead of the LOGITS tasks this way.
            for b in range(r, B, cp):
                gate = f"l1a[{b},0]" if l1_groups > 1 else f"l1[{b}]"
                for s in range(QPATH_SLICES):
                    name = f"qpath_mla[{r},{b},{s}]"
                    tasks.append(TaskSpec(name, r, (WaitEdge(gate),), tuple(NotifyEdge(f"qm_ready[{b}]", d) for d in range(cp)),
                                          (b, 1 + s, QPATH_SLICES)))
                    ops[name] = N.OP_QPATH
        if l1_groups > 1:
            for b in range(B):
                for g in range(l1_groups):
                    name = f"merge_l1a[{r},{b},{g}]"
                    tasks.append(TaskSpec(name, r, (WaitEdge(f"l1a[{b},{g}]"),), (NotifyEdge(f"l1[{b}]", r),), (b, g, 0)))
                    ops[name] = N.OP_MERGE_L1A
        for b in range(0 if cand_direct else B):
            name = f"merge_l1[{r},{b}]"
            # one rank: the local top-k is the selection, MERGE_L1 publishes it and no MERGE_L2 runs
            out = (NotifyEdge(f"topk[{b}]", r),) if cp == 1 else tuple(NotifyEdge(f"cand[{b}]", d) for d in range(cp))
            tasks.append(TaskSpec(name, r, (WaitEdge(f"l1[{b}]"),), out, (b, 0, 0)))
            ops[name] = N.OP_MERGE_L1
        for b in range(B if cp > 1 else 0):
            name = f"merge_l2[{r},{b}]"
            tasks.append(TaskSpec(name, r, (WaitEdge(f"cand[{b}]"),), (NotifyEdge(f"topk[{b}]", r),), (b, 0, 0)))
            ops[name] = N.OP_MERGE_L2
        for b in range(B):
            for j in range(n_attn):
                for s in range(attn_splits):
                    name = f"attn[{r},{b},{j},{s}]"
                    waits = (WaitEdge(f"topk[{b}]"),) + ((WaitEdge(f"qm_ready[{b}]"),) if qpath else ())
                    tasks.append(TaskSpec(name, r, waits, (NotifyEdge(f"part[{b}]", b % cp),), (b, j, s)))
                    ops[name] = N.OP_ATTN
        for b in range(B):
            if b % cp == r:
                for hq in range(LSE_GROUPS):  # head groups: the merge of one sequence runs on several blocks
                    name = f"lse_merge[{r},{b},{hq}]"
                    tasks.append(TaskSpec(name, r, (WaitEdge(f"part[{b}]"),), (), (b, hq, LSE_GROUPS)))
                    ops[name] = N.OP_LSE_MERGE
    if compressor:
        events += [EventSpec(f"cmp_stats[{b}]", cross) for b in range(B)]
        for r in range(cp):
            for b in range(B):
                name = f"cmp_step[{r},{b}]"
                tasks.append(TaskSpec(name, r, (), tuple(NotifyEdge(f"cmp_stats[{b}]", d) for d in range(cp)), (b, 0, 0)))
                ops[name] = N.OP_CMP_STEP
            for b in range(B):
                name = f"cmp_fin[{r},{b}]"
                tasks.append(TaskSpec(name, r, (WaitEdge(f"cmp_stats[{b}]"),), (), (b, 0, 0)))
                ops[name] = N.OP_CMP_FIN
    return tasks, events, ops


def q_block_bytes(heads: int = 128, d_qk: int = 576) -> int:
    """One sequence's per-step query block: bf16 indexer q (64 x 128), fp32 gate weights (64), bf16 attention q."""
    return 64 * 128 * 2 + 64 * 4 + heads * d_qk * 2


def arena_regions(B: int, cp: int, top_k: int, heads: int = 128, attn_splits: int = 1, cmp_stats_bytes: int = 0,
                  q_bytes: int = 0, cand_lists: int = 1, thr_chunks: int = 0):
    cand = B * cp * cand_lists * (top_k * 8 + 16)
    inbox = -(-B // cp) * cp * attn_splits * (heads * D_V * 2 + heads * 4)
    regions = {"cand": cand, "inbox": inbox}
    if q_bytes:
        regions["q"] = B * q_bytes
    if cmp_stats_bytes:
        regions["cmp_stats"] = B * cp * cmp_stats_bytes
    if thr_chunks:   # exact row selection: per row, per rank a histogram, per (rank, chunk) a key slot
        regions["thr"] = B * cp * (THR_HIST_BYTES + thr_chunks * THR_SLOT_BYTES)
    return regions


@dataclass
class LayerInputs:
    kv_pages: torch.Tensor      # (num_pages, page_bytes) uint8 index-K cache of this rank
    block_table: torch.Tensor   # (B, max_pages) int32
    seq_lens: torch.Tensor      # (B,) int32 rank-local token counts
    q_idx: torch.Tensor         # (B, 64, 128) bf16 indexer query (replicated on all ranks); with distribute_q the
                                # three query tensors hold the OWNED sequences only (b = rank, rank + cp, ...) or are None
    w_idx: torch.Tensor         # (B, 64) fp32 head-gate weights
    q_mla: torch.Tensor         # (B, 1, H, d_qk) bf16 attention query (replicated)
    kv_mla: torch.Tensor        # (B * kv_seq_stride, 1, d_qk) bf16 local KV rows


class DsaDecodeLayer:
    """Owns the schedule, the symmetric buffers and the scratch of one layer."""

    def __init__(self, B: int, cp: int = 1, rank: int = 0, top_k: int = 2048, heads: int = 128, d_qk: int = 576,
                 fmt: str = "nvfp4", page_tokens: int = 64, max_pages: int = 256, blocks_per_chunk: int = 64,
                 kv_seq_stride: int | None = None, n_ctas: int | None = None, group_name: str = "0",
                 device="cuda", out_dtype=torch.bfloat16, phases: int = 2, softmax_scale: float | None = None,
                 attn_splits: int | None = None, compressor=None, distribute_q: bool = False, kvwrite: bool = False,
                 row_threshold: bool = True, kv_group: int = 1, cand_direct: bool = True, row_exact=None,
                 q_tasks: bool | None = None, dynamic: bool = False, host_query: bool = False):
        """kv_group: consecutive batch entries that share one sequence's KV rows (chunked prefill: the
        query tokens of a tile as batch entries, see prefill.py); 1 = every entry its own sequence.
        distribute_q: the step's query block of sequence b is supplied by its owner rank only (bind()
        then takes the owned sequences' tensors) and a QPATH task stores it into every rank's arena.
        With one rank the kernels read the staging block in place and no QPATH task runs, unless
        q_tasks=True asks for them.
        host_query (with distribute_q): step_from_host() copies the attention query on a second stream while
        the step's indexer phase already runs; the tasks that read it wait for a flag the copy stream writes.
        (Measured at one rank: slower than the plain sequence, 214 against 182 us per step: the query's copy
        takes 23 us, the extra stream operations more.  Off by default.)
        row_exact: the chunk tasks settle the row's exact top-k themselves (default: with one rank;
        across ranks the two exchange rounds cost more than the merge they save: measured).
        compressor: an optional tiles.compress.CompressorState of this rank; the layer-step then also
        runs its step / finalize as tasks (bind_compressor() supplies the per-step tensors)."""
        self.B, self.cp, self.rank, self.K, self.H, self.d_qk = B, cp, rank, top_k, heads, d_qk
        self.fmt, self.P, self.max_pages, self.bpc = fmt, page_tokens, max_pages, blocks_per_chunk
        self.n_chunks = -(-max_pages // blocks_per_chunk)
        self.kv_seq_stride = kv_seq_stride or max_pages * page_tokens
        self.kv_group = kv_group
        self.q_tasks = distribute_q and (cp > 1 if q_tasks is None else bool(q_tasks))
        assert kv_group >= 1 and not (kv_group > 1 and (kvwrite or compressor is not None))
        self.device = torch.device(device)
        self.phases = phases
        self.scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d_qk)
        if n_ctas is None:
            n_ctas = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.n_ctas = n_ctas
        if attn_splits is None:
            # split the local slot range until the attention tasks about fill the blocks; a split
            # should keep a few 64-slot tiles, and the LSE merge takes at most 16 slices
            tiles = -(-(top_k // cp + 128) // 64)
            attn_splits = max(1, min(tiles // 4, n_ctas // max(1, B * 4 * (heads // 128 or 1)), 16 // cp))
        self.attn_splits = attn_splits
        # what the launcher's own check would refuse, refused here with a readable message
        assert heads % 64 == 0 and top_k % 2 == 0, "heads must be a multiple of 64, top_k even"
        assert cp * attn_splits <= 16, f"cp * attn_splits = {cp * attn_splits} exceeds the 16 slices the LSE merge takes"
        assert 0 <= rank < cp
        # row_threshold: the chunk tasks of a sequence agree on a lower bound of the row's k-th score
        # (shared histogram) and emit only what reaches it, so one merge level suffices; otherwise every
        # chunk emits its exact top-k and long rows merge in two levels
        self.row_threshold = row_threshold
        self.l1_groups = 1 if row_threshold else l1_groups_for(self.n_chunks)
        # several ranks, one merge level: the chunk lists go straight to every rank (no exact local top-k
        # in between: the global top-k lies inside the union of what the chunks emit)
        # row_exact = "local" (several ranks): each rank's chunk tasks settle the rank's own exact top-k and
        # store it as the rank's candidate list on every rank (one list per rank, MERGE_L1 only passes on)
        local_exact = row_exact == "local" and cp > 1 and row_threshold and self.l1_groups == 1 and top_k % 4 == 0 \
            and self.n_chunks <= 256
        self.cand_direct = (cand_direct and not local_exact and row_threshold and cp > 1 and self.l1_groups == 1
                            and cp * self.n_chunks <= 256 and top_k % 4 == 0)
        # row_exact: the chunk tasks of a row (on all ranks) settle the exact top-k themselves; the merge
        # task behind them stays in the graph and only acts on rows that fell back (heavy ties)
        if row_exact is None:
            row_exact = cp == 1
        self.row_exact = 2 if local_exact else int(bool(row_exact and row_exact != "local" and row_threshold
                                                        and cp * self.n_chunks <= 256 and top_k % 4 == 0
                                                        and (cp == 1 or self.cand_direct)))
        self.compressor = compressor
        if compressor is not None:
            assert (compressor.B, compressor.cp, compressor.rank) == (B, cp, rank)
        tasks, events, ops = build_layer_dag(B, self.n_chunks, cp, heads, attn_splits, self.l1_groups,
                                             compressor=compressor is not None, qpath=self.q_tasks, kvwrite=kvwrite,
                                             cand_direct=self.cand_direct)
        self.kvwrite = kvwrite
        self.distribute_q = distribute_q
        # dynamic: one shared queue in dependency order, the blocks pull tasks with an atomic counter
        self.dynamic = dynamic
        self.schedule = codegen_schedule(tasks, events, rank=rank, n_ctas=1 if dynamic else n_ctas, world_size=cp, op_of=ops)
        if row_threshold:
            # The LOGITS tasks of a row wait for each other inside the task.  That is free of deadlock as
            # long as, in this rank's dealing order, they come row by row and nothing that depends on a
            # row's candidates is queued ahead of a LOGITS task (the scheduler's FIFO order gives both).
            order = [(self.schedule.op_of[i], tasks[i].coords) for i in self.schedule.topo]
            seen_consumer, last_row, closed = False, None, set()
            for op, coords in order:
                if op == N.OP_LOGITS:
                    if coords[0] != last_row:
                        closed.add(last_row)
                        last_row = coords[0]
                    assert not seen_consumer and coords[0] not in closed, "LOGITS tasks must be queued first, row by row"
                elif op in (N.OP_MERGE_L1, N.OP_MERGE_L1A, N.OP_MERGE_L2, N.OP_ATTN, N.OP_LSE_MERGE):
                    seen_consumer = True
        self.dsched = upload_schedule(self.schedule, self.device, dynamic_ctas=n_ctas if dynamic else None)
        self.n_dag_events = len(events)
        self.events = alloc_event_buffer(len(events) + (2 * B if self.row_exact else 0), rank, cp, group_name, self.device)
        from .tiles.compress import stats_bytes
        cmp_bytes = stats_bytes(compressor.ratio) if compressor is not None else 0
        self.arena = alloc_arena(arena_regions(B, cp, top_k, heads, attn_splits, cmp_bytes,
                                               q_block_bytes(heads, d_qk) if self.q_tasks else 0,
                                               self.n_chunks if self.cand_direct else 1,
                                               self.n_chunks if self.row_exact else 0),
                                 phases, rank, cp, group_name, self.device)
        self.n_owned = len(range(rank, B, cp))
        # distribute_q: the owned sequences' query blocks, one contiguous block [q_idx | w | q_mla] that a
        # caller fills from the host in one copy (views below); sequence b = j * cp + rank is entry j
        self.q_stage = None
        self.host_query = host_query and distribute_q
        if self.host_query:
            self.q_flag = torch.zeros(1, dtype=torch.int64, device=self.device)
            self._h_flags = torch.zeros(8, dtype=torch.int64).pin_memory()
            self._side = torch.cuda.Stream(device=self.device)
            self._prev_done = None
        if distribute_q:
            n = self.n_owned
            nq, nw, nm = n * 64 * 128 * 2, n * 64 * 4, n * heads * d_qk * 2
            self.q_stage = torch.zeros(nq + nw + nm, dtype=torch.uint8, device=self.device)
            self.q_idx_owned = self.q_stage[:nq].view(torch.bfloat16).view(n, 64, 128)
            self.w_idx_owned = self.q_stage[nq:nq + nw].view(torch.float32).view(n, 64)
            self.q_mla_owned = self.q_stage[nq + nw:].view(torch.bfloat16).view(n, 1, heads, d_qk)
        dev = self.device
        C, K = self.n_chunks, top_k
        self.cand_v = torch.empty(B, 1, C, K, device=dev)
        self.cand_i = torch.empty(B, 1, C, K, dtype=torch.int32, device=dev)
        self.cand_c = torch.zeros(B, 1, C, dtype=torch.int32, device=dev)
        G = self.l1_groups
        self.mid_v = torch.empty(B, G, K, device=dev)
        self.mid_i = torch.empty(B, G, K, dtype=torch.int32, device=dev)
        self.mid_c = torch.zeros(B, G, dtype=torch.int32, device=dev)
        self.thr_hist = torch.zeros(2, B, THR_BINS, dtype=torch.int32, device=dev) if row_threshold else None
        self.thr_done = torch.zeros(B, dtype=torch.int32, device=dev) if row_threshold else None
        self.sel_v = torch.zeros(B, K, device=dev)
        self.sel_i = torch.zeros(B, K, dtype=torch.int32, device=dev)
        self.sel_c = torch.zeros(B, dtype=torch.int32, device=dev)
        self.pt_local = torch.zeros(B, K, dtype=torch.int32, device=dev)
        self.k_valid = torch.zeros(B, dtype=torch.int32, device=dev)
        n_owned = -(-B // cp)   # the merged rows of the sequences this rank owns (b % cp == rank), at row b // cp
        self.out = torch.zeros(n_owned, heads, D_V, dtype=out_dtype, device=dev)
        self.out_lse = torch.zeros(n_owned, heads, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)
        self.phase = 0
        self._params = None
        self._inputs = None

    def bind(self, x: LayerInputs) -> None:
        """Fixes the input tensors (their addresses are baked into the launch parameters)."""
        B, K = self.B, self.K
        if self.distribute_q:
            # q comes through the arena: x.q_idx / x.w_idx / x.q_mla, when given, are the OWNED sequences'
            # tensors and are copied into the staging block once here (refresh q_stage before later steps)
            if x.q_idx is not None:
                self.q_idx_owned.copy_(x.q_idx)
                self.w_idx_owned.copy_(x.w_idx)
                self.q_mla_owned.copy_(x.q_mla)
            if self.q_tasks:
                qbase = self.arena.tensor.data_ptr() + self.arena.regions["q"]
                q_ptr, w_ptr, qm_ptr = qbase, qbase + B * 64 * 128 * 2, qbase + B * (64 * 128 * 2 + 64 * 4)
            else:   # one rank: every sequence is owned, the kernels read the staging block in place
                q_ptr, w_ptr, qm_ptr = N.ptr(self.q_idx_owned), N.ptr(self.w_idx_owned), N.ptr(self.q_mla_owned)
        else:
            assert x.q_idx.dtype == torch.bfloat16 and x.q_mla.dtype == torch.bfloat16
            q_ptr, w_ptr, qm_ptr = N.ptr(x.q_idx), N.ptr(x.w_idx), N.ptr(x.q_mla)
        lp = N.LogitsParams(
            kv_pages=N.ptr(x.kv_pages), num_pages=x.kv_pages.shape[0], page_tokens=self.P,
            fmt=N.FMT_MXFP4 if self.fmt == "mxfp4" else N.FMT_NVFP4, q_fmt=N.Q_BF16,
            q=q_ptr, q_sf=None, weights=w_ptr, block_table=N.ptr(x.block_table),
            max_pages=self.max_pages, seq_lens=N.ptr(x.seq_lens), logits=None, logits_stride=0,
            cand_v=N.ptr(self.cand_v), cand_i=N.ptr(self.cand_i), cand_c=N.ptr(self.cand_c), top_k=K,
            B=B, q_len=1, heads=64, blocks_per_chunk=self.bpc, n_chunks=self.n_chunks, window_exclude=0,
            id_mul=self.cp, id_add=self.rank, status=N.ptr(self.status))
        mp = N.SparseMlaParams(
            q=qm_ptr, kv_win=None, kv_cmp=N.ptr(x.kv_mla), pt_win=None, pt_cmp=N.ptr(self.pt_local),
            k_valid=N.ptr(self.k_valid), win_valid=None, attn_sink=None, o=N.ptr(self.out), lse=N.ptr(self.out_lse),
            o_stride=self.H * D_V, lse_stride=self.H, ws_o=None, ws_lse=None,
            B=B, q_len=1, H=self.H, d_qk=self.d_qk, d_v=D_V, pages_win=0, pages_cmp=x.kv_mla.shape[0], page_cmp=1,
            pt_cols=K, kv_dtype=N.DT_BF16, out_dtype=N.DT_BF16, n_splits=1, fp8_p=0,
            softmax_scale=self.scale, output_scale=1.0, status=N.ptr(self.status))
        L = N.LayerParams()
        L.cp, L.rank, L.B, L.top_k, L.H, L.n_chunks = self.cp, self.rank, B, K, self.H, self.n_chunks
        L.kv_seq_stride = self.kv_seq_stride
        L.kv_group = self.kv_group
        L.cand_direct = int(self.cand_direct)
        if self.row_exact:
            L.thr_exact, L.thr_ev_base, L.thr_off = self.row_exact, self.n_dag_events, self.arena.regions["thr"]
        L.attn_splits = self.attn_splits
        L.l1_groups = self.l1_groups
        L.mid_v, L.mid_i, L.mid_c = N.ptr(self.mid_v), N.ptr(self.mid_i), N.ptr(self.mid_c)
        L.logits, L.mla = lp, mp
        L.cand_off, L.inbox_off = self.arena.regions["cand"], self.arena.regions["inbox"]
        L.phase_bytes, L.phases = self.arena.nbytes_per_phase, self.phases
        L.sel_v, L.sel_i, L.sel_c = N.ptr(self.sel_v), N.ptr(self.sel_i), N.ptr(self.sel_c)
        L.out, L.out_lse = N.ptr(self.out), N.ptr(self.out_lse)
        L.out_dtype = N.DT_F32 if self.out.dtype == torch.float32 else N.DT_BF16
        if self.q_tasks:
            L.q_stage, L.q_off = N.ptr(self.q_stage), self.arena.regions["q"]
        L.thr_hist, L.thr_done = N.ptr(self.thr_hist), N.ptr(self.thr_done)
        self._params, self._inputs = L, x
        if self.host_query:   # step_from_host() launches with a copy of the parameters that carries the flag
            self._params_hq = N.LayerParams.from_buffer_copy(L)
            self._params_hq.q_host_flag = N.ptr(self.q_flag)

    def bind_compressor(self, seq_len, new_attn, new_idx, ape_attn, ape_idx, norm_w_attn, norm_w_idx, norm_eps: float,
                        freqs, fp8_scale: float = 1.0) -> None:
        """Fixes the compressor's per-step tensors (the caller refreshes their contents before each
        step): seq_len (B,) int32 GLOBAL lengths before the step, the new records of this rank, the slot
        biases, norm weights and rope table.  Call after bind()."""
        from .tiles.compress import fill_finalize_params
        assert self._params is not None and self.compressor is not None and not self.host_query
        st = self.compressor
        c = N.CompressParams()
        c.B, c.cp, c.rank, c.q_len, c.ratio = st.B, st.cp, st.rank, st.q_len, st.ratio
        c.seq_len = N.ptr(seq_len)
        c.ring_attn, c.ring_idx, c.state = N.ptr(st.ring_attn), N.ptr(st.ring_idx), N.ptr(st.state)
        c.new_attn, c.new_idx, c.ape_attn, c.ape_idx = N.ptr(new_attn), N.ptr(new_idx), N.ptr(ape_attn), N.ptr(ape_idx)
        c.stats_off, c.do_push = self.arena.regions["cmp_stats"], 1
        fill_finalize_params(c, st, norm_w_attn, norm_w_idx, norm_eps, freqs, fp8_scale)
        self._params.cmp = c
        self._cmp_keep = (seq_len, new_attn, new_idx, ape_attn, ape_idx, norm_w_attn, norm_w_idx, freqs)

    def bind_kvwrite(self, k_idx_new, kv_new, global_len, advance: bool = True) -> None:
        """Fixes the new-token inputs of the KVWRITE tasks (layer built with kvwrite=True; call after
        bind()): k_idx_new (B, 128) fp32 and kv_new (B, d_qk) bf16, replicated on every rank and refreshed
        by the caller before each step; global_len (B,) int32 = sequence lengths before the step.  With
        `advance` the kernel adds 1 to global_len itself.  The bound block table must already hold a page
        for the new slot; seq_lens and the caches are written by the step."""
        assert self._params is not None and self.kvwrite and not self.host_query
        assert k_idx_new.dtype == torch.float32 and global_len.dtype == torch.int32
        L = self._params
        L.kvw_k_idx, L.kvw_kv, L.kvw_glen, L.kvw_advance = N.ptr(k_idx_new), N.ptr(kv_new), N.ptr(global_len), int(advance)
        self._kvw_keep = (k_idx_new, kv_new, global_len)

    def step(self, wait_budget_ns: int = 2_000_000_000, stream=None, trace=None, _params=None) -> None:
        """Launches one layer-step (asynchronous): exactly one kernel launch, nothing else.  The
        phase lives on the device and the kernel advances it, so a step can be captured in a CUDA
        graph and replayed.  Every rank must run the same number of steps."""
        assert self._params is not None, "bind() inputs first"
        launch_megakernel(self.dsched, self.events, self.arena, self.status, layer=_params or self._params,
                          wait_budget_ns=wait_budget_ns, stream=stream, trace=trace, device_phase=True)
        self.phase += 1   # host mirror, for reporting only

    def step_from_host(self, hblock: torch.Tensor, h_out: torch.Tensor | None = None, wait_budget_ns: int = 2_000_000_000) -> None:
        """One step whose query block comes from pinned host memory (`hblock`: uint8, the layout of
        q_stage: [q_idx | w | q_mla] of the owned sequences) and whose owned output rows go back to pinned
        host memory (`h_out`, optional), all asynchronous on the current stream (synchronize it to read
        h_out).  Built with host_query=True, the indexer part is copied on the current stream ahead of the
        launch and the attention query, nine tenths of the block, on a second stream while the indexer
        phase runs; a flag copied behind it releases the tasks that read it."""
        assert self.q_stage is not None and hblock.numel() == self.q_stage.numel()
        main = torch.cuda.current_stream(self.device)
        if not self.host_query:
            self.q_stage.copy_(hblock, non_blocking=True)
            self.step(wait_budget_ns=wait_budget_ns)
        else:
            n_idx = self.n_owned * (64 * 128 * 2 + 64 * 4)
            self.q_stage[:n_idx].copy_(hblock[:n_idx], non_blocking=True)
            slot = self.phase % self._h_flags.numel()
            self._h_flags[slot] = self.phase + 1        # (read by the copy below; eight steps may be in flight)
            if self._prev_done is not None:
                self._side.wait_event(self._prev_done)  # the previous step has finished reading its query
            with torch.cuda.stream(self._side):
                self.q_stage[n_idx:].copy_(hblock[n_idx:], non_blocking=True)
                self.q_flag.copy_(self._h_flags[slot:slot + 1], non_blocking=True)
            self.step(wait_budget_ns=wait_budget_ns, _params=self._params_hq)
            self._prev_done = torch.cuda.Event()
            self._prev_done.record(main)
        if h_out is not None:
            h_out.copy_(self.out, non_blocking=True)

    def capture_host_step(self, hblock: torch.Tensor, h_out: torch.Tensor | None = None):
        """The plain step_from_host() sequence (query block in, one launch, owned rows out) captured once as a
        CUDA graph over the given pinned buffers: graph.replay() then costs one host call per step instead of
        three.  The caller refreshes `hblock` before a replay and synchronizes before reading `h_out`."""
        assert self.q_stage is not None and self._params is not None
        stream = torch.cuda.Stream(device=self.device)
        stream.wait_stream(torch.cuda.current_stream(self.device))
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            with torch.cuda.graph(graph, stream=stream):
                self.q_stage.copy_(hblock, non_blocking=True)
                self.step(stream=stream)
                if h_out is not None:
                    h_out.copy_(self.out, non_blocking=True)
        self.phase -= 1   # (the capture itself ran nothing)
        return graph

    def owned_rows(self):
        """Sequences whose merged output this rank holds; sequence b is row b // cp of `out`."""
        return [b for b in range(self.B) if b % self.cp == self.rank]

    def check_status(self) -> None:
        st = self.status.tolist()
        if st[0] != 0:
            raise N.MdcError(f"device failure: code {st[0]} block {st[1]} detail {st[2:4]} seen/wanted {st[4:]}")
