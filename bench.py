"""Benchmark of the DSA decode hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Every N times the same workload family: one full DSA decode layer-step at
128K context (indexer logits over the paged NVFP4 index cache, exact top-k
2048, sparse MLA over the selection, LSE merge) as ONE persistent-kernel
launch per rank, 8 sequences per rank, the context sharded token-interleaved
over the N ranks (weak scaling; N = 8 is BASELINE config 4: B = 64, 16384
tokens per rank per sequence).  One step = one layer-call of the operator;
the metric is decode tokens per second (B * q_len / step time).  Prints ONE
JSON line (rank 0).

Timing: CUDA events on the launching stream around exactly K steps after W
warm-up steps, barrier + synchronize on both sides, max over ranks.  Each rank
rotates over two independent copies of its caches (index cache 75.5 MB and
KV pool 1.2 GB per copy), so every step streams from HBM, not from L2.

At N = 1 the line also carries the roofline of the dominant kernel family
measured alone: the indexer (BASELINE config 2: B = 32, context 32768,
logits + exact top-k 2048 in one launch) and the tcgen05 sparse-MLA tile.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

METRIC = "dsa_decode_tokens_per_s"
UNIT = "tokens/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._t = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                    capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._t.join(timeout=6)

    def summary(self):
        mhz, mx, reasons = [], 0, set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                mhz.append(float(s[0]))
                mx = max(mx, float(s[1]))
                for n, v in zip(names, s[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                continue
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


class Ranks:
    """The process group of the run, or a stand-in at N = 1 (no rendezvous needed)."""

    def __init__(self):
        import torch

        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", self.rank))
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.dist = None
        self.group_name = "0"
        if self.world > 1:
            import torch.distributed as dist

            dist.init_process_group("nccl", device_id=self.dev)
            self.dist = dist
            self.group_name = dist.group.WORLD.group_name

    def barrier(self):
        if self.dist is not None:
            self.dist.barrier()

    def reduce_max(self, values):
        import torch

        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    def reduce_min(self, values):
        import torch

        t = torch.tensor(values, device=self.dev, dtype=torch.float64)
        if self.dist is not None:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MIN)
        return t.tolist()

    def sum_(self, t):
        if self.dist is not None:
            self.dist.all_reduce(t)
        return t

    def gather(self, t):
        import torch

        if self.dist is None:
            return [t]
        out = [torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(out, t.contiguous())
        return out

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()


# ----------------------------------------------------------------------------
# the workload: one decode layer-step at 128K context, context parallel over N ranks
# ----------------------------------------------------------------------------
def cp_config(n):
    """128K-token context sharded over n ranks, 8 sequences per rank (BASELINE
    config 4 at n = 8: B = 64, 16384 tokens per rank per sequence)."""
    return dict(B=8 * n, S=131072, page=64, top_k=2048, H=128, d_qk=576, cp=n, copies=2, blocks_per_chunk=128)


def layer_algorithmic_bytes(c, attn_splits):
    """Bytes one rank's layer-step must move, per phase (the per-unit figures: 72 B per (sequence,
    token) of NVFP4 index-K + 4 B per page + 16640 B of query per sequence; 8 B per candidate read or
    written; 1152 B per selected KV row + 147456 B of query per sequence; 131584 B per partial)."""
    B, cp, K, P = c["B"], c["cp"], c["top_k"], c["page"]
    S_loc = c["S"] // cp
    pages = S_loc // P
    n_chunks = -(-pages // c["blocks_per_chunk"])
    part = 128 * 512 * 2 + 128 * 4
    owned = -(-B // cp)
    phases = {
        # the chunk tasks of a row emit about top-k candidates between them (row threshold); at cp > 1 they
        # store them into every rank's arena themselves and no local merge runs
        "LOGITS": B * S_loc * 72 + B * pages * 4 + B * 16640 + B * K * 8 * cp,
        "MERGE_L1": B * K * 8 + B * K * 12,
        "MERGE_L2": B * cp * K * 8 + B * K * 12,
        "ATTN": B * (K // cp) * 1152 + B * 128 * 576 * 2 + B * attn_splits * part,
        "LSE_MERGE": owned * (cp * attn_splits * part + part),
    }
    phases.pop("MERGE_L1" if cp > 1 else "MERGE_L2")
    return phases


OP_NAMES = {1: "LOGITS", 2: "MERGE_L1", 3: "MERGE_L2", 4: "ATTN", 5: "LSE_MERGE", 6: "MERGE_L1A",
            7: "CMP_STEP", 8: "CMP_FIN", 9: "QPATH", 10: "KVWRITE"}


def task_timeline(layer, dev):
    """One traced layer-step: per op the task count, mean wait / body time and the time its last task
    ended (us from the first task's start), from the megakernel's optional trace buffer; plus the
    LSE-merge latency per owned sequence: from the moment the first merge task of the sequence saw
    all partials present to the moment its last head group was written."""
    import torch

    trace = torch.zeros(4 + 4 * 8192, dtype=torch.int64, device=dev)
    layer.step(trace=trace)
    torch.cuda.synchronize()
    t = trace.cpu()
    n = min(int(t[0]), 8192)
    e = t[4:4 + 4 * n].reshape(n, 4)
    if n == 0:
        return {}, None
    t0 = int(e[:, 1].min())
    ops = (e[:, 0] >> 24) & 0xff
    out = {}
    for op in sorted(set(ops.tolist())):
        m = ops == op
        a, b, c = e[m, 1].double(), e[m, 2].double(), e[m, 3].double()
        out[OP_NAMES.get(op, str(op))] = {"tasks": int(m.sum()), "wait_us": round(float((b - a).mean()) / 1e3, 1),
                                          "body_us": round(float((c - b).mean()) / 1e3, 1),
                                          "first_start_us": round(float(b.min() - t0) / 1e3, 1),
                                          "last_end_us": round(float(c.max() - t0) / 1e3, 1)}
    lat = None
    m = ops == 5
    if bool(m.any()):
        seq = (e[m, 0] >> 12) & 0xfff
        lats = []
        for b in sorted(set(seq.tolist())):
            mb = seq == b
            lats.append(float(e[m][mb, 3].max() - e[m][mb, 2].min()) / 1e3)
        lat = {"mean_us": round(sum(lats) / len(lats), 2), "max_us": round(max(lats), 2), "sequences": len(lats),
               "definition": "first merge task of a sequence sees all partials arrived -> last head group written"}
    return out, lat


def build_rank(R, c, seed0=1000):
    """This rank's caches (c['copies'] rotation copies), the replicated per-step query block and
    one DsaDecodeLayer per copy."""
    import torch
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from mega_dsa_cp_b200.tiles.fp4 import fuse_pages

    dev, world, rank = R.dev, R.world, R.rank
    B, P, K, H, DQK = c["B"], c["page"], c["top_k"], c["H"], c["d_qk"]
    S_loc = c["S"] // world
    pages = S_loc // P
    g = torch.Generator(device=dev).manual_seed(seed0 + rank)
    gq = torch.Generator(device=dev).manual_seed(7)      # replicated tensors: same seed on every rank
    # the per-step query tensors (same values on every rank: the oracle check needs them); a rank feeds the
    # layer only the sequences it owns, the QPATH task of the step distributes them over NVLink
    q_idx = torch.randn(B, 64, 128, generator=gq, device=dev).to(torch.bfloat16)
    w_idx = (torch.randn(B, 64, generator=gq, device=dev) / 64.0).contiguous()
    q_mla = (torch.randn(B, 1, H, DQK, generator=gq, device=dev) * 0.5).to(torch.bfloat16)
    seq_loc = torch.full((B,), S_loc, dtype=torch.int32, device=dev)
    layers, inputs = [], []
    for _ in range(c["copies"]):   # rotate over cache copies so every step streams from HBM
        parts = [fuse_pages(torch.randn(B * S_loc // 8, 128, generator=g, device=dev), "nvfp4", P)[0] for _ in range(8)]
        cache = torch.cat(parts)
        del parts
        bt = torch.randperm(B * pages, generator=g, device=dev).to(torch.int32).reshape(B, pages).contiguous()
        kv = (torch.randn(B * S_loc, 1, DQK, generator=g, device=dev) * 0.5).to(torch.bfloat16)
        layer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, heads=H, d_qk=DQK, max_pages=pages,
                               blocks_per_chunk=c["blocks_per_chunk"], kv_seq_stride=S_loc,
                               group_name=R.group_name, device=dev, distribute_q=True, row_exact=c.get("row_exact"),
                               cand_direct=c.get("cand_direct", True), dynamic=c.get("dynamic", False))
        layer.bind(LayerInputs(cache, bt, seq_loc, q_idx[rank::world], w_idx[rank::world], q_mla[rank::world], kv))
        layers.append(layer)
        inputs.append((cache, bt, kv))
    return layers, inputs, (q_idx, w_idx, q_mla)


def parity_block(R, c, layer, inp, q):
    """Outside the timed region: one owned sequence per rank against the CPU oracle at full size.
    The sequence's index-K shards and the KV rows of the ids the kernel selected are collected from
    all ranks; the owner recomputes the logits (dequantised FP4, fp32), the exact hierarchical
    top-k and the cp-way attention + LSE merge over the kernel's own selection.  Returns the worst
    figures over all ranks."""
    import torch
    from oracle import dsa_oracle as orc

    world, rank, dev = R.world, R.rank, R.dev
    cache, bt, kv = inp
    q_idx, w_idx, q_mla = q
    B, K, P, S, DQK = c["B"], c["top_k"], c["page"], c["S"], c["d_qk"]
    S_loc = S // world
    d_o = d_l = 0.0
    overlap, count_ok, same_sel = 1.0, 1.0, 1.0
    for b in range(min(world, B)):          # sequence b is owned by rank b % world == b
        shards = R.gather(cache[bt[b].long()])                       # [world] x (pages, page bytes)
        n = int(layer.sel_c[b])
        sel = layer.sel_i[b, :n].clone()
        ref_sel = sel.clone()
        if R.dist is not None:
            R.dist.broadcast(ref_sel, 0)
        same_sel = min(same_sel, 1.0 if torch.equal(ref_sel, sel) else 0.0)
        rows = torch.zeros(K, DQK, dtype=torch.float32, device=dev)
        mine = (sel % world) == rank
        rows[:n][mine] = kv[(b * S_loc + sel[mine] // world).long(), 0].float()
        R.sum_(rows)                                                  # every id is held by exactly one rank
        if rank != b % world:
            continue
        kd = torch.empty(S, 128)
        for r, sh in enumerate(shards):
            data, sf = orc.split_index_pages(sh.cpu(), "nvfp4", P)
            kd[r::world] = orc.dequant_fp4(data, sf, "nvfp4").reshape(S_loc, 128)
        qi, wi = q_idx[b].float().cpu(), w_idx[b].cpu()
        want = orc.select_topk_ref(qi, wi, kd, S, K, cp=world)
        got = sel.cpu()
        overlap = min(overlap, len(set(got.tolist()) & set(want.tolist())) / max(1, want.numel()))
        count_ok = min(count_ok, 1.0 if n == want.numel() else 0.0)
        # attention over the kernel's own selection: row j of `rows` is the KV row of sel[j]
        o, l = orc.attend_selected_ref(q_mla[b, 0].float().cpu(), rows[:n].cpu(), got, 1.0 / math.sqrt(DQK),
                                       cp=world, rows_are_selected=True)
        d_o = max(d_o, float((layer.out[b // world].float().cpu() - o).abs().max()))
        d_l = max(d_l, float((layer.out_lse[b // world].cpu() - l).abs().max()))
    worst = R.reduce_max([d_o, d_l])
    best = R.reduce_min([overlap, count_ok, same_sel])
    ok = worst[0] < 2e-2 and worst[1] < 1e-3 and best[0] >= 0.999 and best[1] == 1.0 and best[2] == 1.0
    return {"checked_rows": min(world, B), "max_abs_o": worst[0], "max_abs_lse": worst[1], "sel_overlap": best[0],
            "sel_count_exact": bool(best[1] == 1.0), "sel_identical_on_all_ranks": bool(best[2] == 1.0),
            "tolerance": "o 2e-2 abs (bf16), log2-LSE 1e-3, selection overlap >= 0.999 vs oracle logits",
            "ok": bool(ok)}


def prefill_sample(R, c, inp, tiles=4):
    """BASELINE config 5's shape on a bounded sample (chunked prefill: B = 2 sequences x 4096 query
    tokens at 128 K context): `tiles` tiles of 8 x world query tokens at the end of sequence 0's context,
    each tile one layer-step in which every query token is a batch entry with its own causal length
    (mega_dsa_cp_b200/prefill.py).  Every rank takes part; returns query tokens/s (max time over ranks)."""
    import torch
    from mega_dsa_cp_b200.prefill import DsaPrefillChunk

    world, rank, dev = R.world, R.rank, R.dev
    cache, bt, kv = inp
    S, P, K, H, DQK = c["S"], c["page"], c["top_k"], c["H"], c["d_qk"]
    S_loc = S // world
    tile = 8 * world
    Tq = tiles * tile
    pf = DsaPrefillChunk(tile, cp=world, rank=rank, top_k=K, heads=H, d_qk=DQK, max_pages=S_loc // P,
                         blocks_per_chunk=c["blocks_per_chunk"], group_name=R.group_name, device=dev)
    pf.bind(cache, bt[0], kv[:S_loc])
    gq = torch.Generator(device=dev).manual_seed(11)
    q_idx = torch.randn(Tq, 64, 128, generator=gq, device=dev).to(torch.bfloat16)
    w_idx = (torch.randn(Tq, 64, generator=gq, device=dev) / 64.0).contiguous()
    q_mla = (torch.randn(Tq, 1, H, DQK, generator=gq, device=dev) * 0.5).to(torch.bfloat16)
    pos = torch.arange(S - Tq, S)
    out = torch.zeros(Tq // world, H, 512, dtype=torch.bfloat16, device=dev)
    sel_c = torch.zeros(Tq, dtype=torch.int32, device=dev)
    pf.run(q_idx, w_idx, q_mla, pos, out, sel_c=sel_c)          # warm-up
    torch.cuda.synchronize()
    pf.check_status()
    R.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    pf.run(q_idx, w_idx, q_mla, pos, out, sel_c=sel_c)
    ev1.record()
    torch.cuda.synchronize()
    pf.check_status()
    R.barrier()
    ms = R.reduce_max([ev0.elapsed_time(ev1)])[0]
    full = bool((sel_c == K).all()) and bool(torch.isfinite(out.float()).all())
    return {"workload": f"chunked prefill sample: {Tq} query tokens of one sequence at context {S}, tiles of {tile} "
                        f"query tokens as batch entries of the decode layer-step (causal lengths), cp{world}",
            "query_tokens_per_s": Tq / (ms * 1e-3), "us_per_tile": ms * 1e3 / tiles, "tiles": tiles,
            "kernel_launches": tiles, "selected_full_and_finite": full,
            "note": "the index cache is re-streamed per query token (from L2 within a tile); parity of this path: "
                    "tests/test_gpu_prefill.py, tests/mp_prefill_worker.py"}


def nccl_baseline(R, c, attn_splits, reps=20):
    """NCCL collectives of the same payloads as the two exchange steps, timed beside the P2P path
    (the measured baseline only; the product path never calls them): all-gather of every sequence's
    candidate list, and the all-to-all of the bf16 partials + LSEs to their owners."""
    import torch

    if R.dist is None:
        return None
    B, K, cp = c["B"], c["top_k"], R.world
    cand = torch.zeros(B * (K * 8 + 16), dtype=torch.uint8, device=R.dev)
    cand_all = torch.zeros(cp * cand.numel(), dtype=torch.uint8, device=R.dev)
    part = (B // cp) * attn_splits * (128 * 512 * 2 + 128 * 4)
    send = torch.zeros(cp * part, dtype=torch.uint8, device=R.dev)
    recv = torch.zeros_like(send)
    out = {}
    for name, fn in (("all_gather_candidates_us", lambda: R.dist.all_gather_into_tensor(cand_all, cand)),
                     ("all_to_all_partials_us", lambda: R.dist.all_to_all_single(recv, send))):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        R.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        out[name] = round(R.reduce_max([e0.elapsed_time(e1) / reps * 1e3])[0], 1)
    out["bytes_per_rank"] = {"candidates": cand.numel(), "partials": send.numel()}
    return out


def run_layer(args):
    import torch

    R = Ranks()
    world, rank, dev = R.world, R.rank, R.dev
    c = cp_config(world)
    c["row_exact"] = {"default": None, "local": "local", "global": True, "off": False, "l1": False}[args.row_exact]
    c["dynamic"] = args.dynamic
    c["cand_direct"] = args.row_exact != "l1"   # l1: every rank merges its chunk lists exactly before the exchange
    B, H, DQK = c["B"], c["H"], c["d_qk"]
    layers, inputs, q = build_rank(R, c)
    R.barrier()
    torch.cuda.synchronize()

    def step(i):
        layers[i % len(layers)].step()

    for i in range(args.warmup * len(layers)):
        step(i)
    torch.cuda.synchronize()
    R.barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(R.local) as clk:
        time.sleep(0.1)
        R.barrier()
        torch.cuda.synchronize()
        ev0.record()
        for i in range(args.steps):
            step(i)
        ev1.record()
        torch.cuda.synchronize()
        R.barrier()
        ms = ev0.elapsed_time(ev1)
        time.sleep(0.1)
    for l in layers:
        l.check_status()
    R.barrier()
    timeline, lse_lat = task_timeline(layers[0], dev)   # every rank steps (the ranks wait on each other); rank 0 reports
    layers[0].check_status()
    R.barrier()
    parity = parity_block(R, c, layers[0], inputs[0], q)

    # end to end through DsaDecodeLayer: the step's query block comes from pinned host memory, the
    # owned output rows go back to pinned host memory, both inside the timed region
    hblock = layers[0].q_stage.cpu().pin_memory()     # [q_idx | w | q_mla] of the sequences this rank owns
    owned = layers[0].owned_rows()
    h_out = torch.empty(len(owned), H, 512, dtype=torch.bfloat16).pin_memory()

    # one rank: the sequence is captured once per cache copy as a CUDA graph (199 against 206 us per step on one
    # box); with several ranks it is issued call by call (a capture next to the process group's watchdog thread
    # was not tried)
    graphs = [l.capture_host_step(hblock, h_out) for l in layers] if world == 1 else None

    def e2e_step(i):
        # one copy of the query block in, one launch, one contiguous copy of the owned rows back.  (Copying the
        # attention query on a second stream behind the launch, host_query=True, was measured on the same
        # box: 214 us against 182 us per step; the extra stream operations cost more than the 23 us the copy takes.)
        if graphs is not None:
            graphs[i % len(graphs)].replay()
            torch.cuda.synchronize()
        else:
            layers[i % len(layers)].step_from_host(hblock, h_out)
            torch.cuda.current_stream().synchronize()

    for i in range(args.warmup):
        e2e_step(i)
    R.barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        e2e_step(i)
    torch.cuda.synchronize()
    R.barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    last = layers[(args.steps - 1) % len(layers)]
    e2e_same = bool(torch.equal(h_out.to(dev), last.out))   # the rows that came back are the step's output
    for l in layers:
        l.check_status()
    ms_step, e2e_step_ms = [x / args.steps for x in R.reduce_max([ms, e2e_ms])]
    nccl = nccl_baseline(R, c, layers[0].attn_splits)
    prefill = prefill_sample(R, c, inputs[0])
    # notify -> wait one-way latency of the event layer (ping-pong, round trip / 2): block to block on this GPU,
    # and rank 0 <-> rank 1 over NVLink; the reference publishes 1.1 us / 2.85 us on B200 (docs/event-system.md:5)
    from mega_dsa_cp_b200.events.latency import cross_gpu_notify_latency, local_notify_latency
    latency = {"published_reference_ns": {"local": 1100, "cross_gpu": 2850}}
    if R.dist is not None:
        cross = cross_gpu_notify_latency(rank, world, R.group_name, dev)
        if rank == 0:
            latency["cross_gpu"] = cross
    if rank == 0:
        latency["local"] = local_notify_latency(dev)
    for l in layers:
        l.check_status()

    line = None
    if rank == 0:
        peaks = measured_peaks()
        phases = layer_algorithmic_bytes(c, layers[0].attn_splits)
        algo = sum(phases.values())
        gbs = algo / (ms_step * 1e-3) / 1e9
        per_phase = {}
        for name, nbytes in phases.items():
            t = timeline.get(name)
            if t:
                span = max(1e-3, t["last_end_us"] - t["first_start_us"])
                per_phase[name] = {"algorithmic_bytes": nbytes, "span_us": round(span, 1),
                                   "gb_per_s": round(nbytes / span / 1e3, 1),
                                   "frac_of_hbm": round(nbytes / span / 1e3 / peaks["hbm_gbs"], 4)}
        line = {
            "metric": METRIC, "value": B / (ms_step * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp4(e2m1 x ue4m3) x bf16 -> f32 indexer; bf16 MLA, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": f"full DSA decode layer-step, CP={world}: B={B}, ctx 131072 sharded token-interleaved "
                                   f"({c['S'] // world} tokens/rank/seq), indexer + top-k 2048 + sparse MLA (128 heads, "
                                   "512+64) + LSE merge, one persistent kernel per rank" +
                                   (", P2P stores into symmetric memory (query blocks, candidates, partials)" if world > 1 else ""),
                       "l2": f"rotating {c['copies']} cache copies per rank (index cache + KV pool 1.3 GB each > 126 MB L2)",
                       "parallelism": f"cp{world}", "attn_splits": layers[0].attn_splits},
            "step_us": ms_step * 1e3,
            "e2e": {"value": B / (e2e_step_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": hblock.numel(),
                    "d2h_bytes_per_step": h_out.numel() * 2, "ms_per_step": e2e_step_ms, "output_read_back_intact": e2e_same,
                    "api": ("DsaDecodeLayer.capture_host_step() + graph.replay()" if world == 1 else "DsaDecodeLayer.step_from_host()") + ": each rank sends the query block of the sequences it owns from pinned host "
                           "memory (" + ("the step's QPATH tasks spread it over NVLink" if world > 1 else
                                         "one rank: the kernels read the staging block in place") +
                           ") and reads its owned output rows back"},
            "gpu_launches": args.steps, "kernels_per_step": 1,
            "parity": parity,
            "timeline_rank0": timeline, "lse_merge_latency": lse_lat,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "peak_kind": f"of {peaks['kind']}",
                         "kernel": "mega_kernel (the whole layer-step: a chain of dependent phases)",
                         "algorithmic_bytes": algo, "traffic": None, "phases": per_phase},
            "nccl_baseline": nccl, "notify_latency": latency, "prefill_chunk": prefill,
            "clocks": clk.summary(),
        }
    return R, line, layers, inputs


# ----------------------------------------------------------------------------
# kernels measured alone (N = 1): the source of the roofline blocks
# ----------------------------------------------------------------------------
CFG2 = dict(B=32, S=32768, page=64, top_k=2048, q_len=1, copies=4, blocks_per_chunk=128)

# dram__bytes_read.sum + dram__bytes_write.sum of one row-mode indexer launch at BASELINE config 2,
# from the ncu capture summarised in profiles/logits_row_kernel_cfg2.md
NCU_TRAFFIC_BYTES = 77_485_056   # 76,164,096 read + 1,320,960 written


def cfg2_algorithmic_bytes(c) -> int:
    """Bytes one row-mode indexer launch must move: 72 B per (sequence, token) of NVFP4 index-K,
    4 B per page-table entry, 16640 B of bf16 query + weights per sequence, 8 B per emitted entry."""
    B, S, P, K = c["B"], c["S"], c["page"], c["top_k"]
    return B * S * 72 + B * (S // P) * 4 + B * 16640 + B * K * 8


def indexer_alone(args, dev):
    """BASELINE config 2 (indexer logits + exact top-k 2048, B = 32, context 32768, one row-mode
    launch) over 4 rotating cache copies (302 MB > L2): kernel time by CUDA events, end to end
    through the public runner with the per-step tensors sent from pinned host memory."""
    import torch
    from mega_dsa_cp_b200.tiles.fp4 import fuse_pages
    from mega_dsa_cp_b200.tiles.logits import run_fp4_paged_mqa_logits

    c = CFG2
    B, S, P, K, T, bpc = c["B"], c["S"], c["page"], c["top_k"], c["q_len"], c["blocks_per_chunk"]
    g = torch.Generator(device=dev).manual_seed(0)
    pages_per_seq = S // P
    pool = B * pages_per_seq
    caches, tables = [], []
    for _ in range(c["copies"]):
        parts = [fuse_pages(torch.randn(pool // 8 * P, 128, generator=g, device=dev), "nvfp4", P)[0] for _ in range(8)]
        caches.append(torch.cat(parts))
        del parts
        tables.append(torch.randperm(pool, generator=g, device=dev).to(torch.int32).reshape(B, pages_per_seq).contiguous())
    q = torch.randn(B, 64 * T, 128, generator=g, device=dev).to(torch.bfloat16)
    w = (torch.randn(B, 64 * T, generator=g, device=dev) / 64.0).contiguous()
    ov = torch.empty(B, T, K, device=dev)
    oi = torch.empty(B, T, K, dtype=torch.int32, device=dev)
    oc = torch.empty(B, T, dtype=torch.int32, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)

    def launch(i):
        r = i % c["copies"]
        run_fp4_paged_mqa_logits(caches[r], q, None, w, tables[r], None, bpc, top_k=K, fmt="nvfp4",
                                 page_tokens=P, status=status, row_topk=(ov, oi, oc))

    reps = max(args.steps, 20)
    for i in range(max(args.warmup, c["copies"])):
        launch(i)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for i in range(reps):
        launch(i)
    k1.record()
    torch.cuda.synchronize()
    ms = k0.elapsed_time(k1) / reps
    assert status[0].item() == 0 and int(oc.min()) == K, f"device failure {status.tolist()}"
    # the same pipeline without the selection (logits written out, 4.2 MB more): what the select adds
    logits = torch.empty(B * T, S, device=dev)
    plain = lambda i: run_fp4_paged_mqa_logits(caches[i % c["copies"]], q, None, w, tables[i % c["copies"]], logits, bpc,
                                               fmt="nvfp4", page_tokens=P, status=status)
    for i in range(c["copies"]):
        plain(i)
    torch.cuda.synchronize()
    k0.record()
    for i in range(reps):
        plain(i)
    k1.record()
    torch.cuda.synchronize()
    ms_plain = k0.elapsed_time(k1) / reps
    del logits

    # end to end: [q | w | page table] in one pinned block down, [ids | counts] in one block back
    nq, nw, nbt = q.numel() * 2, w.numel() * 4, tables[0].numel() * 4
    hin = []
    for r in range(c["copies"]):
        h = torch.empty(nq + nw + nbt, dtype=torch.uint8).pin_memory()
        h[:nq].copy_(q.cpu().view(torch.uint8).reshape(-1))
        h[nq:nq + nw].copy_(w.cpu().view(torch.uint8).reshape(-1))
        h[nq + nw:].copy_(tables[r].cpu().view(torch.uint8).reshape(-1))
        hin.append(h)
    din = torch.empty(nq + nw + nbt, dtype=torch.uint8, device=dev)
    dq = din[:nq].view(torch.bfloat16).view_as(q)
    dw = din[nq:nq + nw].view(torch.float32).view_as(w)
    dbt = din[nq + nw:].view(torch.int32).view_as(tables[0])
    dout = torch.empty(B * T * K + B * T, dtype=torch.int32, device=dev)
    e_oi, e_oc = dout[:B * T * K].view(B, T, K), dout[B * T * K:].view(B, T)
    hout = torch.empty(B * T * K + B * T, dtype=torch.int32).pin_memory()

    def e2e_step(i):
        r = i % c["copies"]
        din.copy_(hin[r], non_blocking=True)
        run_fp4_paged_mqa_logits(caches[r], dq, None, dw, dbt, None, bpc, top_k=K, fmt="nvfp4",
                                 page_tokens=P, status=status, row_topk=(ov, e_oi, e_oc))
        hout.copy_(dout, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(max(args.warmup, c["copies"])):
        e2e_step(i)
    t0 = time.perf_counter()
    for i in range(reps):
        e2e_step(i)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / reps
    assert status[0].item() == 0 and int(hout[B * T * K:].min()) == K
    peaks = measured_peaks()
    algo = cfg2_algorithmic_bytes(c)
    achieved = algo / (ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_kind": f"of {peaks['kind']}",
            "frac_of_nominal_8TBs": achieved / 8000.0, "kernel": "logits_row_kernel<NVFP4,64,1>",
            "workload": "BASELINE config 2: B=32, ctx 32768, indexer logits + exact top-k 2048, one launch",
            "launch_us": ms * 1e3, "algorithmic_bytes": algo, "traffic": NCU_TRAFFIC_BYTES}
    extra = {"step_us": ms * 1e3, "logits_without_select_us": ms_plain * 1e3, "tokens_per_s": B * T / (ms * 1e-3), "e2e_step_us": e2e_ms * 1e3,
             "e2e_tokens_per_s": B * T / (e2e_ms * 1e-3), "h2d_bytes_per_step": hin[0].numel(),
             "d2h_bytes_per_step": hout.numel() * 4,
             "l2": f"rotating {c['copies']} cache copies ({c['copies'] * 75.5:.0f} MB > 126 MB L2)"}
    return roof, extra


def mla_alone(args, dev):
    """The tcgen05 sparse-MLA tile alone: B = 32 queries x 2048 selected rows, 128 heads, bf16
    576/512, no slot splits; flops = 278528 per selected token against the bf16 burst peak."""
    import torch
    from mega_dsa_cp_b200.tiles.hca import run_sparse_mla

    B, H, DQK, K, E = 32, 128, 576, 2048, 1 << 20     # KV pool 1.2 GB > L2
    g = torch.Generator(device=dev).manual_seed(3)
    q = (torch.randn(B, 1, H, DQK, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    kv = (torch.randn(E, 1, DQK, generator=g, device=dev) * 0.5).to(torch.bfloat16)
    pts = [torch.randint(0, E, (B, K), generator=g, device=dev, dtype=torch.int32) for _ in range(4)]
    kvalid = torch.full((B,), 128 + K, dtype=torch.int32, device=dev)
    o = torch.empty(B, 1, H, 512, dtype=torch.bfloat16, device=dev)
    lse = torch.empty(B, 1, H, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    run = lambda i: run_sparse_mla(q, None, kv, None, pts[i % 4], o, lse, kvalid, None, None, 1 / math.sqrt(DQK),
                                   n_splits=1, status=status)
    reps = max(args.steps, 20)
    for i in range(4):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(reps):
        run(i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    assert status[0].item() == 0
    peaks = measured_peaks()
    flops = B * K * 278528
    tf = flops / (ms * 1e-3) / 1e12
    return {"bound": "tensor", "achieved": tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": tf / peaks["bf16_tflops"], "peak_kind": f"of {peaks['kind']} (burst)", "kernel": "mla_umma_kernel<576>",
            "workload": "B=32 queries x 2048 selected rows, 128 heads, bf16 576/512, random gather from a 1.2 GB pool",
            "launch_us": ms * 1e3, "algorithmic_flops": flops, "algorithmic_bytes": B * (K * 1152 + 147456 + 131072),
            "traffic": None}


def merge_alone(args, dev):
    """The candidate merge alone: 8 queries, 4 lists of 2048 candidates each -> exact top-2048 (the size of a
    first-level merge of BASELINE config 2's chunk lists)."""
    import torch
    from mega_dsa_cp_b200.tiles.merge import run_merge_topk

    B, K, L = 8, 2048, 4
    g = torch.Generator(device=dev).manual_seed(4)
    v = torch.randn(B, 1, L, K, generator=g, device=dev)
    i = torch.randint(0, 1 << 20, (B, 1, L, K), generator=g, device=dev, dtype=torch.int32)
    c = torch.full((B, 1, L), K, dtype=torch.int32, device=dev)
    ov = torch.zeros(B, 1, K, device=dev)
    oi = torch.zeros(B, 1, K, dtype=torch.int32, device=dev)
    oc = torch.zeros(B, 1, dtype=torch.int32, device=dev)
    reps = max(args.steps, 20)
    for _ in range(4):
        run_merge_topk(v, i, c, ov, oi, oc, None, top_k=K)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        run_merge_topk(v, i, c, ov, oi, oc, None, top_k=K)
    e1.record()
    torch.cuda.synchronize()
    return {"kernel": "merge_topk_kernel", "workload": f"{B} queries x {L} lists x {K} candidates -> top-{K}",
            "launch_us": e0.elapsed_time(e1) / reps * 1e3, "count_ok": bool((oc == K).all()),
            "note": "launch-to-launch time of back-to-back host launches (a lower bound of ~14 us is the host's launch rate)"}


# ----------------------------------------------------------------------------
# CPU arm: the oracle port of the same path on the host cores
# ----------------------------------------------------------------------------
def cpu_layer_sample(world, max_steps=10, budget_s=20.0):
    """One sequence of the CP = world layer-step (context 131072, indexer + hierarchical top-k 2048 +
    sparse MLA + LSE merge) per step through the oracle, on all host cores."""
    import torch
    from oracle import dsa_oracle as orc

    # torchrun pins OMP_NUM_THREADS=1; inside an N-rank GPU run the other ranks' host threads sit in a barrier
    # and keep a core each, so they are left out (a thread that has to share its core stalls the whole team)
    busy = int(os.environ.get("WORLD_SIZE", "1")) - 1 if os.environ.get("RANK") is not None else 0
    torch.set_num_threads(max(1, (os.cpu_count() or 1) - busy))
    cc = cp_config(world)
    S, K, H, DQK = cc["S"], cc["top_k"], cc["H"], cc["d_qk"]
    g = torch.Generator().manual_seed(0)
    kd = torch.randn(S, 128, generator=g)
    data, sf = orc.quant_nvfp4(kd)
    q_idx = torch.randn(64, 128, generator=g).bfloat16().float()
    w_idx = torch.randn(64, generator=g) / 64.0
    q_mla = (torch.randn(H, DQK, generator=g) * 0.5).bfloat16().float()
    kv = (torch.randn(S, DQK, generator=g) * 0.5).bfloat16().float()

    def once():   # the path reads the quantised cache: the dequantisation is part of a step
        k = orc.dequant_fp4(data, sf, "nvfp4")
        return orc.decode_step_ref(q_idx, w_idx, k, q_mla, kv, S, K, 1.0 / math.sqrt(DQK), cp=world)

    for _ in range(2):
        once()
    t0 = time.perf_counter()
    steps = 0
    while steps < max_steps and (steps < 3 or time.perf_counter() - t0 < budget_s):
        once()
        steps += 1
    dt = (time.perf_counter() - t0) / steps
    return {"value": 1.0 / dt, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of the {cc['B']} sequences of the CP={world} layer-step per step (ctx {S}: NVFP4 dequant, "
                      f"64-head logits, hierarchical top-k {K}, sparse MLA, LSE merge), {steps} timed steps, torch CPU, "
                      f"{os.cpu_count()} host cpus"}, dt * 1e3, steps


def run_reference(args):
    """The reference's CPU implementation of the path, as restated in oracle/ (the reference is pure
    Python + a GPU JIT and is not installed on the bench box).  Rank 0 alone works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = max(args.gpus, int(os.environ.get("WORLD_SIZE", "1")))
    cpu, ms, steps = cpu_layer_sample(world, max_steps=max(3, min(args.steps, 20)), budget_s=60.0)
    cc = cp_config(world)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": 2, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"sample on host cores of the full DSA decode layer-step at CP={world}: 1 of the "
                               f"{cc['B']} sequences per step, ctx {cc['S']}, indexer + top-k {cc['top_k']} + sparse MLA "
                               "+ LSE merge"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--copies", type=int, default=None, help="rotation copies of the config-2 index cache (profiling runs)")
    ap.add_argument("--skip-cpu", action="store_true", help="omit the CPU baseline leg (profiling runs)")
    ap.add_argument("--skip-alone", action="store_true", help="N=1: omit the kernels-alone legs (indexer, MLA)")
    ap.add_argument("--row-exact", default="default", choices=["default", "local", "global", "off", "l1"],
                    help="where the chunk tasks settle the exact selection (default: the layer's choice for N)")
    ap.add_argument("--dynamic", action="store_true", help="blocks pull tasks from one shared queue (dynamic scheduling)")
    ap.add_argument("--only", default=None, choices=["indexer", "mla", "merge"],
                    help="run only one kernel-alone leg and print its block (profiling runs)")
    args = ap.parse_args()
    if args.copies:
        CFG2["copies"] = args.copies
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
        return
    if args.only:
        import torch

        torch.cuda.set_device(0)
        dev = torch.device("cuda", 0)
        out = {"indexer": indexer_alone, "mla": mla_alone, "merge": merge_alone}[args.only](args, dev)
        print(json.dumps(out))
        return
    R, line, layers, inputs = run_layer(args)
    if R.rank == 0:
        if R.world == 1 and not args.skip_alone:
            # free the layer-step's caches first: the kernels-alone legs bring their own
            layers.clear()
            inputs.clear()
            import torch

            torch.cuda.empty_cache()
            layer_roof = line["roofline"]
            roof, extra = indexer_alone(args, R.dev)
            line["roofline"] = roof               # the dominant kernel, alone, on BASELINE config 2
            line["roofline_layer_step"] = layer_roof
            line["roofline_mla"] = mla_alone(args, R.dev)
            line["cfg2_indexer"] = extra
        line["cpu_baseline"] = None if args.skip_cpu else cpu_layer_sample(R.world)[0]
        print(json.dumps(line), flush=True)
    R.barrier()
    R.close()


if __name__ == "__main__":
    main()
