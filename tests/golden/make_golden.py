"""Regenerate the golden fixtures in this directory from the reference's own
CPU-runnable torch code.

Run where the reference checkout is available:

    MDC_REF_PATH=/path/to/mega-dsa-cp python tests/golden/make_golden.py

The fixtures (small .npz / .json files) are committed; tests never need the
reference checkout.  Each fixture stores the seeded inputs next to the outputs
the reference produced for them, so the oracle (oracle/dsa_oracle.py) and the
host-side package code can be pinned to the reference bit for bit (integers,
bytes, queue words) or to fp32 round-off (floating point).
"""

from __future__ import annotations

import json
import os
import random
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("MDC_REF_PATH")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set MDC_REF_PATH to a checkout of the reference (mega-dsa-cp)")
sys.dont_write_bytecode = True
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            if v.dtype == torch.float8_e4m3fn:
                v = v.view(torch.uint8)
            if v.dtype == torch.bfloat16:
                v = v.view(torch.int16)
            v = v.cpu().numpy()
        out[k] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: tuple(a.shape) for k, a in out.items()})


def gen_fp4():
    from mega_dsa_cp.tiles import fp4

    g = torch.Generator().manual_seed(11)
    x = torch.randn(96, 128, generator=g) * torch.logspace(-3, 2, 96).unsqueeze(1)
    x[5] = 0.0
    x[6, :32] = 1e-7
    packed, sf = fp4.quant_mxfp4(x)
    deq = fp4.dequant_mxfp4(packed, sf)
    sf2 = torch.randint(0, 255, (256, 4), generator=g, dtype=torch.uint8)
    atom = fp4.sf_to_atom(sf2)
    save("fp4", x=x, packed=packed, sf=sf, deq=deq, sf_plain=sf2, sf_atom=atom)

    kv_fused, kv_sf = fp4.make_index_cache(2, 2, device="cpu", seed=0)
    qp, qsf, qatom, w = fp4.make_q(2, q_len=2, device="cpu", seed=1)
    bt = torch.tensor([[3, 0], [1, 2]], dtype=torch.int32)
    out = fp4.ref_logits(qp, qsf, kv_fused, kv_sf, w, bt, q_len=2)
    save("logits_mxfp4", kv_fused=kv_fused, kv_sf=kv_sf, q_packed=qp, q_sf=qsf,
         q_sf_atom=qatom, w=w, bt=bt, logits=out)


def gen_merge():
    from mega_dsa_cp.tiles.merge_ref import merge_topk_ref

    cases = {}
    g = torch.Generator().manual_seed(5)
    for name, (B, q, L, maxK, K, mode) in {
        "full": (1, 2, 4, 64, 64, "full"),
        "var": (2, 1, 5, 48, 32, "var"),
        "ties": (1, 1, 6, 64, 64, "ties"),
        "neginf": (1, 2, 3, 64, 32, "neginf"),
        "tiny": (1, 1, 4, 32, 64, "tiny"),
        "const": (1, 1, 2, 64, 32, "const"),
    }.items():
        v = torch.randn(B, q, L, maxK, generator=g)
        c = torch.full((B, q, L), maxK, dtype=torch.int32)
        if mode == "var":
            c = torch.randint(0, maxK + 1, (B, q, L), generator=g, dtype=torch.int32)
        if mode == "tiny":
            c = torch.randint(0, 6, (B, q, L), generator=g, dtype=torch.int32)
        if mode == "ties":
            v = torch.randint(0, 8, (B, q, L, maxK), generator=g).float() / 4.0
        if mode == "const":
            v = torch.full((B, q, L, maxK), 0.25)
        if mode == "neginf":
            v = v.masked_fill(torch.rand(B, q, L, maxK, generator=g) < 0.4, -float("inf"))
        ids = torch.empty(B, q, L, maxK, dtype=torch.int32)
        for b in range(B):
            for t in range(q):
                ids[b, t] = torch.randperm(1 << 20, generator=g)[: L * maxK].reshape(L, maxK).to(torch.int32)
        ids.view(-1)[0] = 0
        ids.view(-1)[1] = (1 << 31) - 1
        ov, oi, oc = merge_topk_ref(v, ids, c, K)
        cases.update({f"{name}_v": v, f"{name}_i": ids, f"{name}_c": c, f"{name}_k": np.int32(K),
                      f"{name}_ov": ov, f"{name}_oi": oi, f"{name}_oc": oc})
    save("merge", **cases)


def gen_lse():
    from mega_dsa_cp.tiles.lse_merge_ref import lse_merge_ref

    g = torch.Generator().manual_seed(9)
    acc_o = torch.randn(3, 2, 4, 8, 16, generator=g) * 2.0
    acc_l = torch.randn(3, 2, 4, 8, generator=g) * 4.0 + 2.0
    acc_l = acc_l.masked_fill(torch.rand(3, 2, 4, 8, generator=g) < 0.3, -float("inf"))
    acc_l[:, :, :, :2] = -float("inf")
    out = {}
    for cp in (1, 3, 4):
        o, l = lse_merge_ref(acc_o, acc_l, cp)
        out[f"o_cp{cp}"], out[f"lse_cp{cp}"] = o, l
    save("lse_merge", acc_o=acc_o, acc_lse=acc_l, **out)


def gen_hca():
    from mega_dsa_cp.tiles import hca_ref

    hca_ref.H, hca_ref.D = 16, 64  # shrink the module constants; code untouched
    H, D = 16, 64
    g = torch.Generator().manual_seed(21)
    B, T = 2, 2
    q = hca_ref.quant_fp8(torch.randn(B, T, H, D, generator=g) * 0.5)
    kwin = hca_ref.quant_fp8(torch.randn(B, 128, D, generator=g) * 0.5)
    E = 700
    kcmp = hca_ref.quant_fp8(torch.randn(E, 1, D, generator=g) * 0.5)
    cols = 384
    pt_cmp = torch.zeros(B * T, cols, dtype=torch.int32)
    n_sel = [300, 37, 384, 1]
    k_valid = torch.zeros(B * T, dtype=torch.int32)
    win_valid = torch.tensor([128, 90, 0, 128], dtype=torch.int32)
    for r in range(B * T):
        pt_cmp[r, : n_sel[r]] = torch.randperm(E, generator=g)[: n_sel[r]].to(torch.int32)
        k_valid[r] = 128 + n_sel[r]
    inp = {
        "q32": q.float(), "kwin32": kwin.float(), "kcmp32": kcmp.float().view(-1, D),
        "pt_cmp": pt_cmp, "k_valid": k_valid, "win_valid": win_valid, "page_cmp": 1,
    }
    sink_off = torch.full((H,), -float("inf"))
    sink_on = torch.randn(H, generator=g) * 0.5 - 1.0
    out = {}
    for tag, sink in (("nosink", sink_off), ("sink", sink_on)):
        o1, l1 = hca_ref.ref_hca(inp, sink, 0.05, fp8_p=True)
        o2, l2 = hca_ref.ref_hca(inp, sink, 0.05, fp8_p=False)
        o3, l3 = hca_ref.ref_hca_online(inp, sink, 0.05)
        out.update({f"{tag}_o_fp8p": o1, f"{tag}_l_fp8p": l1, f"{tag}_o": o2, f"{tag}_l": l2,
                    f"{tag}_o_online": o3, f"{tag}_l_online": l3})
    # paged compressed pool (16 entries per page), dense page table
    kcmp16 = hca_ref.quant_fp8(torch.randn(12, 16, D, generator=g) * 0.5)
    pt16 = torch.zeros(B * T, 8, dtype=torch.int32)
    for r in range(B * T):
        pt16[r] = torch.randperm(12, generator=g)[:8].to(torch.int32)
    kv16 = torch.tensor([128 + 128, 128 + 77, 128 + 16, 128 + 100], dtype=torch.int32)
    inp16 = dict(inp, kcmp32=kcmp16.float().view(-1, D), pt_cmp=pt16, k_valid=kv16, page_cmp=16)
    o4, l4 = hca_ref.ref_hca(inp16, sink_on, 0.05, fp8_p=False)
    o5, l5 = hca_ref.ref_hca_online(inp16, sink_on, 0.05)
    save("hca", q=q, kwin=kwin, kcmp=kcmp.view(-1, D), pt_cmp=pt_cmp, k_valid=k_valid,
         win_valid=win_valid, sink_on=sink_on, scale=np.float32(0.05),
         kcmp16=kcmp16.view(-1, D), pt16=pt16, k_valid16=kv16,
         paged_o=o4, paged_l=l4, paged_o_online=o5, paged_l_online=l5, **out)


def gen_compress():
    from mega_dsa_cp.tiles import compress_ref as cr

    g = torch.Generator().manual_seed(33)
    x = torch.randn(6, 128, generator=g)
    had = cr.hadamard128_staged(x)
    had_m = x @ cr.hadamard_matrix(128)
    w512 = torch.rand(512, generator=g) + 0.5
    w128 = torch.rand(128, generator=g) + 0.5
    y = torch.randn(3, 512, generator=g)
    freqs = cr.make_freqs_cis(64)
    normed = cr.rms_norm(y, w512, 1e-6)
    roped = cr.rope_last64(normed, freqs, 17)
    e4 = cr.post_attn(y[0], w512, 1e-6, freqs, 17, 0.02)
    yi = torch.randn(128, generator=g)
    pk, sf = cr.post_indexer_bitexact(yi, w128, 1e-6, freqs, 12)
    qx = torch.randn(8, 128, generator=g) * torch.logspace(-2, 2, 8).unsqueeze(1)
    qpk, qsf = cr.quant_mxfp4_bitexact(qx)

    kv = torch.randn(8, 128, generator=g)
    sc = torch.randn(8, 128, generator=g) * 3
    ape = cr.synth_ape(128, 8)
    full = cr.csa_pool_window(kv, sc, ape)
    p0 = cr.csa_partial(kv[0::2], sc[0::2], ape[0::2])
    p1 = cr.csa_partial(kv[1::2], sc[1::2], ape[1::2])
    merged = cr.csa_merge([p0, p1])

    recs = torch.stack([cr.synth_record(1, p, 512, False, seed=3) for p in range(12)])
    bias = cr.synth_ape(512, 16)
    st = [cr.c128_state_init(), cr.c128_state_init()]
    for p in range(12):
        st[p % 2] = cr.c128_update(st[p % 2], recs[p, :512], recs[p, 512:], bias[p])
    merged128 = cr.c128_merge_states(st[0], st[1])
    rec_dual = cr.synth_record(2, 7, 128, True, seed=0)
    save("compress", x=x, had=had, had_m=had_m, w512=w512, w128=w128, y=y, freqs=freqs,
         normed=normed, roped=roped, e4=e4, yi=yi, idx_packed=pk, idx_sf=sf,
         qx=qx, q_packed=qpk, q_sf=qsf, kv=kv, sc=sc, ape=ape, pool_full=full,
         p0_m=p0[0], p0_l=p0[1], p0_w=p0[2], pool_merged=merged,
         recs=recs, bias128=bias, st0_m=st[0][0], st0_l=st[0][1], st0_k=st[0][2],
         merged128=merged128, rec_dual=rec_dual)


def _dag_to_json(tasks, events):
    return {
        "events": [[e.name, e.scope] for e in events],
        "tasks": [
            {"name": t.name, "rank": t.rank, "waits": [w.event for w in t.waits],
             "notifies": [[n.event, n.dst_rank] for n in t.notifies], "coords": list(t.coords)}
            for t in tasks
        ],
    }


def gen_schedule():
    from dag_gen import random_dag
    from mega_dsa_cp.events import (SCOPE_LOCAL, SCOPE_SYS, EventSpec, NotifyEdge, TaskSpec,
                                    WaitEdge, validate)
    from mega_dsa_cp.schedule.codegen import codegen_schedule

    cases = []
    for seed in range(6):
        n_ctas = 8 if seed % 2 == 0 else 5
        tasks, events, _, preds, _ = random_dag(seed, 80, 0.05, n_ctas)
        errors, table = validate(tasks, events, world_size=1)
        op_of = {t.name: (i % 3) + 1 for i, t in enumerate(tasks)}
        extent_of = {tasks[0].name: 1, tasks[3].name: 2}
        s = codegen_schedule(tasks, events, rank=0, n_ctas=n_ctas, op_of=op_of, extent_of=extent_of)
        cases.append({
            "dag": _dag_to_json(tasks, events), "world": 1, "rank": 0, "n_ctas": n_ctas,
            "op_of": op_of, "extent_of": extent_of, "errors": errors,
            "arities": [[k[0], k[1], v] for k, v in sorted(table.arities.items())],
            "queues": s.queues, "arity": s.arity, "scopes": s.scopes, "topo": s.topo,
            "op_list": s.op_of, "n_events": s.n_events,
        })
    # two-rank DAG with coords, both ranks
    rng = random.Random(4)
    tasks, events = [], []
    for i in range(12):
        r = i % 2
        ev_in = f"in{i}"
        waits = ()
        if i >= 1:
            events.append(EventSpec(ev_in, SCOPE_SYS))
            waits = (WaitEdge(ev_in),)
        notifies = []
        if i + 1 < 12:
            notifies.append(NotifyEdge(f"in{i+1}", (i + 1) % 2))
        if i + 3 < 12:
            notifies.append(NotifyEdge(f"in{i+3}", (i + 3) % 2))
        tasks.append(TaskSpec(f"k{i}", r, waits=waits, notifies=tuple(notifies),
                              coords=(i, rng.randrange(9), rng.randrange(9))))
    for rank in (0, 1):
        s = codegen_schedule(tasks, events, rank=rank, n_ctas=3, world_size=2,
                             op_of={t.name: 7 for t in tasks})
        errors, table = validate(tasks, events, 2)
        cases.append({
            "dag": _dag_to_json(tasks, events), "world": 2, "rank": rank, "n_ctas": 3,
            "op_of": {t.name: 7 for t in tasks}, "extent_of": {}, "errors": errors,
            "arities": [[k[0], k[1], v] for k, v in sorted(table.arities.items())],
            "queues": s.queues, "arity": s.arity, "scopes": s.scopes, "topo": s.topo,
            "op_list": s.op_of, "n_events": s.n_events,
        })
    # injected faults: the validator must report at least one error for each
    faults = {
        "cycle": ([TaskSpec("a", 0, (WaitEdge("e1"),), (NotifyEdge("e2", 0),)),
                   TaskSpec("b", 0, (WaitEdge("e2"),), (NotifyEdge("e1", 0),))],
                  [EventSpec("e1", SCOPE_LOCAL), EventSpec("e2", SCOPE_LOCAL)], 1),
        "unknown_event": ([TaskSpec("a", 0, (WaitEdge("nope"),))], [], 1),
        "wait_without_producer": ([TaskSpec("a", 0, (WaitEdge("e"),))], [EventSpec("e", SCOPE_LOCAL)], 1),
        "notify_without_consumer": ([TaskSpec("a", 0, (), (NotifyEdge("e", 0),))],
                                    [EventSpec("e", SCOPE_LOCAL)], 1),
        "local_cross_rank": ([TaskSpec("a", 0, (), (NotifyEdge("e", 1),)),
                              TaskSpec("b", 1, (WaitEdge("e"),))], [EventSpec("e", SCOPE_LOCAL)], 2),
        "sys_without_cross": ([TaskSpec("a", 0, (), (NotifyEdge("e", 0),)),
                               TaskSpec("b", 0, (WaitEdge("e"),))], [EventSpec("e", SCOPE_SYS)], 2),
        "dst_out_of_range": ([TaskSpec("a", 0, (), (NotifyEdge("e", 7),))], [EventSpec("e", SCOPE_SYS)], 2),
        "valid_pingpong": ([TaskSpec("a", 0, (), (NotifyEdge("e", 1),)),
                            TaskSpec("b", 1, (WaitEdge("e"),), (NotifyEdge("f", 0),)),
                            TaskSpec("c", 0, (WaitEdge("f"),))],
                           [EventSpec("e", SCOPE_SYS), EventSpec("f", SCOPE_SYS)], 2),
    }
    fault_out = {}
    for name, (tasks, events, world) in faults.items():
        errors, _ = validate(tasks, events, world)
        fault_out[name] = {"dag": _dag_to_json(tasks, events), "world": world, "errors": errors}
    with open(os.path.join(HERE, "schedule.json"), "w") as f:
        json.dump({"cases": cases, "faults": fault_out}, f)
    print("wrote schedule.json", len(cases), "cases")


if __name__ == "__main__":
    torch.manual_seed(0)
    gen_fp4()
    gen_merge()
    gen_lse()
    gen_hca()
    gen_compress()
    gen_schedule()
