"""GPU tests of the event / scheduler / comm device layer and of the decode
megakernel on one GPU (world size 1), through the C ABI."""

import math
import random

import pytest
import torch

from mega_dsa_cp.events import SCOPE_LOCAL, EventSpec, NotifyEdge, TaskSpec, WaitEdge
from mega_dsa_cp.schedule.codegen import codegen_schedule

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _random_dag(seed, n_tasks, edge_prob):
    rng = random.Random(seed)
    order = list(range(n_tasks))
    rng.shuffle(order)
    pos = {t: i for i, t in enumerate(order)}
    preds = {j: [i for i in range(n_tasks) if pos[i] < pos[j] and rng.random() < edge_prob] for j in range(n_tasks)}
    events, tasks = [], []
    for t in range(n_tasks):
        if preds[t]:
            events.append(EventSpec(f"e{t}", SCOPE_LOCAL))
        tasks.append(TaskSpec(f"t{t}", 0, (WaitEdge(f"e{t}"),) if preds[t] else (),
                              tuple(NotifyEdge(f"e{j}", 0) for j in range(n_tasks) if t in preds[j]), (t, 0, 0)))
    return tasks, events, preds


def _setup(tasks, events, ops, n_ctas):
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.events.symm import alloc_event_buffer
    from mega_dsa_cp_b200.schedule.device import upload_schedule

    sched = codegen_schedule(tasks, events, rank=0, n_ctas=n_ctas, op_of=ops)
    ds = upload_schedule(sched, DEV)
    ev = alloc_event_buffer(max(len(events), 1), device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    return ds, ev, status


def test_random_dag_runs_in_dependency_order_over_two_phases():
    """512 tasks with random dependencies on 32 blocks; the logged execution
    order must be a valid linearisation, also when the same launch is replayed
    with only the phase scalar advanced (the reference's single-GPU event and
    scheduler tests)."""
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.schedule.device import launch_megakernel

    tasks, events, preds = _random_dag(3, 512, 0.01)
    ds, ev, status = _setup(tasks, events, {t.name: N.OP_LOG for t in tasks}, 32)
    for phase in range(2):
        log = torch.zeros(1024, dtype=torch.int32, device=DEV)
        ds.scalars[0] = phase
        launch_megakernel(ds, ev, None, status, log=log)
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        n = log[0].item()
        order = log[1:1 + n].tolist()
        assert sorted(order) == list(range(512))
        at = {t: i for i, t in enumerate(order)}
        assert all(at[p] < at[t] for t, ps in preds.items() for p in ps)
    cells = ev.tensor.view(-1, 16)[:, 0]
    arity = torch.tensor([len(preds[int(e.name[1:])]) for e in events], device=DEV)
    assert torch.equal(cells[:len(events)], 2 * arity)   # counters only ever grow


def test_random_dag_with_dynamic_task_pulling():
    """The same random DAG as one shared queue in dependency order: 32 blocks pull the next task with an
    atomic counter; three launches (the counters rewind themselves), the order stays a valid linearisation."""
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.events.symm import alloc_event_buffer
    from mega_dsa_cp_b200.schedule.device import launch_megakernel, upload_schedule

    tasks, events, preds = _random_dag(5, 512, 0.01)
    sched = codegen_schedule(tasks, events, rank=0, n_ctas=1, op_of={t.name: N.OP_LOG for t in tasks})
    ds = upload_schedule(sched, DEV, dynamic_ctas=32)
    assert ds.n_tasks == 512 and ds.n_ctas == 32
    ev = alloc_event_buffer(max(len(events), 1), device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    for phase in range(3):
        log = torch.zeros(1024, dtype=torch.int32, device=DEV)
        ds.scalars[0] = phase
        launch_megakernel(ds, ev, None, status, log=log)
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        order = log[1:1 + log[0].item()].tolist()
        assert sorted(order) == list(range(512))
        at = {t: i for i, t in enumerate(order)}
        assert all(at[p] < at[t] for t, ps in preds.items() for p in ps)
        assert ds.dyn_ctl.tolist() == [0, 0]


def test_wait_gives_up_within_its_budget_and_reports():
    """A wait whose event nobody notifies must end after the budget with a
    status record (code, event, seen, wanted) and leave the context usable."""
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.schedule.device import launch_megakernel, upload_schedule
    from mega_dsa_cp_b200.events.symm import alloc_event_buffer
    from mega_dsa_cp_b200.schedule.codegen import Schedule, pack_header, OP_END

    # hand-made queue: one block waits on event 0 (arity 3) that nothing notifies; another block just logs
    q0 = [pack_header(N.OP_LOG, 1, 0, 0), 7, 0, 0, 0, pack_header(OP_END, 0, 0, 0)]
    q1 = [pack_header(N.OP_LOG, 0, 0, 0), 9, 0, 0, pack_header(OP_END, 0, 0, 0)]
    sched = Schedule(queues=[q0, q1], arity=[3], scopes=[0], topo=[0, 1], op_of=[N.OP_LOG] * 2, n_events=1)
    ds = upload_schedule(sched, DEV)
    ev = alloc_event_buffer(1, device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    log = torch.zeros(16, dtype=torch.int32, device=DEV)
    launch_megakernel(ds, ev, None, status, log=log, wait_budget_ns=20_000_000)
    torch.cuda.synchronize()
    st = status.tolist()
    assert st[0] == N.DEV_WAIT_TIMEOUT and st[2] == 0 and st[4] == 0 and st[6] == 3, st
    assert log[0].item() == 1 and log[1].item() == 9
    # the context is alive and the library still works
    assert torch.ones(4, device=DEV).sum().item() == 4


def test_bulk_push_and_verify_world1():
    """smem -> arena bulk push, release notify, system-scope read-back (the
    world-size-1 degenerate of the reference's comm test)."""
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.comm.buffers import alloc_arena
    from mega_dsa_cp_b200.schedule.device import launch_megakernel

    slots, nbytes = 6, 4096
    events = [EventSpec(f"arrived{s}", SCOPE_LOCAL) for s in range(slots)]
    tasks, ops = [], {}
    for s in range(slots):
        tasks.append(TaskSpec(f"push{s}", 0, (), (NotifyEdge(f"arrived{s}", 0),), (s, 0, s)))
        tasks.append(TaskSpec(f"check{s}", 0, (WaitEdge(f"arrived{s}"),), (), (s, 0, s)))
        ops[f"push{s}"], ops[f"check{s}"] = N.OP_PUSH, N.OP_VERIFY
    ds, ev, status = _setup(tasks, events, ops, 4)
    arena = alloc_arena({"test": slots * nbytes}, phases=1, device=DEV)
    for phase in range(2):
        ds.scalars[0] = phase
        launch_megakernel(ds, ev, arena, status, test_off=arena.region_off("test"), test_slot_bytes=nbytes)
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
    assert arena.tensor.view(torch.int32).abs().sum().item() != 0


@pytest.mark.parametrize("B,S,K,bpc,qpath,exact,dynamic", [
    (2, 4096, 512, 16, False, True, False), (3, 8192, 2048, 32, False, True, False), (3, 8192, 2048, 32, True, True, False),
    (3, 8192, 2048, 32, False, False, False), (3, 8192, 2048, 32, True, True, True)])
def test_decode_layer_cp1_matches_oracle(B, S, K, bpc, qpath, exact, dynamic):
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from oracle import dsa_oracle as orc

    P, H, DQK = 64, 128, 576
    case = indexer_case(B, S, P, "nvfp4", seed=4)
    g = torch.Generator().manual_seed(8)
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S - 100 * b for b in range(B)], dtype=torch.int32)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=64, distribute_q=qpath, q_tasks=qpath,   # qpath: q through the QPATH task
                           dynamic=dynamic,   # dynamic: the blocks pull tasks from one shared queue
                           row_exact=exact)   # exact: the chunk tasks settle the row's top-k, the merge only passes it on
    d = lambda t: t.to(DEV)
    layer.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), d(case["q"]), d(case["w"]), d(q_mla), d(kv)))
    for phase in range(2):   # the second launch replays with the phase bumped
        layer.step()
        torch.cuda.synchronize()
        layer.check_status()
    # the optional task timeline: one entry per task of this rank, stamps in order
    trace = torch.zeros(4 + 4 * 1024, dtype=torch.int64, device=DEV)
    layer.step(trace=trace)
    torch.cuda.synchronize()
    layer.check_status()
    n_tasks = len(layer.schedule.topo)
    assert int(trace[0]) == n_tasks
    e = trace[4:4 + 4 * n_tasks].reshape(n_tasks, 4).cpu()
    assert bool((e[:, 1] <= e[:, 2]).all()) and bool((e[:, 2] <= e[:, 3]).all())
    assert set(((e[:, 0] >> 24) & 0xff).tolist()) <= {1, 2, 3, 4, 5, 6, 9}
    data, sf = orc.split_index_pages(case["fused"], "nvfp4", P)
    kd_all = orc.dequant_fp4(data, sf, "nvfp4").reshape(-1, P, 128)
    for b in range(B):
        kd = kd_all[case["bt"][b].long()].reshape(S, 128)
        sel, _, _ = orc.decode_step_ref(case["q_deq"][b], case["w"][b], kd, q_mla[b, 0].float(),
                                        kv[b * S:(b + 1) * S, 0].float(), int(seq[b]), K, 1 / math.sqrt(DQK))
        n = int(layer.sel_c[b])
        got = torch.sort(layer.sel_i[b, :n].cpu()).values
        overlap = len(set(got.tolist()) & set(sel.tolist())) / max(1, sel.numel())
        assert n == sel.numel() and overlap >= 0.999, (n, sel.numel(), overlap)
        # attention + LSE merge are always held to the oracle, on the ids the kernel selected
        # (a near-tie at the selection boundary may swap an id; the attention must still be right)
        o, l = orc.attend_selected_ref(q_mla[b, 0].float(), kv[b * S:(b + 1) * S, 0].float(),
                                       layer.sel_i[b, :n].cpu(), 1 / math.sqrt(DQK))
        assert (layer.out[b].cpu() - o).abs().max() < 2e-2
        assert (layer.out_lse[b].cpu() - l).abs().max() < 1e-3


def test_layer_steps_replay_from_a_cuda_graph():
    """The phase counter lives on the device and the kernel advances it, so a model step -- here 61
    layer-calls, the reference's count (docs/overview.md:10) -- captured once as a CUDA graph replays
    with no host update in between; every replay gives the eager result."""
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs

    B, S, K, bpc, P, H, DQK = 2, 4096, 512, 16, 64, 128, 576
    case = indexer_case(B, S, P, "nvfp4", seed=6)
    g = torch.Generator().manual_seed(9)
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S, S - 300], dtype=torch.int32)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=32)
    d = lambda t: t.to(DEV)
    layer.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), d(case["q"]), d(case["w"]), d(q_mla), d(kv)))
    layer.step()
    torch.cuda.synchronize()
    layer.check_status()
    want_o, want_l, want_i = layer.out.clone(), layer.out_lse.clone(), layer.sel_i.clone()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(61):
                layer.step(stream=stream)
    for _ in range(2):
        layer.out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        layer.check_status()
        assert torch.equal(layer.out, want_o) and torch.equal(layer.out_lse, want_l) and torch.equal(layer.sel_i, want_i)
    assert int(layer.dsched.scalars[0]) == 1 + 2 * 61   # one eager step + two replays of 61


@pytest.mark.parametrize("ratio", [4, 64])
def test_layer_step_runs_the_compressor_as_tasks(ratio):
    """CMP_STEP / CMP_FIN inside the persistent kernel (cp = 1): the layer-step rolls the compressor
    over closing groups; entries against single-machine pooling and the oracle's post chain (bit for
    bit for the MXFP4 codes), the attention path's result unchanged."""
    from dsa_inputs import indexer_case
    from test_gpu_compress import _post_checks
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from mega_dsa_cp_b200.tiles.compress import CompressorState
    from oracle import dsa_oracle as orc

    B, S, K, bpc, P, H, DQK = 2, 4096, 512, 16, 64, 128, 576
    steps = 13 if ratio == 4 else 2 * ratio + 3
    case = indexer_case(B, S, P, "nvfp4", seed=7)
    g = torch.Generator().manual_seed(10)
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S, S - 300], dtype=torch.int32)
    st = CompressorState(B, 1, 0, ratio, 128 if ratio == 4 else 16,
                         attn_dtype=torch.float8_e4m3fn if ratio == 4 else torch.bfloat16)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=32, compressor=st)
    d = lambda t: t.to(DEV)
    layer.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), d(case["q"]), d(case["w"]), d(q_mla), d(kv)))
    hd_rec = 4 * 512 if ratio == 4 else 2 * 512
    rec_a = torch.stack([torch.stack([orc.synth_record(b, p, 512, ratio == 4, seed=3) for p in range(steps)]) for b in range(B)])
    rec_i = torch.stack([torch.stack([orc.synth_record(b, p, 128, True) for p in range(steps)]) for b in range(B)])
    ape_a = orc.synth_bias(512, 8 if ratio == 4 else ratio)
    ape_i = orc.synth_bias(128, 8)
    gn = torch.Generator().manual_seed(2)
    norm_a, norm_i = torch.rand(512, generator=gn) + 0.5, torch.rand(128, generator=gn) + 0.5
    freqs = orc.make_freqs(4 * max(ratio, 64))
    glen = torch.zeros(B, dtype=torch.int32, device=DEV)
    new_a = torch.zeros(B, hd_rec, device=DEV)
    new_i = torch.zeros(B, 4 * 128, device=DEV)
    layer.bind_compressor(glen, new_a, new_i if ratio == 4 else None, d(ape_a), d(ape_i) if ratio == 4 else None,
                          d(norm_a), d(norm_i) if ratio == 4 else None, 1e-6, d(freqs), fp8_scale=0.02 if ratio == 4 else 1.0)
    tally = {"e4m3": 0, "e4m3_off_by_one": 0, "nibbles": 0}
    closed = 0
    first_out = None
    for s in range(steps):
        glen.fill_(s)
        new_a.copy_(rec_a[:, s])
        if ratio == 4:
            new_i.copy_(rec_i[:, s])
        layer.step()
        torch.cuda.synchronize()
        layer.check_status()
        if first_out is None:
            first_out = layer.out.clone()
        if (s + 1) % ratio == 0:
            n = s // ratio
            closed += 1
            for b in range(B):
                if ratio == 4:
                    pa = orc.csa_entry_ref(rec_a[b], ape_a, n, 512)
                    pi = orc.csa_entry_ref(rec_i[b], ape_i, n, 128)
                    _post_checks(st, b, n, pa, pi, 4 * n, norm_a, norm_i, freqs, 0.02, (ratio, s, b), tally)
                else:
                    want = orc.online_entry_ref(rec_a[b], ape_a, n, 512, ratio)
                    got = st.dbg_attn[b, n].cpu()
                    assert torch.allclose(got, want, rtol=2e-4, atol=2e-5), (s, b, (got - want).abs().max())
                    ent = orc.post_attn_bf16(got, norm_a, 1e-6, freqs, n * ratio).float()
                    assert torch.equal(st.attn_pool[b, n].cpu().float(), ent)
            assert st.k_valid.tolist() == [n + 1] * B
    assert closed >= 2
    assert torch.equal(layer.out, first_out)   # the attention path does not depend on the compressor tasks


def test_layer_step_writes_the_new_token_before_it_scores():
    """KVWRITE tasks (cp = 1): each step quantises the host-supplied index-K record of the new token into
    the paged NVFP4 cache (bit-exact against the oracle's quantiser), copies its KV row, grows the
    length, and the same step's selection and attention already see the token (oracle on the updated
    caches).  The global length advances on the device, so the steps need no host update of it."""
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from oracle import dsa_oracle as orc

    B, S, K, bpc, P, H, DQK = 2, 4096, 512, 16, 64, 128, 576
    case = indexer_case(B, S, P, "nvfp4", seed=12, shuffle=True)
    g = torch.Generator().manual_seed(13)
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    start = [1000, 63]                       # the second sequence crosses a page boundary on its second step
    seq = torch.tensor(start, dtype=torch.int32)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=32, kvwrite=True)
    d = lambda t: t.to(DEV)
    cache, kv_d, seq_d = d(case["fused"]), d(kv), d(seq)
    layer.bind(LayerInputs(cache, d(case["bt"]), seq_d, d(case["q"]), d(case["w"]), d(q_mla), kv_d))
    k_new = torch.zeros(B, 128, device=DEV)
    kv_new = torch.zeros(B, DQK, dtype=torch.bfloat16, device=DEV)
    glen = seq_d.clone()
    layer.bind_kvwrite(k_new, kv_new, glen, advance=True)
    steps = 3
    k_all = torch.randn(steps, B, 128, generator=g) * 1.7
    kv_all = (torch.randn(steps, B, DQK, generator=g) * 0.5).bfloat16()
    for s in range(steps):
        k_new.copy_(k_all[s])
        kv_new.copy_(kv_all[s])
        layer.step()
        torch.cuda.synchronize()
        layer.check_status()
    assert seq_d.tolist() == [x + steps for x in start] and glen.tolist() == [x + steps for x in start]
    pages = cache.cpu()
    for b in range(B):
        for s in range(steps):
            slot = start[b] + s
            pg = pages[int(case["bt"][b, slot // P])]
            codes, sf = orc.quant_nvfp4(k_all[s, b][None])
            assert torch.equal(pg[(slot % P) * 64:(slot % P + 1) * 64], codes[0]), (b, s)
            assert torch.equal(pg[P * 64 + (slot % P) * 8:P * 64 + (slot % P + 1) * 8], sf[0]), (b, s)
            assert torch.equal(kv_d[b * S + slot, 0].cpu(), kv_all[s, b])
    # the last step's result against the oracle on the updated caches
    data, sf = orc.split_index_pages(pages, "nvfp4", P)
    kd_all = orc.dequant_fp4(data, sf, "nvfp4").reshape(-1, P, 128)
    kv_h = kv_d.cpu()
    for b in range(B):
        n_tok = start[b] + steps
        kd = kd_all[case["bt"][b].long()].reshape(S, 128)
        want = orc.select_topk_ref(case["q_deq"][b], case["w"][b], kd, n_tok, K)
        n = int(layer.sel_c[b])
        got = layer.sel_i[b, :n].cpu()
        assert n == want.numel() and len(set(got.tolist()) & set(want.tolist())) >= n - 1
        assert int(got.max()) <= n_tok - 1 and (n_tok - 1) in set(got.tolist()) or n_tok > K   # short rows select every token, the new one included
        o, l = orc.attend_selected_ref(q_mla[b, 0].float(), kv_h[b * S:(b + 1) * S, 0].float(), got, 1 / math.sqrt(DQK))
        assert (layer.out[b].cpu() - o).abs().max() < 2e-2
        assert (layer.out_lse[b].cpu() - l).abs().max() < 1e-3


def test_local_notify_latency_probe():
    """Block-to-block notify -> wait on one GPU (two blocks of one launch): the probe completes every
    round inside its budget and reports a one-way latency of a plausible size (the reference publishes
    1.1 us on B200, docs/event-system.md:5)."""
    from mega_dsa_cp_b200.events.latency import local_notify_latency

    r = local_notify_latency(DEV, rounds=500)
    assert r["rounds"] == 450 and 100 < r["one_way_ns_median"] < 20000, r
    print("local notify->wait one-way ns:", r)


def test_decode_layer_tied_rows_fall_back_to_the_merge():
    """Rows whose scores tie heavily (all gate weights zero: every score is +0; and a row of few distinct
    values) overflow the exact selection's key slots; the chunk tasks then hand candidates to the merge
    task, which picks by (score descending, id ascending) like the oracle.  A normal row in the same
    batch is still published by the chunk tasks."""
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from oracle import dsa_oracle as orc

    B, S, K, bpc, P, H, DQK = 3, 8192, 1024, 32, 64, 128, 576
    case = indexer_case(B, S, P, "nvfp4", seed=21)
    case["w"][0] = 0.0                        # row 0: every score is exactly 0
    case["w"][1, 1:] = 0.0                    # row 1: one head only: few distinct values, many ties
    g = torch.Generator().manual_seed(22)
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S, S - 7, S - 64], dtype=torch.int32)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=64)
    assert layer.row_exact
    d = lambda t: t.to(DEV)
    layer.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), d(case["q"]), d(case["w"]), d(q_mla), d(kv)))
    for _ in range(2):
        layer.step()
        torch.cuda.synchronize()
        layer.check_status()
    data, sf = orc.split_index_pages(case["fused"], "nvfp4", P)
    kd_all = orc.dequant_fp4(data, sf, "nvfp4").reshape(-1, P, 128)
    for b in range(B):
        kd = kd_all[case["bt"][b].long()].reshape(S, 128)
        n = int(layer.sel_c[b])
        got = torch.sort(layer.sel_i[b, :n].cpu()).values
        assert n == K and got.unique().numel() == K and int(got.max()) < int(seq[b])
        if b == 0:
            assert got.tolist() == list(range(K))      # all tied: the lowest ids win
        else:
            sel, _, _ = orc.decode_step_ref(case["q_deq"][b], case["w"][b], kd, q_mla[b, 0].float(),
                                            kv[b * S:(b + 1) * S, 0].float(), int(seq[b]), K, 1 / math.sqrt(DQK))
            # the kernel's logits differ from the oracle's in the last fp32 bits, so near-ties may break differently:
            # every selected score must still reach the oracle's k-th score
            lg = ((case["q_deq"][b] @ kd[: int(seq[b])].T).clamp(min=0) * case["w"][b][:, None]).sum(dim=0)
            kth = float(torch.topk(lg, K).values[-1])
            assert float(lg[got.long()].min()) >= kth - 1e-4 * abs(kth) - 1e-6, (b, float(lg[got.long()].min()), kth)
            if b == 2:
                assert len(set(got.tolist()) & set(sel.tolist())) / K >= 0.999
        o, l = orc.attend_selected_ref(q_mla[b, 0].float(), kv[b * S:(b + 1) * S, 0].float(), layer.sel_i[b, :n].cpu(),
                                       1 / math.sqrt(DQK))
        assert (layer.out[b].cpu() - o).abs().max() < 2e-2
        assert (layer.out_lse[b].cpu() - l).abs().max() < 1e-3


def test_step_from_host_copies_the_attention_query_behind_the_launch():
    """The step's query block comes from pinned host memory: the indexer part ahead of the launch, the attention
    query on a second stream while the step already runs.  Four steps with a different query each; every
    step's output must belong to ITS query (a task that read the query before it landed would show the
    previous step's), against the oracle for the last one."""
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from oracle import dsa_oracle as orc

    B, S, K, bpc, P, H, DQK = 3, 8192, 1024, 32, 64, 128, 576
    case = indexer_case(B, S, P, "nvfp4", seed=41)
    g = torch.Generator().manual_seed(42)
    kv = (torch.randn(B * S, 1, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S, S - 9, S - 200], dtype=torch.int32)
    layer = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=64, distribute_q=True, host_query=True)
    d = lambda t: t.to(DEV)
    layer.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), None, None, None, d(kv)))
    hblock = torch.zeros(layer.q_stage.numel(), dtype=torch.uint8).pin_memory()
    nq, nw = B * 64 * 128 * 2, B * 64 * 4
    hblock[:nq].view(torch.bfloat16).copy_(case["q"].reshape(-1))
    hblock[nq:nq + nw].view(torch.float32).copy_(case["w"].reshape(-1))
    h_out = torch.zeros(B, H, 512, dtype=torch.float32).pin_memory()
    outs, qs = [], []
    for step in range(4):
        q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
        hblock[nq + nw:].view(torch.bfloat16).copy_(q_mla.reshape(-1))
        layer.step_from_host(hblock, h_out)
        torch.cuda.current_stream().synchronize()
        layer.check_status()
        outs.append(h_out.clone())
        qs.append(q_mla)
    assert all(not torch.equal(outs[i], outs[i + 1]) for i in range(3))
    for b in range(B):
        n = int(layer.sel_c[b])
        for step in (2, 3):   # the selection is the same every step (same indexer query); the attention follows q_mla
            o, _ = orc.attend_selected_ref(qs[step][b, 0].float(), kv[b * S:(b + 1) * S, 0].float(), layer.sel_i[b, :n].cpu(),
                                           1 / math.sqrt(DQK))
            assert (outs[step][b] - o).abs().max() < 2e-2, (b, step)
    # the plain sequence (block in, launch, rows out) captured once and replayed with a new query
    plain = DsaDecodeLayer(B, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, kv_seq_stride=S,
                           out_dtype=torch.float32, n_ctas=64, distribute_q=True)
    plain.bind(LayerInputs(d(case["fused"]), d(case["bt"]), d(seq), None, None, None, d(kv)))
    plain.step_from_host(hblock, h_out)
    torch.cuda.synchronize()
    assert (h_out - outs[3]).abs().max() < 1e-5      # same inputs as the last step above
    graph = plain.capture_host_step(hblock, h_out)
    q_new = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    hblock[nq + nw:].view(torch.bfloat16).copy_(q_new.reshape(-1))
    graph.replay()
    torch.cuda.synchronize()
    plain.check_status()
    for b in range(B):
        n = int(plain.sel_c[b])
        o, _ = orc.attend_selected_ref(q_new[b, 0].float(), kv[b * S:(b + 1) * S, 0].float(), plain.sel_i[b, :n].cpu(),
                                       1 / math.sqrt(DQK))
        assert (h_out[b] - o).abs().max() < 2e-2, b
