"""Host-side task-graph code (validator, schedule generator, arena layout)
against the reference's outputs stored in tests/golden/schedule.json."""

import random

import pytest

from conftest import load_json
from mega_dsa_cp.events import (SCOPE_LOCAL, SCOPE_SYS, EventSpec, NotifyEdge, TaskSpec, WaitEdge, validate)
from mega_dsa_cp.schedule.codegen import OP_END, codegen_schedule, pack_header, pack_queues, unpack_header
from mega_dsa_cp_b200.comm.buffers import layout_regions


def _dag(d):
    events = [EventSpec(n, s) for n, s in d["events"]]
    tasks = [TaskSpec(t["name"], t["rank"], tuple(WaitEdge(w) for w in t["waits"]),
                      tuple(NotifyEdge(e, r) for e, r in t["notifies"]), tuple(t["coords"]))
             for t in d["tasks"]]
    return tasks, events


def test_codegen_matches_reference_word_for_word():
    g = load_json("schedule")
    assert len(g["cases"]) >= 8
    for case in g["cases"]:
        tasks, events = _dag(case["dag"])
        errors, table = validate(tasks, events, case["world"])
        assert errors == [] and case["errors"] == []
        assert sorted([k[0], k[1], v] for k, v in table.arities.items()) == case["arities"]
        s = codegen_schedule(tasks, events, rank=case["rank"], n_ctas=case["n_ctas"], world_size=case["world"],
                             op_of=case["op_of"], extent_of=case["extent_of"])
        assert s.queues == case["queues"]
        assert s.arity == case["arity"] and s.scopes == case["scopes"]
        assert s.topo == case["topo"] and s.op_of == case["op_list"] and s.n_events == case["n_events"]


def test_validator_accepts_and_rejects_like_the_reference():
    g = load_json("schedule")
    for name, f in g["faults"].items():
        tasks, events = _dag(f["dag"])
        errors, _ = validate(tasks, events, f["world"])
        assert bool(errors) == bool(f["errors"]), (name, errors)


def _random_dag(seed, n_tasks, edge_prob, world=1):
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
                              tuple(NotifyEdge(f"e{j}", 0) for j in range(n_tasks) if t in preds[j])))
    return tasks, events, preds


def _parse(words):
    out, i = [], 0
    while True:
        op, nw, nn, ext = unpack_header(words[i])
        if op == OP_END:
            return out
        out.append((op, words[i + 1], words[i + 4:i + 4 + nw], words[i + 4 + nw:i + 4 + nw + nn], ext))
        i += 4 + nw + nn


@pytest.mark.parametrize("seed", range(10))
def test_random_dags_every_task_once_and_block_order_topological(seed):
    tasks, events, preds = _random_dag(seed, 150, 0.03)
    errors, table = validate(tasks, events, 1)
    assert errors == []
    for ev in events:
        assert table.arities[(ev.name, 0)] == len(preds[int(ev.name[1:])])
    s = codegen_schedule(tasks, events, rank=0, n_ctas=7, op_of={t.name: 1 + i % 3 for i, t in enumerate(tasks)},
                         extent_of={tasks[0].name: 1})
    placed = []
    ev_id = {ev.name: i for i, ev in enumerate(events)}
    for q in s.queues:
        entries = _parse(q)
        where = {e[1]: k for k, e in enumerate(entries)}
        placed += list(where)
        for t, ps in preds.items():
            for p in ps:
                if t in where and p in where:
                    assert where[p] < where[t]
        for op, c0, waits, notifies, ext in entries:
            t = tasks[c0]
            assert waits == [ev_id[w.event] for w in t.waits]
            assert notifies == [ev_id[n.event] << 8 | n.dst_rank for n in t.notifies]
            assert op == 1 + c0 % 3
    assert sorted(placed) == list(range(150))
    flat, row = pack_queues(s)
    assert len(flat) == 7 * row and flat[row - 1] & 0xFF == OP_END


def test_two_rank_filtering_and_symmetric_tables():
    tasks = [TaskSpec("a", 0, notifies=(NotifyEdge("e", 1),)),
             TaskSpec("b", 1, waits=(WaitEdge("e"),), notifies=(NotifyEdge("f", 0),)),
             TaskSpec("c", 0, waits=(WaitEdge("f"),))]
    events = [EventSpec("e", SCOPE_SYS), EventSpec("f", SCOPE_SYS)]
    s0 = codegen_schedule(tasks, events, rank=0, n_ctas=2, world_size=2)
    s1 = codegen_schedule(tasks, events, rank=1, n_ctas=2, world_size=2)
    assert sorted(e[1] for q in s0.queues for e in _parse(q)) == [0, 2]
    assert [e[1] for q in s1.queues for e in _parse(q)] == [1]
    assert s0.arity == [0, 1] and s1.arity == [1, 0]
    with pytest.raises(ValueError):
        codegen_schedule([TaskSpec("a", 0, waits=(WaitEdge("nope"),))], [], rank=0, n_ctas=1)


def test_header_and_arena_layout():
    assert unpack_header(pack_header(7, 3, 63, 255)) == (7, 3, 63, 255)
    offs, per_phase = layout_regions({"cand": 1000, "inbox": 256, "stats": 7696})
    assert offs == {"cand": 0, "inbox": 1024, "stats": 1280} and per_phase == 1280 + 7936
