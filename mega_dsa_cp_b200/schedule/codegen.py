"""Turns a validated multi-rank task graph into this rank's per-block queues.

Queue format (int32 words, one stream per thread block):

    [header][c0][c1][c2][wait event id]*[notify word]*   ...   [end header]
    header      = op | n_waits << 8 | n_notifies << 14 | extent_src << 20
    notify word = event id << 8 | destination rank
    end header  = OP_END with zero counts

Tasks are dealt round-robin to the blocks in one global topological order, so
each block's stream is itself topologically ordered and the static schedule
cannot deadlock as long as all blocks are co-resident.  Every rank runs this
with the same inputs and gets the same event ids, arities and scopes.

Word-for-word compatible with mega_dsa_cp/schedule/codegen.py:23-128 of the
reference (same queue words for the same graph).
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import List

from ..events.validator import validate

OP_END = 0xFF
MAX_EDGES_PER_TASK = 63   # 6-bit counts in the header
MAX_EXTENT_SRC = 255      # 8-bit scalar index in the header


@dataclass
class Schedule:
    queues: List[List[int]]  # per block, including the end header
    arity: List[int]         # per event id: notifies per phase into THIS rank's cell
    scopes: List[int]        # per event id: 0 local, 1 sys
    topo: List[int]          # this rank's task indices in execution order
    op_of: List[int]         # per task index: op code
    n_events: int


def pack_header(op: int, n_waits: int, n_notifies: int, extent_src: int) -> int:
    return (op & 0xFF) | (n_waits & 0x3F) << 8 | (n_notifies & 0x3F) << 14 | (extent_src & 0xFF) << 20


def unpack_header(word: int):
    return word & 0xFF, (word >> 8) & 0x3F, (word >> 14) & 0x3F, (word >> 20) & 0xFF


def topo_sort(tasks: list, events: list) -> List[int]:
    """Kahn order with first-in-first-out ties: sources in list order, and the
    consumers of a finished task in list order."""
    producers = {}
    for i, t in enumerate(tasks):
        for n in t.notifies:
            producers.setdefault(n.event, set()).add(i)
    succ = [[] for _ in tasks]
    indeg = [0] * len(tasks)
    for j, t in enumerate(tasks):
        for w in t.waits:
            for i in producers.get(w.event, ()):
                if i != j:
                    succ[i].append(j)
                    indeg[j] += 1
    ready = deque(i for i, d in enumerate(indeg) if d == 0)
    order = []
    while ready:
        i = ready.popleft()
        order.append(i)
        for j in succ[i]:
            indeg[j] -= 1
            if indeg[j] == 0:
                ready.append(j)
    if len(order) != len(tasks):
        raise ValueError("dependency cycle in the task graph")
    return order


def codegen_schedule(tasks: list, events: list, rank: int, n_ctas: int, world_size: int = 1,
                     op_of: dict = None, extent_of: dict = None) -> Schedule:
    """`tasks` / `events` describe ALL ranks; only tasks of `rank` are queued.
    op_of / extent_of map task name -> op code / index of the dynamic-extent
    scalar (0 = none)."""
    errors, table = validate(tasks, events, world_size=world_size)
    if errors:
        raise ValueError(f"invalid DAG: {errors}")
    op_of = op_of or {}
    extent_of = extent_of or {}
    event_id = {ev.name: i for i, ev in enumerate(events)}

    mine = [i for i in topo_sort(tasks, events) if tasks[i].rank == rank]
    queues: List[List[int]] = [[] for _ in range(n_ctas)]
    for slot, i in enumerate(mine):
        t = tasks[i]
        if len(t.waits) > MAX_EDGES_PER_TASK or len(t.notifies) > MAX_EDGES_PER_TASK:
            raise AssertionError(f"task {t.name}: more than {MAX_EDGES_PER_TASK} edges of one kind")
        extent = extent_of.get(t.name, 0)
        if not 0 <= extent <= MAX_EXTENT_SRC:
            raise AssertionError(f"task {t.name}: extent scalar {extent} out of range")
        coords = tuple(t.coords) if t.coords else (i, 0, 0)
        words = [pack_header(op_of.get(t.name, 0), len(t.waits), len(t.notifies), extent), *coords]
        words += [event_id[w.event] for w in t.waits]
        words += [event_id[n.event] << 8 | n.dst_rank for n in t.notifies]
        queues[slot % n_ctas] += words
    for q in queues:
        q.append(pack_header(OP_END, 0, 0, 0))
    return Schedule(
        queues=queues,
        arity=[table.arities.get((ev.name, rank), 0) for ev in events],
        scopes=[0 if ev.scope == "local" else 1 for ev in events],
        topo=mine,
        op_of=[op_of.get(t.name, 0) for t in tasks],
        n_events=len(events),
    )


def pack_queues(schedule: Schedule):
    """Pads the per-block streams to one row length.  Returns (flat list of
    n_ctas * row_words int32 words, row_words)."""
    row = max(len(q) for q in schedule.queues)
    flat = []
    end = pack_header(OP_END, 0, 0, 0)
    for q in schedule.queues:
        flat += q + [end] * (row - len(q))
    return flat, row
