"""Static checks of a task graph, run on the host before anything is launched.

`validate(tasks, events, world_size)` returns `(errors, EventTable)`; an empty
error list means the graph can be scheduled.  It rejects, with one message
each: duplicate names, ranks out of range, references to undeclared events,
a local-scope event notified across ranks, a cell that is waited on but never
notified (a certain deadlock) or notified but never waited on, a sys-scope
event that never crosses ranks, a local event whose per-rank use is one-sided,
and dependency cycles.

Behaviourally equivalent to mega_dsa_cp/events/validator.py:29-142 of the
reference (same accept / reject decisions and the same arity table).
"""

from __future__ import annotations

from collections import defaultdict, deque
from typing import List, Tuple

from .table import SCOPE_LOCAL, SCOPE_SYS, EventTable


def _has_cycle(tasks, producers_of) -> bool:
    """Kahn's algorithm on task -> task edges induced by (producer, consumer) pairs."""
    index = {t.name: i for i, t in enumerate(tasks)}
    succ = defaultdict(list)
    indeg = [0] * len(tasks)
    for t in tasks:
        for w in t.waits:
            for p in producers_of.get(w.event, ()):
                if p != t.name:
                    succ[index[p]].append(index[t.name])
                    indeg[index[t.name]] += 1
    ready = deque(i for i, d in enumerate(indeg) if d == 0)
    done = 0
    while ready:
        i = ready.popleft()
        done += 1
        for j in succ[i]:
            indeg[j] -= 1
            if indeg[j] == 0:
                ready.append(j)
    return done != len(tasks)


def validate(tasks: list, events: list, world_size: int) -> Tuple[List[str], EventTable]:
    errors: List[str] = []
    by_name = {}
    for ev in events:
        if ev.name in by_name:
            errors.append(f"event {ev.name!r} is declared twice")
        by_name[ev.name] = ev
        if ev.scope not in (SCOPE_LOCAL, SCOPE_SYS):
            errors.append(f"event {ev.name!r} has unknown scope {ev.scope!r}")

    seen_tasks = set()
    for t in tasks:
        if t.name in seen_tasks:
            errors.append(f"task {t.name!r} is declared twice")
        seen_tasks.add(t.name)
        if not 0 <= t.rank < world_size:
            errors.append(f"task {t.name!r} runs on rank {t.rank}, outside 0..{world_size - 1}")

    arity = {}                       # (event, rank of the cell) -> notifies per phase
    waited = set()                   # (event, rank of the cell)
    producers_of = defaultdict(set)  # event -> task names that notify it
    prod_ranks = defaultdict(set)
    cons_ranks = defaultdict(set)
    dst_ranks = defaultdict(set)
    self_notified = defaultdict(set)  # event -> ranks that notify their own cell
    for t in tasks:
        for w in t.waits:
            if w.event not in by_name:
                errors.append(f"task {t.name!r} waits on undeclared event {w.event!r}")
                continue
            waited.add((w.event, t.rank))
            cons_ranks[w.event].add(t.rank)
        for n in t.notifies:
            if n.event not in by_name:
                errors.append(f"task {t.name!r} notifies undeclared event {n.event!r}")
                continue
            producers_of[n.event].add(t.name)
            prod_ranks[n.event].add(t.rank)
            if not 0 <= n.dst_rank < world_size:
                errors.append(f"task {t.name!r} notifies {n.event!r} on rank {n.dst_rank}, outside the world")
                continue
            dst_ranks[n.event].add(n.dst_rank)
            if by_name[n.event].scope == SCOPE_LOCAL and n.dst_rank != t.rank:
                errors.append(f"task {t.name!r} notifies local event {n.event!r} on another rank ({n.dst_rank})")
            if n.dst_rank == t.rank:
                self_notified[n.event].add(t.rank)
            arity[(n.event, n.dst_rank)] = arity.get((n.event, n.dst_rank), 0) + 1

    for cell in sorted(waited - set(arity)):
        errors.append(f"event {cell[0]!r} is waited on rank {cell[1]} but nothing notifies that cell: deadlock")
    for cell in sorted(set(arity) - waited):
        errors.append(f"event {cell[0]!r} is notified on rank {cell[1]} but nothing waits there")

    for ev in events:
        name = ev.name
        if ev.scope == SCOPE_SYS and world_size > 1:
            if not any(r != d for r in prod_ranks[name] for d in dst_ranks[name]):
                errors.append(f"event {name!r} is declared sys but no notify crosses ranks")
        if ev.scope == SCOPE_LOCAL and len(prod_ranks[name] | cons_ranks[name]) > 1:
            # a local event used on several ranks must be produced and consumed rank by rank
            for r in sorted(prod_ranks[name] | cons_ranks[name]):
                if (r in self_notified[name]) != (r in cons_ranks[name]):
                    errors.append(f"local event {name!r} is produced or consumed one-sidedly on rank {r}")

    if _has_cycle(tasks, producers_of):
        errors.append("the task graph has a dependency cycle")
    return errors, EventTable(events=by_name, arities=arity)
