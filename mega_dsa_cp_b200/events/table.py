"""Task-graph metadata shared by the validator, the schedule generator and the
runners: events (one counter cell per rank), wait / notify edges and tasks.

An event owns one u64 cell on every rank.  A task always waits on the cell of
its own rank; a notify edge names the rank whose cell it bumps.  The number of
notify edges that target a cell is the cell's per-phase arity: a consumer in
phase p (0-based) waits until the cell holds arity * (p + 1).  Cells only grow,
nothing is ever reset, so a captured launch can be replayed with only the phase
scalar advanced.

Mirrors mega_dsa_cp/events/table.py of the reference (same names and fields).
Plain Python, no torch import: usable without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Tuple

SCOPE_LOCAL = "local"  # producers and consumers all live on one rank (gpu-scope ordering)
SCOPE_SYS = "sys"      # at least one notify crosses ranks (system-scope ordering)


@dataclass(frozen=True)
class EventSpec:
    name: str
    scope: str


@dataclass(frozen=True)
class WaitEdge:
    event: str


@dataclass(frozen=True)
class NotifyEdge:
    event: str
    dst_rank: int


@dataclass(frozen=True)
class TaskSpec:
    name: str
    rank: int
    waits: Tuple[WaitEdge, ...] = ()
    notifies: Tuple[NotifyEdge, ...] = ()
    # (c0, c1, c2) handed to the tile; empty = (index of the task in the list, 0, 0)
    coords: Tuple[int, ...] = ()


@dataclass
class EventTable:
    """Result of validation: the events by name and the arity of every cell."""

    events: Dict[str, EventSpec] = field(default_factory=dict)
    arities: Dict[Tuple[str, int], int] = field(default_factory=dict)

    def event_id(self, name: str) -> int:
        for i, key in enumerate(self.events):
            if key == name:
                return i
        raise KeyError(name)
