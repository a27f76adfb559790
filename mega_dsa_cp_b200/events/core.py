"""Event cells: layout constants and the host view of the device-side event set.

Device code lives in csrc/events.cuh (`mdc::EventSet`: cell / peer_cell /
notify / wait with a bounded poll).  This module keeps what the host needs: the
cell geometry (mega_dsa_cp/events/core.py:31-37 of the reference) and a plain
descriptor that marshals an event buffer into the C ABI.
"""

from __future__ import annotations

from dataclasses import dataclass

CELL_BYTES = 128            # one u64 counter per 128-byte line: no cell shares a line with another writer
CELL_ELEMS = CELL_BYTES // 8

SCOPE_LOCAL = "gpu"
SCOPE_SYS = "sys"

DEFAULT_BACKOFF_NS = 64


@dataclass(frozen=True)
class EventSet:
    """What a kernel needs to reach every rank's cells: the local base address,
    the device table of byte offsets to each peer's base, and this rank."""

    base: int       # device address of the local cells
    offsets: int    # device address of int64[world_size]: peer base - local base
    my_rank: int
    world_size: int = 1

    def cell_addr(self, event_id: int) -> int:
        return self.base + event_id * CELL_BYTES
