"""Allocation of event cells that every rank of a context-parallel group can
write: plain device memory for a single rank, torch symmetric memory (peer
mappings over NVLink) otherwise.

`alloc_event_buffer` must be called by all ranks with the same arguments.  It
returns the local cells plus an int64 device table `offsets[r] = base of rank r
- base of this rank`, which is all the device side needs to reach a peer's cell.
Same contract as mega_dsa_cp/events/symm.py:69-95 of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .core import CELL_BYTES, EventSet


@dataclass
class EventBuffer:
    num_events: int
    rank: int
    world_size: int
    tensor: torch.Tensor    # int64 view of the local u64 cells
    offsets: torch.Tensor   # int64[world_size] on the device
    handle: object = None   # keeps the peer mappings alive

    @property
    def data_ptr(self) -> int:
        return self.tensor.data_ptr()

    def device_view(self) -> EventSet:
        return EventSet(self.tensor.data_ptr(), self.offsets.data_ptr(), self.rank, self.world_size)


def _enable_symm_mem(group_name: str) -> None:
    """torch < 2.11 needs the group registered for symmetric memory first."""
    major, minor = (int(x) for x in torch.__version__.split(".")[:2])
    if (major, minor) >= (2, 11):
        return
    from torch.distributed._symmetric_memory import enable_symm_mem_for_group

    enable_symm_mem_for_group(group_name)


def symmetric_empty(numel: int, dtype: torch.dtype, rank: int, world_size: int, group_name: str, device):
    """(local tensor, offsets int64[world] on device, multicast address or 0, handle)."""
    if world_size == 1:
        t = torch.zeros(numel, dtype=dtype, device=device)
        return t, torch.zeros(1, dtype=torch.int64, device=device), 0, None
    import torch.distributed._symmetric_memory as symm_mem

    _enable_symm_mem(group_name)
    t = symm_mem.empty(numel, dtype=dtype, device=device)
    handle = symm_mem.rendezvous(t, group=group_name)
    bases = [handle.get_buffer(r, (numel,), dtype, storage_offset=0).data_ptr() for r in range(world_size)]
    offsets = torch.tensor([b - bases[rank] for b in bases], dtype=torch.int64, device=device)
    t.zero_()
    mc = int(getattr(handle, "multicast_ptr", 0) or 0)
    return t, offsets, mc, handle


def alloc_event_buffer(num_events: int, rank: int = 0, world_size: int = 1, group_name: str = "0",
                       device: str = "cuda") -> EventBuffer:
    numel = num_events * CELL_BYTES // 8
    tensor, offsets, _, handle = symmetric_empty(numel, torch.int64, rank, world_size, group_name, device)
    return EventBuffer(num_events, rank, world_size, tensor, offsets, handle)
