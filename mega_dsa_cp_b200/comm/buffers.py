"""Symmetric payload arena: named regions, rotated by phase.

One symmetric allocation holds `phases` copies of the same region layout:

    [phase 0: region A | region B | ...][phase 1: region A | region B | ...]

Every rank allocates the identical layout, so one table of per-rank byte
offsets (peer base - local base) maps any local byte offset to any peer, the
same translation the event cells use.  Regions start on 256-byte boundaries.
Same contract as mega_dsa_cp/comm/buffers.py:40-77 of the reference.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..events.symm import symmetric_empty
from .device import PeerBuffer

REGION_ALIGN = 256


@dataclass
class SymmetricArena:
    nbytes_per_phase: int
    phases: int
    rank: int
    world_size: int
    tensor: torch.Tensor    # uint8, the local copy
    offsets: torch.Tensor   # int64[world_size] on the device
    mc_base: int            # NVLS multicast address of the arena, 0 when there is none
    handle: object
    regions: dict           # name -> byte offset inside one phase

    def region_off(self, name: str, phase: int = 0) -> int:
        return (phase % self.phases) * self.nbytes_per_phase + self.regions[name]

    @property
    def data_ptr(self) -> int:
        return self.tensor.data_ptr()

    def device_view(self) -> PeerBuffer:
        return PeerBuffer(self.tensor.data_ptr(), self.offsets.data_ptr(), self.rank, self.mc_base, self.world_size)


def layout_regions(regions: dict):
    """name -> offset for the given {name: nbytes}, plus the phase size."""
    offsets, pos = {}, 0
    for name, nbytes in regions.items():
        offsets[name] = pos
        pos += -(-nbytes // REGION_ALIGN) * REGION_ALIGN
    return offsets, pos


def alloc_arena(regions: dict, phases: int = 2, rank: int = 0, world_size: int = 1, group_name: str = "0",
                device: str = "cuda") -> SymmetricArena:
    offs, per_phase = layout_regions(regions)
    tensor, offsets, mc, handle = symmetric_empty(per_phase * phases, torch.uint8, rank, world_size, group_name, device)
    return SymmetricArena(per_phase, phases, rank, world_size, tensor, offsets, mc, handle, offs)
