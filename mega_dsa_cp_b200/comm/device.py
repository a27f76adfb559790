"""Host view of the byte-addressed peer buffer the kernels receive.

Device code lives in csrc/comm.cuh (`mdc::PeerBuffer`: local_addr / peer_addr,
bulk push start / finish).  Mirrors mega_dsa_cp/comm/device.py:11-44 of the
reference.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class PeerBuffer:
    base: int        # device address of the local arena
    offsets: int     # device address of int64[world_size]: peer base - local base
    my_rank: int
    mc_base: int = 0  # NVLS multicast base, 0 when unavailable
    world_size: int = 1

    def local_addr(self, byte_off: int) -> int:
        return self.base + byte_off

    def has_mc(self) -> bool:
        return self.mc_base != 0
