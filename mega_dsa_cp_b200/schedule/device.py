"""Host side of the persistent scheduler kernel: uploads a Schedule and
launches mdc_megakernel_launch (csrc/megakernel.cu, csrc/sched.cuh).

The device loop replaces StaticScheduler / Cursor of
mega_dsa_cp/schedule/device.py:35-129 of the reference: each block walks its
queue row, waits until every wait event's local cell holds
arity * (phase + 1), runs the task's op, then posts its notifies.  `phase` is
scalars[0]; replaying a launch only needs that scalar bumped.
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _native as N
from ..comm.buffers import SymmetricArena
from ..events.symm import EventBuffer
from .codegen import Schedule, pack_queues


@dataclass
class DeviceSchedule:
    queue: torch.Tensor     # int32 (n_ctas, row_words)
    arity: torch.Tensor     # int32 (n_events,)
    scopes: torch.Tensor    # int32 (n_events,)
    scalars: torch.Tensor   # int64: [0] phase, [1:] dynamic extents
    phase_ctl: torch.Tensor  # int64 (1,): arrival counter of the device-side phase bump
    n_ctas: int
    row_words: int
    n_events: int


def upload_schedule(schedule: Schedule, device="cuda", n_scalars: int = 8) -> DeviceSchedule:
    flat, row = pack_queues(schedule)
    n_ctas = len(schedule.queues)
    i32 = lambda x: torch.tensor(x if len(x) else [0], dtype=torch.int32, device=device)
    return DeviceSchedule(
        queue=torch.tensor(flat, dtype=torch.int32, device=device).view(n_ctas, row),
        arity=i32(schedule.arity), scopes=i32(schedule.scopes),
        scalars=torch.zeros(n_scalars, dtype=torch.int64, device=device),
        phase_ctl=torch.zeros(1, dtype=torch.int64, device=device),
        n_ctas=n_ctas, row_words=row, n_events=schedule.n_events,
    )


def launch_megakernel(ds: DeviceSchedule, events: EventBuffer, arena: SymmetricArena | None, status: torch.Tensor,
                      layer: N.LayerParams | None = None, log: torch.Tensor | None = None,
                      wait_budget_ns: int = 2_000_000_000, test_off: int = 0, test_slot_bytes: int = 0,
                      stream=None, trace: torch.Tensor | None = None, device_phase: bool = False) -> None:
    """One launch of the persistent kernel on this rank (asynchronous).  `trace`: optional int64
    tensor of 4 + 4 * entries words that receives the task timeline (word 0 = entry count).
    `device_phase`: the kernel itself advances scalars[0] after every block has read it (the
    reference's device-side step counter, docs/event-system.md:32-36), so the same launch can be
    replayed, also from a captured CUDA graph, with no host write in between."""
    p = N.MegaParams()
    p.queue, p.row_words, p.n_ctas = N.ptr(ds.queue), ds.row_words, ds.n_ctas
    p.scalars, p.arity, p.scopes, p.n_events = N.ptr(ds.scalars), N.ptr(ds.arity), N.ptr(ds.scopes), ds.n_events
    p.events = N.EventSetC(events.tensor.data_ptr(), events.offsets.data_ptr(), events.rank, events.world_size)
    if arena is not None:
        p.arena = N.PeerBufferC(arena.tensor.data_ptr(), arena.offsets.data_ptr(), arena.rank, arena.world_size,
                                arena.mc_base)
    else:
        p.arena = N.PeerBufferC(None, events.offsets.data_ptr(), events.rank, events.world_size, 0)
    p.wait_budget_ns = wait_budget_ns
    p.status = N.ptr(status)
    p.log = N.ptr(log)
    p.log_cap = 0 if log is None else log.numel()
    p.test_off, p.test_slot_bytes = test_off, test_slot_bytes
    if layer is not None:
        p.layer = layer
    p.trace = N.ptr(trace)
    p.trace_cap = 0 if trace is None else (trace.numel() - 4) // 4
    p.phase_ctl = N.ptr(ds.phase_ctl) if device_phase else None
    N.call("mdc_megakernel_launch", p, stream)
