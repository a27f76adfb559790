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
    task_off: torch.Tensor | None = None   # dynamic scheduling: int32 word offset of every task in the one shared row
    dyn_ctl: torch.Tensor | None = None    # ... and its two counters (next task, finished blocks)
    n_tasks: int = 0


def task_offsets(row) -> list[int]:
    """Word offsets of the task entries of one packed queue row (format of schedule/codegen.py)."""
    offs, pos = [], 0
    while (row[pos] & 0xFF) != 0xFF:
        offs.append(pos)
        pos += 4 + ((row[pos] >> 8) & 0x3F) + ((row[pos] >> 14) & 0x3F)
    return offs


def upload_schedule(schedule: Schedule, device="cuda", n_scalars: int = 8, dynamic_ctas: int | None = None) -> DeviceSchedule:
    """dynamic_ctas: the schedule was generated for ONE queue (n_ctas = 1: all tasks of the rank in dependency
    order); the kernel runs dynamic_ctas blocks that pull tasks from it with an atomic counter."""
    flat, row = pack_queues(schedule)
    n_ctas = len(schedule.queues)
    i32 = lambda x: torch.tensor(x if len(x) else [0], dtype=torch.int32, device=device)
    dyn = {}
    if dynamic_ctas is not None:
        assert n_ctas == 1, "dynamic scheduling pulls from one shared queue: generate the schedule with n_ctas = 1"
        offs = task_offsets(flat[:row])
        dyn = dict(task_off=i32(offs), dyn_ctl=torch.zeros(2, dtype=torch.int32, device=device), n_tasks=len(offs))
        n_ctas = dynamic_ctas
    return DeviceSchedule(**dyn, 
        queue=torch.tensor(flat, dtype=torch.int32, device=device).view(len(schedule.queues), row),
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
    if ds.task_off is not None:
        p.dyn_task_off, p.dyn_n_tasks, p.dyn_ctl = N.ptr(ds.task_off), ds.n_tasks, N.ptr(ds.dyn_ctl)
    N.call("mdc_megakernel_launch", p, stream)
