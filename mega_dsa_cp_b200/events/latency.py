"""Notify -> wait latency of the event layer, measured on the device (the CUDA counterpart of the
reference's tests/bench_notify_latency.py): a ping-pong over two event cells, one-way = round trip / 2."""

from __future__ import annotations

import torch

from .. import _native as N
from .symm import alloc_event_buffer


def _launch(ev, role, peer, rounds, base, out, status, budget_ns):
    p = N.PingpongParams()
    p.events = N.EventSetC(ev.tensor.data_ptr(), ev.offsets.data_ptr(), ev.rank, ev.world_size)
    p.role, p.peer, p.ev_ping, p.ev_pong, p.rounds = role, peer, 0, 1, rounds
    p.base, p.wait_budget_ns, p.out_ns, p.status = base, budget_ns, N.ptr(out), N.ptr(status)
    N.call("mdc_test_pingpong_launch", p, None)


def _summary(out, rounds):
    rtt = out[:rounds].double().cpu()
    rtt = rtt[rounds // 10:]          # the first rounds include the start-up skew of the two sides
    return {"one_way_ns_median": float(rtt.median()) / 2, "one_way_ns_mean": float(rtt.mean()) / 2,
            "one_way_ns_min": float(rtt.min()) / 2, "satisfied_wait_ns": float(out[rounds]), "rounds": int(rtt.numel())}


def local_notify_latency(device="cuda", rounds: int = 2000, budget_ns: int = 200_000_000) -> dict:
    """Block-to-block on one GPU: both sides run as two blocks of one launch."""
    ev = alloc_event_buffer(2, device=device)
    out = torch.zeros(rounds + 1, dtype=torch.int64, device=device)
    status = torch.zeros(8, dtype=torch.int32, device=device)
    _launch(ev, 2, 0, rounds, 0, out, status, budget_ns)
    torch.cuda.synchronize()
    if status[0].item() != 0:
        raise N.MdcError(f"ping-pong gave up: {status.tolist()}")
    return _summary(out, rounds)


def cross_gpu_notify_latency(rank: int, world: int, group_name: str, device, rounds: int = 2000,
                             budget_ns: int = 2_000_000_000) -> dict | None:
    """Rank 0 pings rank 1 over NVLink (system-scope reduction into the peer's cell, poll of the own cell);
    every rank of the group must call this (the cells are a symmetric allocation).  Returns the summary
    on rank 0, None elsewhere."""
    import torch.distributed as dist

    ev = alloc_event_buffer(2, rank, world, group_name, device)
    out = torch.zeros(rounds + 1, dtype=torch.int64, device=device)
    status = torch.zeros(8, dtype=torch.int32, device=device)
    dist.barrier()
    if rank < 2:
        _launch(ev, rank, 1 - rank, rounds, 0, out if rank == 0 else None, status, budget_ns)
    torch.cuda.synchronize()
    dist.barrier()
    if status[0].item() != 0:
        raise N.MdcError(f"ping-pong gave up on rank {rank}: {status.tolist()}")
    return _summary(out, rounds) if rank == 0 else None
