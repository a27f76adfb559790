"""Two or more GPUs (torchrun, one process per GPU): the event, comm and scheduler layers by themselves,
after the reference's dual-GPU tests -- ping-pong, fan-in and fan-out with a payload that travels by bulk
push and is checked behind a flag-only wait (tests/test_events_dual_gpu.py:53-99,
tests/test_comm_dual_gpu.py:70-157), driven through per-rank task queues over many phases
(tests/test_scheduler_dual_gpu.py:42-59,153-168) -- and the cross-GPU notify latency."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def build_dag(world, n_pairs, N):
    from mega_dsa_cp_b200.events import SCOPE_LOCAL, SCOPE_SYS, EventSpec, NotifyEdge, TaskSpec, WaitEdge

    events, tasks, ops = [], [], {}
    slot = 0
    # ping-pong: src pushes slot s to dst, dst verifies behind the flag and answers, src logs the answer
    for s in range(n_pairs):
        src, dst = s % world, (s + 1) % world
        events += [EventSpec(f"ping{s}", SCOPE_SYS), EventSpec(f"pong{s}", SCOPE_SYS)]
        tasks.append(TaskSpec(f"push{s}", src, (), (NotifyEdge(f"ping{s}", dst),), (s, dst, slot)))
        tasks.append(TaskSpec(f"check{s}", dst, (WaitEdge(f"ping{s}"),), (NotifyEdge(f"pong{s}", src),), (s, src, slot)))
        tasks.append(TaskSpec(f"ack{s}", src, (WaitEdge(f"pong{s}"),), (), (1000 + s, 0, 0)))
        ops[f"push{s}"], ops[f"check{s}"], ops[f"ack{s}"] = N.OP_PUSH, N.OP_VERIFY, N.OP_LOG
        slot += 1
    # fan-in: every rank pushes into rank 0 and bumps one event of arity `world`; rank 0 verifies all
    events.append(EventSpec("fanin", SCOPE_SYS))
    for r in range(world):
        tasks.append(TaskSpec(f"in_push{r}", r, (), (NotifyEdge("fanin", 0),), (0, 0, slot)))
        tasks.append(TaskSpec(f"in_check{r}", 0, (WaitEdge("fanin"),), (), (0, r, slot)))
        ops[f"in_push{r}"], ops[f"in_check{r}"] = N.OP_PUSH, N.OP_VERIFY
    slot += 1
    # fan-out: rank 0 pushes to every rank, each verifies its copy
    for d in range(world):
        events.append(EventSpec(f"fanout{d}", SCOPE_SYS if d != 0 else SCOPE_LOCAL))   # rank 0 -> itself stays local
        tasks.append(TaskSpec(f"out_push{d}", 0, (), (NotifyEdge(f"fanout{d}", d),), (0, d, slot)))
        tasks.append(TaskSpec(f"out_check{d}", d, (WaitEdge(f"fanout{d}"),), (), (0, 0, slot)))
        ops[f"out_push{d}"], ops[f"out_check{d}"] = N.OP_PUSH, N.OP_VERIFY
    slot += 1
    return tasks, events, ops, slot


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from mega_dsa_cp_b200 import _native as N
    from mega_dsa_cp_b200.comm.buffers import alloc_arena
    from mega_dsa_cp_b200.events.latency import cross_gpu_notify_latency, local_notify_latency
    from mega_dsa_cp_b200.events.symm import alloc_event_buffer
    from mega_dsa_cp_b200.schedule.codegen import codegen_schedule
    from mega_dsa_cp_b200.schedule.device import launch_megakernel, upload_schedule

    group = dist.group.WORLD.group_name
    n_pairs, nbytes, phases = 40, 4096, 25          # 25 launches x 40 ping-pong hand-offs = 1000 payload chains
    tasks, events, ops, n_slots = build_dag(world, n_pairs, N)
    sched = codegen_schedule(tasks, events, rank=rank, n_ctas=8, world_size=world, op_of=ops)
    ds = upload_schedule(sched, dev)
    ev = alloc_event_buffer(len(events), rank, world, group, dev)
    arena = alloc_arena({"test": n_slots * world * nbytes}, 1, rank, world, group, dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    mine = sum(1 for t in tasks if t.rank == rank and ops[t.name] == N.OP_LOG)
    ok = True
    dist.barrier()
    for phase in range(phases):
        log = torch.zeros(256, dtype=torch.int32, device=dev)
        ds.scalars[0] = phase
        launch_megakernel(ds, ev, arena, status, log=log, test_off=arena.region_off("test"), test_slot_bytes=nbytes,
                          wait_budget_ns=5_000_000_000)
        torch.cuda.synchronize()
        ok &= status[0].item() == 0 and int(log[0]) == mine
        dist.barrier()          # a slot is rewritten in the next phase only after every rank has verified it
    if status[0].item() != 0:
        print(f"[rank {rank}] status {status.tolist()}", flush=True)
    lat = cross_gpu_notify_latency(rank, world, group, dev)
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        loc = local_notify_latency(dev)
        print(("MP_EVENTS_OK" if flag.item() == 1 else "MP_EVENTS_FAIL") +
              f" world={world} cross_gpu_one_way_ns={lat['one_way_ns_median']:.0f} local_one_way_ns={loc['one_way_ns_median']:.0f}"
              f" satisfied_wait_ns={lat['satisfied_wait_ns']:.0f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
