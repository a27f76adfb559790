"""Multi-GPU worker (torchrun, one process per GPU): chunked prefill of one
sequence at cp = world size; every query token of the chunk against the CPU
oracle's decode step at that token's causal length, on the owner rank."""

import math
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    from mega_dsa_cp_b200.prefill import DsaPrefillChunk
    from oracle import dsa_oracle as orc

    S, K, P, H, DQK, Tq, tile = 8192, 512, 64, 128, 576, 16, 8
    S_loc, pages = S // world, S // world // P
    g = torch.Generator().manual_seed(321)
    kraw = torch.randn(S, 128, generator=g)
    q_idx = torch.randn(Tq, 64, 128, generator=g).bfloat16()
    w_idx = torch.randn(Tq, 64, generator=g) / 64.0
    q_mla = (torch.randn(Tq, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(S, DQK, generator=g) * 0.5).bfloat16()
    pos = torch.arange(S - Tq, S)
    pos[0], pos[1] = world + 1, K * world // 2 + 3          # two short prefixes (fewer tokens than top-k)
    fused, _ = orc.build_index_pages(kraw[rank::world].contiguous(), "nvfp4", P)
    bt_row = torch.randperm(pages, generator=torch.Generator().manual_seed(5)).to(torch.int32)
    fused = fused[torch.argsort(bt_row.long())]              # page table row = a permutation of the pool
    kv_loc = kv[rank::world].reshape(S_loc, 1, DQK).contiguous()
    d = lambda t: t.to(dev)
    pf = DsaPrefillChunk(tile, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                         out_dtype=torch.float32, n_ctas=64, group_name=dist.group.WORLD.group_name, device=dev)
    pf.bind(d(fused), d(bt_row), d(kv_loc))
    out = torch.zeros(Tq // world, H, 512, device=dev)
    lse = torch.zeros(Tq // world, H, device=dev)
    sel_i = torch.zeros(Tq, K, dtype=torch.int32, device=dev)
    sel_c = torch.zeros(Tq, dtype=torch.int32, device=dev)
    dist.barrier()
    pf.run(d(q_idx), d(w_idx), d(q_mla), pos, out, lse, sel_i, sel_c)
    torch.cuda.synchronize()
    pf.check_status()
    dist.barrier()
    pk, sf = orc.quant_nvfp4(kraw)
    kd = orc.dequant_fp4(pk, sf, "nvfp4")
    scale = 1 / math.sqrt(DQK)
    ok, worst_o, worst_l = True, 0.0, 0.0
    for j in range(Tq):
        if j % world != rank:
            continue
        n_ctx = int(pos[j]) + 1
        sel, _, _ = orc.decode_step_ref(q_idx[j].float(), w_idx[j], kd, q_mla[j, 0].float(), kv.float(), n_ctx, K,
                                        scale, cp=world)
        n = int(sel_c[j])
        got = sel_i[j, :n].cpu()
        overlap = len(set(got.tolist()) & set(sel.tolist())) / max(1, sel.numel())
        good = n == sel.numel() and overlap >= 0.999 and int(got.max()) < n_ctx
        o, l = orc.attend_selected_ref(q_mla[j, 0].float(), kv.float(), got, scale, cp=world)
        d_o = float((out[j // world].cpu() - o).abs().max())
        d_l = float((lse[j // world].cpu() - l).abs().max())
        worst_o, worst_l = max(worst_o, d_o), max(worst_l, d_l)
        good &= d_o < 2e-2 and d_l < 1e-3
        if not good:
            print(f"[rank {rank}] query {j}: n {n}/{sel.numel()} overlap {overlap:.4f} d_o {d_o:.3e} d_l {d_l:.3e}", flush=True)
        ok &= good
    ref_sel = sel_i.clone()
    dist.broadcast(ref_sel, 0)
    ok &= bool(torch.equal(ref_sel, sel_i))
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    worst = torch.tensor([worst_o, worst_l], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(("MP_PREFILL_OK" if flag.item() == 1 else "MP_PREFILL_FAIL") +
              f" world={world} max_abs_o={worst[0].item():.3e} max_abs_lse={worst[1].item():.3e}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
