"""Multi-GPU worker (launched with torchrun, one process per GPU): runs the
decode megakernel at cp = world size on a small seeded case and checks the
selection and the merged attention output against the CPU oracle."""

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
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from mega_dsa_cp_b200.layer import DsaDecodeLayer, LayerInputs
    from oracle import dsa_oracle as orc

    B, S, K, P, H, DQK = 4, 8192, 512, 64, 128, 576
    S_loc = S // world
    g = torch.Generator().manual_seed(123)
    kraw = torch.randn(B, S, 128, generator=g)
    q_idx = torch.randn(B, 64, 128, generator=g).bfloat16()
    w_idx = torch.randn(B, 64, generator=g) / 64.0
    q_mla = (torch.randn(B, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(B, S, DQK, generator=g) * 0.5).bfloat16()
    seq = torch.tensor([S - 64 * b - 3 for b in range(B)], dtype=torch.int32)
    # this rank's shard: token t -> local index t // world on rank t % world
    k_loc = kraw[:, rank::world].reshape(B * S_loc, 128)
    fused, _ = orc.build_index_pages(k_loc, "nvfp4", P)
    pages = S_loc // P
    bt = torch.arange(B * pages, dtype=torch.int32).reshape(B, pages)
    seq_loc = torch.tensor([(int(s) - rank + world - 1) // world for s in seq], dtype=torch.int32)
    kv_loc = kv[:, rank::world].reshape(B * S_loc, 1, DQK).contiguous()
    dev = torch.device("cuda", torch.cuda.current_device())
    d = lambda t: t.to(dev)
    # the query block of a sequence comes from its owner only (QPATH task: P2P stores into every rank's arena)
    layer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                           kv_seq_stride=S_loc, out_dtype=torch.float32, n_ctas=64,
                           group_name=dist.group.WORLD.group_name, device=dev, distribute_q=True)
    layer.bind(LayerInputs(d(fused), d(bt), d(seq_loc), d(q_idx[rank::world]), d(w_idx[rank::world]),
                           d(q_mla[rank::world]), d(kv_loc)))
    dist.barrier()
    for _ in range(3):
        layer.step(wait_budget_ns=5_000_000_000)
        torch.cuda.synchronize()
        layer.check_status()
        dist.barrier()
    # oracle on the dequantised global cache (quantisation is per token row, so sharding commutes with it)
    pk, sf = orc.quant_nvfp4(kraw.reshape(B * S, 128))
    kd = orc.dequant_fp4(pk, sf, "nvfp4").reshape(B, S, 128)
    ok = True
    worst_o = worst_l = 0.0
    for b in range(B):
        sel, _, _ = orc.decode_step_ref(q_idx[b].float(), w_idx[b], kd[b], q_mla[b, 0].float(), kv[b].float(),
                                        int(seq[b]), K, 1 / math.sqrt(DQK), cp=world)
        n = int(layer.sel_c[b])
        got = torch.sort(layer.sel_i[b, :n].cpu()).values
        overlap = len(set(got.tolist()) & set(sel.tolist())) / max(1, sel.numel())
        ok &= n == sel.numel() and overlap >= 0.999
        if b % world == rank:
            # always checked, on the ids the kernel selected: partial attention per rank, push to the
            # owner's inbox and the LSE merge
            o, l = orc.attend_selected_ref(q_mla[b, 0].float(), kv[b].float(), layer.sel_i[b, :n].cpu(),
                                           1 / math.sqrt(DQK), cp=world)
            d_o = float((layer.out[b // world].cpu() - o).abs().max())
            d_l = float((layer.out_lse[b // world].cpu() - l).abs().max())
            worst_o, worst_l = max(worst_o, d_o), max(worst_l, d_l)
            ok &= d_o < 2e-2 and d_l < 1e-3
    # every rank must hold the same selection bit for bit
    ref_sel = layer.sel_i.clone()
    dist.broadcast(ref_sel, 0)
    ok &= bool(torch.equal(ref_sel, layer.sel_i))
    # ---- the exact row selection across ranks (histogram exchange + undecided keys; not the default there):
    # same selection, same order, same output as the candidate-list path above
    xlayer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                            kv_seq_stride=S_loc, out_dtype=torch.float32, n_ctas=64,
                            group_name=dist.group.WORLD.group_name, device=dev, row_exact=True)
    assert xlayer.row_exact
    xlayer.bind(LayerInputs(d(fused), d(bt), d(seq_loc), d(q_idx), d(w_idx), d(q_mla), d(kv_loc)))
    dist.barrier()
    for _ in range(3):
        xlayer.step(wait_budget_ns=5_000_000_000)
        torch.cuda.synchronize()
        xlayer.check_status()
        dist.barrier()
    # ... and each rank settling its own exact list (no exchange between ranks before the cross-rank merge)
    llayer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                            kv_seq_stride=S_loc, out_dtype=torch.float32, n_ctas=64,
                            group_name=dist.group.WORLD.group_name, device=dev, row_exact="local")
    assert llayer.row_exact == 2 and not llayer.cand_direct
    llayer.bind(LayerInputs(d(fused), d(bt), d(seq_loc), d(q_idx), d(w_idx), d(q_mla), d(kv_loc)))
    dist.barrier()
    for _ in range(3):
        llayer.step(wait_budget_ns=5_000_000_000)
        torch.cuda.synchronize()
        llayer.check_status()
        dist.barrier()
    # ... and the default exchange with the blocks pulling tasks from one shared queue (dynamic scheduling)
    dlayer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                            kv_seq_stride=S_loc, out_dtype=torch.float32, n_ctas=64,
                            group_name=dist.group.WORLD.group_name, device=dev, distribute_q=True, dynamic=True)
    dlayer.bind(LayerInputs(d(fused), d(bt), d(seq_loc), d(q_idx[rank::world]), d(w_idx[rank::world]),
                            d(q_mla[rank::world]), d(kv_loc)))
    dist.barrier()
    for _ in range(3):
        dlayer.step(wait_budget_ns=5_000_000_000)
        torch.cuda.synchronize()
        dlayer.check_status()
        dist.barrier()
    for other in (xlayer, llayer, dlayer):
        ok &= bool(torch.equal(other.sel_c, layer.sel_c))
        for b in range(B):
            n = int(layer.sel_c[b])
            ok &= bool(torch.equal(torch.sort(other.sel_i[b, :n]).values, torch.sort(layer.sel_i[b, :n]).values))
            if b % world == rank:
                ok &= float((other.out[b // world] - layer.out[b // world]).abs().max()) < 1e-3
    ok &= all(bool(torch.equal(xlayer.sel_i[b, :int(layer.sel_c[b])], layer.sel_i[b, :int(layer.sel_c[b])])) for b in range(B))
    # ---- the compressor as tasks of the same persistent kernel, across the real ranks: 13 steps of the
    # ratio-4 window machine (3 closing groups), each entry checked on its owner (n % world)
    from test_gpu_compress import _post_checks
    from mega_dsa_cp_b200.tiles.compress import CompressorState
    st = CompressorState(B, world, rank, 4, 128, device=dev)
    clayer = DsaDecodeLayer(B, cp=world, rank=rank, top_k=K, max_pages=pages, blocks_per_chunk=max(1, pages // 2),
                            kv_seq_stride=S_loc, out_dtype=torch.float32, n_ctas=64,
                            group_name=dist.group.WORLD.group_name, device=dev, compressor=st)
    clayer.bind(LayerInputs(d(fused), d(bt), d(seq_loc), d(q_idx), d(w_idx), d(q_mla), d(kv_loc)))
    steps = 13
    rec_a = torch.stack([torch.stack([orc.synth_record(b, p, 512, True) for p in range(steps)]) for b in range(B)])
    rec_i = torch.stack([torch.stack([orc.synth_record(b, p, 128, True) for p in range(steps)]) for b in range(B)])
    ape_a, ape_i = orc.synth_bias(512, 8), orc.synth_bias(128, 8)
    gn = torch.Generator().manual_seed(2)
    norm_a, norm_i = torch.rand(512, generator=gn) + 0.5, torch.rand(128, generator=gn) + 0.5
    freqs = orc.make_freqs(256)
    glen = torch.zeros(B, dtype=torch.int32, device=dev)
    new_a, new_i = torch.zeros(B, 4 * 512, device=dev), torch.zeros(B, 4 * 128, device=dev)
    clayer.bind_compressor(glen, new_a, new_i, d(ape_a), d(ape_i), d(norm_a), d(norm_i), 1e-6, d(freqs), fp8_scale=0.02)
    tally = {"e4m3": 0, "e4m3_off_by_one": 0, "nibbles": 0}
    dist.barrier()
    try:
        for sidx in range(steps):
            glen.fill_(sidx)
            new_a.copy_(rec_a[:, sidx])     # the rank that owns position sidx (sidx % world) appends it
            new_i.copy_(rec_i[:, sidx])
            clayer.step(wait_budget_ns=5_000_000_000)
            torch.cuda.synchronize()
            clayer.check_status()
            dist.barrier()
            if (sidx + 1) % 4 == 0:
                n = sidx // 4
                if n % world == rank:
                    for b in range(B):
                        pa = orc.csa_entry_ref(rec_a[b], ape_a, n, 512)
                        pi = orc.csa_entry_ref(rec_i[b], ape_i, n, 128)
                        _post_checks(st, b, n // world, pa, pi, 4 * n, norm_a, norm_i, freqs, 0.02, (world, sidx, b), tally)
                    ok &= st.k_valid.tolist() == [n // world + 1] * B
    except AssertionError as e:   # report through the common flag so every rank leaves together
        print(f"[rank {rank}] compressor check failed: {e}", flush=True)
        ok = False
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    worst = torch.tensor([worst_o, worst_l], device=dev)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(("MP_LAYER_OK" if flag.item() == 1 else "MP_LAYER_FAIL") +
              f" world={world} max_abs_o={worst[0].item():.3e} max_abs_lse={worst[1].item():.3e}")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
