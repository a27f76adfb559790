"""Chunked prefill on the decode tiles (one GPU, cp = 1): every query token of a
chunk against the CPU oracle's decode step at that token's causal length."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.mark.parametrize("S,Tq,tile,K,bpc", [(4096, 32, 8, 512, 16), (8192, 24, 12, 2048, 32)])
def test_prefill_chunk_matches_oracle_per_query(S, Tq, tile, K, bpc):
    from dsa_inputs import indexer_case
    from mega_dsa_cp_b200.prefill import DsaPrefillChunk, causal_local_lens
    from oracle import dsa_oracle as orc

    P, H, DQK = 64, 128, 576
    case = indexer_case(1, S, P, "nvfp4", seed=14)          # one sequence's index cache and page table
    g = torch.Generator().manual_seed(15)
    q_idx = torch.randn(Tq, 64, 128, generator=g).bfloat16()
    w_idx = torch.randn(Tq, 64, generator=g) / 64
    q_mla = (torch.randn(Tq, 1, H, DQK, generator=g) * 0.5).bfloat16()
    kv = (torch.randn(S, 1, DQK, generator=g) * 0.5).bfloat16()
    # the chunk's tokens are the last Tq of the context, plus two early positions shorter than top-k
    pos = torch.arange(S - Tq, S)
    pos[0], pos[1] = 5, K // 2
    assert causal_local_lens(pos, 1, 0).tolist() == (pos + 1).tolist()
    pf = DsaPrefillChunk(tile, cp=1, top_k=K, max_pages=S // P, blocks_per_chunk=bpc, out_dtype=torch.float32, n_ctas=64)
    d = lambda t: t.to(DEV)
    pf.bind(d(case["fused"]), d(case["bt"][0]), d(kv))
    out = torch.zeros(Tq, H, 512, device=DEV)
    lse = torch.zeros(Tq, H, device=DEV)
    sel_i = torch.zeros(Tq, K, dtype=torch.int32, device=DEV)
    sel_c = torch.zeros(Tq, dtype=torch.int32, device=DEV)
    pf.run(d(q_idx), d(w_idx), d(q_mla), pos, out, lse, sel_i, sel_c)
    torch.cuda.synchronize()
    pf.check_status()
    data, sf = orc.split_index_pages(case["fused"], "nvfp4", P)
    kd = orc.dequant_fp4(data, sf, "nvfp4").reshape(-1, P, 128)[case["bt"][0].long()].reshape(S, 128)
    scale = 1 / math.sqrt(DQK)
    for j in range(Tq):
        n_ctx = int(pos[j]) + 1
        sel, _, _ = orc.decode_step_ref(q_idx[j].float(), w_idx[j], kd, q_mla[j, 0].float(), kv[:, 0].float(),
                                        n_ctx, K, scale)
        n = int(sel_c[j])
        got = sel_i[j, :n].cpu()
        assert n == sel.numel() == min(K, n_ctx), (j, n, sel.numel())
        assert int(got.max()) < n_ctx                     # causal: nothing after the query's own position
        overlap = len(set(got.tolist()) & set(sel.tolist())) / sel.numel()
        assert overlap >= 0.999, (j, overlap)
        o, l = orc.attend_selected_ref(q_mla[j, 0].float(), kv[:, 0].float(), got, scale)
        assert (out[j].cpu() - o).abs().max() < 2e-2, j
        assert (lse[j].cpu() - l).abs().max() < 1e-3, j
