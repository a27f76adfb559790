"""Seeded synthetic inputs with the shapes and value distributions of the
decode configurations (CPU generator, so the same tensors feed the CPU oracle
and, after a copy, the CUDA kernels).  They stand in for no external dataset:
the reference itself measures on seeded random tensors only."""

from __future__ import annotations

import math

import torch

from oracle import dsa_oracle as orc


def indexer_case(B, S, page_tokens, fmt, q_len=1, q_fp4=False, seed=0, pool_pages=None, shuffle=True):
    """Index-K cache of B sequences x S tokens in `fmt` pages, random page table.
    Returns dict with CPU tensors: fused pages, block_table, q (bf16 or FP4), w."""
    g = torch.Generator().manual_seed(seed)
    max_pages = S // page_tokens
    n_pages = pool_pages or B * max_pages
    raw = torch.randn(n_pages * page_tokens, 128, generator=g)
    fused, _ = orc.build_index_pages(raw, fmt, page_tokens)
    if shuffle:
        perm = torch.randperm(n_pages, generator=g)[: B * max_pages]
    else:
        perm = torch.arange(B * max_pages)
    bt = perm.reshape(B, max_pages).to(torch.int32)
    N = q_len * 64
    qraw = torch.randn(B, N, 128, generator=g)
    w = torch.randn(B, N, generator=g) / 64.0
    out = {"fused": fused, "bt": bt, "w": w, "fmt": fmt, "page_tokens": page_tokens, "q_len": q_len}
    if q_fp4:
        packed, sf = orc.quant_mxfp4(qraw)
        blocks = -(-N // 128)
        pad = torch.zeros(B, blocks * 128, 4, dtype=torch.uint8)
        pad[:, :N] = sf
        atom = torch.stack([orc.sf_to_atom(pad[b]) for b in range(B)]).reshape(B, blocks * 512)
        out.update(q=packed, q_sf=atom, q_deq=orc.dequant_fp4(packed, sf, orc.FMT_MXFP4))
    else:
        qb = qraw.to(torch.bfloat16)
        out.update(q=qb, q_sf=None, q_deq=qb.float())
    return out


def mla_case(B, T, H, d_qk, E, n_sel, dtype=torch.bfloat16, with_window=False, seed=0, page_cmp=1):
    """Sparse-MLA inputs: q ~ N(0, 0.5), KV rows ~ N(0, 0.5), random selections
    (n_sel: list of per-row counts)."""
    g = torch.Generator().manual_seed(seed)
    rows = B * T

    def cast(x):
        if dtype == torch.float8_e4m3fn:
            return x.clamp(-448, 448).to(torch.float8_e4m3fn)
        return x.to(dtype)

    q = cast(torch.randn(B, T, H, d_qk, generator=g) * 0.5)
    kv = cast(torch.randn(E, page_cmp, d_qk, generator=g) * 0.5)
    cols = max(n_sel) if page_cmp == 1 else -(-max(n_sel) // page_cmp)
    cols = max(cols, 1)
    pt = torch.zeros(rows, cols, dtype=torch.int32)
    for r in range(rows):
        n = n_sel[r] if page_cmp == 1 else -(-n_sel[r] // page_cmp)
        pt[r, :n] = torch.randperm(E, generator=g)[:n].to(torch.int32)
    k_valid = torch.tensor([128 + n for n in n_sel], dtype=torch.int32)
    out = {"q": q, "kv_cmp": kv, "pt_cmp": pt, "k_valid": k_valid, "page_cmp": page_cmp,
           "kv_win": None, "pt_win": None, "win_valid": None}
    if with_window:
        out["kv_win"] = cast(torch.randn(B, 128, d_qk, generator=g) * 0.5)
        out["pt_win"] = torch.arange(B, dtype=torch.int32).repeat_interleave(T).view(rows, 1)
        out["win_valid"] = torch.randint(0, 129, (rows,), generator=g, dtype=torch.int32)
    return out


def mla_oracle(case, sink, scale, **kw):
    f = lambda t: None if t is None else t.float()
    rows = case["q"].shape[0] * case["q"].shape[1]
    wv = case["win_valid"] if case["win_valid"] is not None else torch.zeros(rows, dtype=torch.int32)
    H = case["q"].shape[2]
    if sink is None:
        sink = torch.full((H,), -math.inf)
    return orc.ref_mla(f(case["q"]), f(case["kv_win"]), f(case["kv_cmp"]).reshape(-1, case["q"].shape[-1]),
                       case["pt_win"], case["pt_cmp"], case["k_valid"], wv, sink, scale,
                       d_v=512, page_cmp=case["page_cmp"], **kw)
