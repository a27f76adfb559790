"""Exact top-k merge over candidate lists: host runner.

Drop-in for mega_dsa_cp/tiles/merge.py:347-379 of the reference
(mdc_merge_topk_launch, csrc/tile_merge.cuh).
"""

from __future__ import annotations

import torch

from .. import _native as N

N_THREADS = 256


def run_merge_topk(
    cand_v: torch.Tensor,   # (B, q_len, L, maxK) fp32
    cand_i: torch.Tensor,   # (B, q_len, L, maxK) int32
    cand_c: torch.Tensor,   # (B, q_len, L) int32
    out_v: torch.Tensor,    # (B, q_len, top_k) fp32
    out_i: torch.Tensor,    # (B, q_len, top_k) int32
    out_c: torch.Tensor,    # (B, q_len) int32
    dbg: torch.Tensor | None,  # (>=1,) int32: [0] counts emit-count mismatches
    stream=None,
    top_k: int = 512,
) -> None:
    B, q_len, L, maxK = cand_v.shape
    assert L <= 256 and out_v.shape[-1] == top_k
    for t in (cand_v, cand_i, cand_c, out_v, out_i, out_c):
        assert t.is_cuda and t.is_contiguous()
    p = N.MergeTopkParams(
        cand_v=N.ptr(cand_v), cand_i=N.ptr(cand_i), cand_c=N.ptr(cand_c),
        out_v=N.ptr(out_v), out_i=N.ptr(out_i), out_c=N.ptr(out_c), dbg=N.ptr(dbg),
        B=B, q_len=q_len, L=L, maxK=maxK, top_k=top_k,
    )
    N.call("mdc_merge_topk_launch", p, stream)
