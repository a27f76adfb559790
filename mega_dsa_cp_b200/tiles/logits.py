"""FP4 paged MQA indexer logits (+ fused exact local top-k): host runner.

Drop-in for mega_dsa_cp/tiles/logits.py:1054-1145 of the reference; the work
happens in libmdc.so (mdc_logits_fp4_launch, csrc/tile_logits.cuh).
"""

from __future__ import annotations

import torch

from .. import _native as N

PAGE_TOKENS = 128
HEAD_DIM = 128
PAGE_DATA_BYTES = PAGE_TOKENS * 64
PAGE_SF_BYTES = 512
PAGE_BYTES = PAGE_DATA_BYTES + PAGE_SF_BYTES
DEFAULT_TOP_K = 1024
HEADS = 64


def run_fp4_paged_mqa_logits(
    kv_fused: torch.Tensor,      # (num_pages, page_bytes) uint8 fused pages
    q_packed: torch.Tensor,      # (B, N, 64) uint8 FP4 query, or (B, N, 128) bf16 query
    q_sf_atom: torch.Tensor | None,  # (B, ceil(N/128)*512) uint8 for the FP4 query
    weights: torch.Tensor,       # (B, N) fp32
    block_table: torch.Tensor,   # (B, max_pages) int32
    logits: torch.Tensor | None,  # (B*q_len, max_pages*page_tokens) fp32; unused when fused
    blocks_per_chunk: int,
    num_kv_stage: int = 8,       # accepted for signature parity; the ring depth is fixed at 8
    seq_lens: torch.Tensor | None = None,  # (B,) int32
    cand_v: torch.Tensor | None = None,    # (B, q_len, n_chunks, top_k) fp32
    cand_i: torch.Tensor | None = None,    # (B, q_len, n_chunks, top_k) int32
    cand_c: torch.Tensor | None = None,    # (B, q_len, n_chunks) int32
    dbg: torch.Tensor | None = None,       # accepted for signature parity, not written
    stream=None,
    top_k: int = DEFAULT_TOP_K,
    *,
    fmt: str = "mxfp4",
    page_tokens: int = 128,
    window_exclude: int | None = None,
    id_mul: int = 1,
    id_add: int = 0,
    status: torch.Tensor | None = None,    # (8,) int32 device-failure block
    row_topk: tuple | None = None,         # (out_v, out_i, out_c): exact top-k of the whole row in one launch
) -> None:
    B, n_rows = q_packed.shape[0], q_packed.shape[1]
    q_len = n_rows // HEADS
    assert n_rows == q_len * HEADS, "query rows must be q_len * 64"
    max_pages = block_table.shape[1]
    fused = cand_v is not None
    row_v = row_i = row_c = None
    if row_topk is not None:
        row_v, row_i, row_c = row_topk
        assert row_v.shape[-1] == top_k and row_i.shape == row_v.shape and row_v.is_contiguous()
    n_chunks = -(-max_pages // blocks_per_chunk)
    q_is_bf16 = q_packed.dtype == torch.bfloat16
    for t in (kv_fused, q_packed, weights, block_table):
        assert t.is_cuda and t.is_contiguous()
    assert block_table.dtype == torch.int32 and weights.dtype == torch.float32
    assert kv_fused.shape[1] == page_tokens * 64 + page_tokens * (4 if fmt == "mxfp4" else 8), \
        "page size does not match fmt/page_tokens"
    if row_topk is not None:
        pass
    elif fused:
        assert cand_v.shape == (B, q_len, n_chunks, top_k) and cand_i.shape == cand_v.shape
        assert cand_c.shape == (B, q_len, n_chunks)
    else:
        assert logits is not None and logits.shape[0] == B * q_len
        assert logits.shape[1] >= max_pages * page_tokens and logits.stride(1) == 1
    if window_exclude is None:
        window_exclude = 128 if (fmt == "mxfp4" and (fused or row_topk is not None)) else 0
    p = N.LogitsParams(
        kv_pages=N.ptr(kv_fused), num_pages=kv_fused.shape[0], page_tokens=page_tokens,
        fmt=N.FMT_MXFP4 if fmt == "mxfp4" else N.FMT_NVFP4,
        q_fmt=N.Q_BF16 if q_is_bf16 else N.Q_FP4,
        q=N.ptr(q_packed), q_sf=N.ptr(q_sf_atom), weights=N.ptr(weights),
        block_table=N.ptr(block_table), max_pages=max_pages, seq_lens=N.ptr(seq_lens),
        logits=None if (fused or row_topk is not None) else N.ptr(logits),
        logits_stride=0 if (fused or row_topk is not None) else logits.stride(0),
        cand_v=N.ptr(cand_v), cand_i=N.ptr(cand_i), cand_c=N.ptr(cand_c), top_k=top_k,
        B=B, q_len=q_len, heads=HEADS, blocks_per_chunk=blocks_per_chunk, n_chunks=n_chunks,
        window_exclude=window_exclude, id_mul=id_mul, id_add=id_add, status=N.ptr(status),
        row_v=N.ptr(row_v), row_i=N.ptr(row_i), row_c=N.ptr(row_c),
    )
    N.call("mdc_logits_fp4_launch", p, stream)
