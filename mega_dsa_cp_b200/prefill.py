"""Chunked prefill of context-parallel DeepSeek sparse attention on the decode
tiles (no counterpart in the reference, whose tiles cover decode only).

A chunk of new tokens of ONE sequence is processed in tiles of `tile` query
tokens.  Inside a tile every query token is a batch entry of the decode
layer-step with its own causal length; all entries read the sequence's index
cache through the same page-table row and gather from the same KV rows
(`kv_group = tile`).  Per query token the step is exactly the decode step:
indexer logits over the tokens at or before its position, exact global
top-k, sparse MLA over the selection, LSE merge on the owner rank.  The new
tokens' cache entries must already be in the caches (written by the caller,
or by decode steps with KVWRITE), as the causal lengths include them.

This version re-streams the index cache once per query token (from L2 for
all but the first entry of a tile: a sequence's shard is a few MB).  A
GEMM-shaped tile that decodes a K tile once for many query tokens is the
faster form and is not built.

Token t lives on rank t % cp at local index t // cp, so query position p
sees (p - rank) // cp + 1 local tokens on ranks <= p and 0 on the others.
Entry j of a tile is owned by rank j % cp, which holds its merged output.
"""

from __future__ import annotations

import torch

from .layer import DsaDecodeLayer, LayerInputs


def causal_local_lens(positions: torch.Tensor, cp: int, rank: int) -> torch.Tensor:
    """Rank-local token counts visible to queries at global `positions` (the token at the position included)."""
    p = positions.to(torch.int64)
    n = torch.div(p - rank, cp, rounding_mode="floor") + 1
    return torch.where(p >= rank, n, torch.zeros_like(n)).to(torch.int32)


class DsaPrefillChunk:
    """Owns one decode layer of batch `tile` and feeds it the query tokens of a chunk tile by tile."""

    def __init__(self, tile: int, cp: int = 1, rank: int = 0, top_k: int = 2048, heads: int = 128, d_qk: int = 576,
                 fmt: str = "nvfp4", page_tokens: int = 64, max_pages: int = 256, blocks_per_chunk: int = 64,
                 group_name: str = "0", device="cuda", out_dtype=torch.bfloat16, **layer_kw):
        assert tile >= 1 and tile % cp == 0, "a tile must give every rank the same number of owned rows"
        self.tile, self.cp, self.rank, self.H = tile, cp, rank, heads
        self.layer = DsaDecodeLayer(tile, cp=cp, rank=rank, top_k=top_k, heads=heads, d_qk=d_qk, fmt=fmt,
                                    page_tokens=page_tokens, max_pages=max_pages, blocks_per_chunk=blocks_per_chunk,
                                    kv_seq_stride=max_pages * page_tokens, kv_group=tile, group_name=group_name,
                                    device=device, out_dtype=out_dtype, **layer_kw)
        dev = self.layer.device
        self.block_table = torch.zeros(tile, max_pages, dtype=torch.int32, device=dev)
        self._caches = None
        self._plan = None

    def bind(self, kv_pages: torch.Tensor, block_table_row: torch.Tensor, kv_mla: torch.Tensor) -> None:
        """The sequence's caches on this rank: index-K pages, its page-table row (max_pages,), its local
        KV rows (max_pages * page_tokens, 1, d_qk) with local token l at row l."""
        self.block_table.copy_(block_table_row.to(torch.int32).view(1, -1).expand_as(self.block_table))
        self._caches = (kv_pages, kv_mla)
        self._plan = None

    def run(self, q_idx: torch.Tensor, w_idx: torch.Tensor, q_mla: torch.Tensor, positions: torch.Tensor,
            out: torch.Tensor, out_lse: torch.Tensor | None = None, sel_i: torch.Tensor | None = None,
            sel_c: torch.Tensor | None = None, stream=None) -> None:
        """q_idx (Tq, 64, 128) bf16, w_idx (Tq, 64) fp32, q_mla (Tq, 1, H, d_qk) bf16 (contiguous, on the
        device) and positions (Tq,) global token positions of the chunk's query tokens, replicated on every
        rank; Tq a multiple of `tile`.  `out` (Tq / cp, H, 512) receives this rank's owned rows: query j of
        the chunk is owned by rank j % cp (tile is a multiple of cp) and lands at row j // cp.  Optional
        `sel_i` (Tq, top_k) / `sel_c` (Tq,) receive every query's selection (identical on all ranks).
        Asynchronous on `stream`.  Per tile: the launch parameters point at the tile's slices of the query
        tensors (no copies of the inputs), one kernel launch, and the copies of the results."""
        assert self._caches is not None, "bind() the sequence's caches first"
        kv_pages, kv_mla = self._caches
        Tq, T, cp = q_idx.shape[0], self.tile, self.cp
        assert Tq % T == 0 and positions.numel() == Tq
        assert q_idx.is_contiguous() and w_idx.is_contiguous() and q_mla.is_contiguous()
        # The launch parameters of every tile (addresses of the tile's slices) are built once per set of
        # tensors and reused while the caller keeps passing the same buffers: building them is host work of
        # about a tile's run time.  The causal lengths go through a buffer of this object for the same reason.
        key = (q_idx.data_ptr(), w_idx.data_ptr(), q_mla.data_ptr(), kv_pages.data_ptr(), kv_mla.data_ptr(), Tq)
        if self._plan is None or self._plan[0] != key:
            lens_buf = torch.zeros(Tq, dtype=torch.int32, device=self.layer.device)
            params = []
            for t0 in range(0, Tq, T):
                self.layer.bind(LayerInputs(kv_pages=kv_pages, block_table=self.block_table, seq_lens=lens_buf[t0:t0 + T],
                                            q_idx=q_idx[t0:t0 + T], w_idx=w_idx[t0:t0 + T], q_mla=q_mla[t0:t0 + T],
                                            kv_mla=kv_mla))
                params.append(self.layer._params)
            self._plan = (key, lens_buf, params, (q_idx, w_idx, q_mla))   # (the tensors are kept alive with the plan)
        _, lens_buf, params, _ = self._plan
        own = T // cp
        ctx = torch.cuda.stream(stream) if stream is not None and hasattr(stream, "cuda_stream") else _null()
        with ctx:
            lens_buf.copy_(causal_local_lens(positions.to(self.layer.device), cp, self.rank), non_blocking=True)
            for i, t0 in enumerate(range(0, Tq, T)):
                self.layer._params = params[i]
                self.layer.step(stream=stream)
                r0 = t0 // cp
                out[r0:r0 + own].copy_(self.layer.out[:own], non_blocking=True)
                if out_lse is not None:
                    out_lse[r0:r0 + own].copy_(self.layer.out_lse[:own], non_blocking=True)
                if sel_i is not None:
                    sel_i[t0:t0 + T].copy_(self.layer.sel_i, non_blocking=True)
                if sel_c is not None:
                    sel_c[t0:t0 + T].copy_(self.layer.sel_c, non_blocking=True)

    def check_status(self) -> None:
        self.layer.check_status()


class _null:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False
