"""Sparse MLA decode attention: host runners.

`run_hca_fp8` is the drop-in for mega_dsa_cp/tiles/hca.py:3160-3270 of the
reference (fp8 operands, latent 512, dual pool, sink).  `run_sparse_mla` is
the same kernel family on bf16 operands with 576 QK / 512 V dims.  Both call
mdc_sparse_mla_launch (csrc/tile_mla.cuh).
"""

from __future__ import annotations

import torch

from .. import _native as N

H = 128
D = 512
STATIC_WS_MAX_SLOTS = 4096   # MDC_STATIC_WS_MAX_SLOTS of include/mdc.h


def sm_count(device) -> int:
    return torch.cuda.get_device_properties(device).multi_processor_count


def pick_splits(rows: int, heads: int, slots: int, sms: int) -> int:
    """KV splits so that rows * heads/64 * splits blocks roughly fill the SMs."""
    blocks = rows * (heads // 64)
    tiles = max(1, (slots + 63) // 64)
    return int(max(1, min(16, tiles, sms // max(1, blocks))))


def split_workspace(rows: int, n_splits: int, heads: int, device):
    """The fp32 workspace a split launch needs: (rows, n_splits, heads, 512) partial outputs and
    (rows, n_splits, heads) log2-LSEs.  The caller allocates it once and passes it to every call."""
    return (torch.empty(rows, n_splits, heads, D, dtype=torch.float32, device=device),
            torch.empty(rows, n_splits, heads, dtype=torch.float32, device=device))


def dense_layer_tables(n_entries: torch.Tensor, first_page: torch.Tensor, page_cmp: int, cols: int | None = None):
    """Page table and k_valid of a layer that attends to EVERY compressed entry of a sequence instead of
    a top-k selection (the ratio-128 layers of DeepSeek-V4: docs/overview.md:50-59 of the reference lists
    them; its kernels take the same tables).  n_entries (rows,) int32 valid entries per query row,
    first_page (rows,) int32 first pool page of the row's sequence (its pages are consecutive), page_cmp
    entries per page.  Returns (pt_cmp (rows, cols) int32 enumerating the pages in order, k_valid (rows,)
    = 128 window slots + entries).  A sliding-window-only layer needs no table at all: k_valid = 128
    everywhere (nothing beyond the window), any pt_cmp of one column."""
    rows = n_entries.numel()
    pages = torch.div(n_entries + page_cmp - 1, page_cmp, rounding_mode="floor")
    cols = int(cols or max(1, int(pages.max())))
    idx = torch.arange(cols, dtype=torch.int32, device=n_entries.device).view(1, cols)
    pt = torch.where(idx < pages.view(rows, 1), first_page.view(rows, 1).to(torch.int32) + idx, torch.zeros_like(idx))
    return pt.contiguous(), (128 + n_entries).to(torch.int32)


def run_sparse_mla(
    q: torch.Tensor,            # (B, T, H, d_qk) bf16 | float8_e4m3fn
    kv_win: torch.Tensor | None,   # (pages_win, 128, d_qk)
    kv_cmp: torch.Tensor,       # (pages_cmp, page_cmp, d_qk)
    pt_win: torch.Tensor | None,   # (B*T, 1) int32
    pt_cmp: torch.Tensor,       # (B*T, cols) int32
    o: torch.Tensor,            # (B, T, H, 512) fp32 | bf16 (row stride free)
    lse: torch.Tensor | None,   # (B, T, H) fp32
    k_valid: torch.Tensor,      # (B*T,) int32, counts the 128 window slots
    win_valid: torch.Tensor | None,
    attn_sink: torch.Tensor | None,
    softmax_scale: float,
    output_scale: float = 1.0,
    n_splits: int | None = None,
    fp8_p: bool = False,
    status: torch.Tensor | None = None,
    stream=None,
    workspace: tuple | None = None,   # split_workspace(...) owned by the caller
) -> None:
    """Nothing is allocated here.  A split launch writes its partials into `workspace` when the
    caller passes one, else into the library's fixed device block (mdc_sparse_mla_launch_static_ws:
    rows * n_splits * heads <= 4096, one call at a time per device); the split count is lowered
    to what that block holds."""
    B, T, heads, d_qk = q.shape
    rows = B * T
    kv_dt = N.DT_E4M3 if q.dtype == torch.float8_e4m3fn else N.DT_BF16
    assert kv_cmp.dtype == q.dtype and kv_cmp.is_contiguous() and q.is_contiguous()
    o2 = o.view(rows, heads, o.shape[-1]) if o.dim() == 4 else o
    assert o2.stride(2) == 1 and o2.stride(1) == o2.shape[2]
    if n_splits is None:
        n_splits = pick_splits(rows, heads, pt_cmp.shape[1] * kv_cmp.shape[1] + 128, sm_count(q.device))
    contiguous_out = o2.stride(0) == heads * o2.shape[2] and (lse is None or lse.is_contiguous())
    if not contiguous_out:
        n_splits = 1
    ws_o = ws_l = None
    entry = "mdc_sparse_mla_launch"
    if n_splits > 1 and workspace is not None:
        ws_o, ws_l = workspace
        assert ws_o.dtype == torch.float32 and ws_o.numel() >= rows * n_splits * heads * D
        assert ws_l.dtype == torch.float32 and ws_l.numel() >= rows * n_splits * heads
    elif n_splits > 1:
        n_splits = max(1, min(n_splits, STATIC_WS_MAX_SLOTS // (rows * heads)))
        if n_splits > 1:
            entry = "mdc_sparse_mla_launch_static_ws"
    p = N.SparseMlaParams(
        q=N.ptr(q), kv_win=N.ptr(kv_win), kv_cmp=N.ptr(kv_cmp), pt_win=N.ptr(pt_win), pt_cmp=N.ptr(pt_cmp),
        k_valid=N.ptr(k_valid), win_valid=N.ptr(win_valid), attn_sink=N.ptr(attn_sink),
        o=N.ptr(o), lse=N.ptr(lse), o_stride=o2.stride(0), lse_stride=heads if lse is None else lse.reshape(rows, heads).stride(0),
        ws_o=N.ptr(ws_o), ws_lse=N.ptr(ws_l),
        B=B, q_len=T, H=heads, d_qk=d_qk, d_v=D,
        pages_win=0 if kv_win is None else kv_win.shape[0], pages_cmp=kv_cmp.shape[0],
        page_cmp=kv_cmp.shape[1], pt_cols=pt_cmp.shape[1],
        kv_dtype=kv_dt, out_dtype=N.DT_F32 if o.dtype == torch.float32 else N.DT_BF16,
        n_splits=n_splits, fp8_p=int(fp8_p), softmax_scale=softmax_scale, output_scale=output_scale,
        status=N.ptr(status),
    )
    N.call(entry, p, stream)


def run_hca_fp8(
    q, kv_win, kv_cmp, pt_win, pt_cmp, o, lse, k_valid, win_valid, attn_sink,
    softmax_scale: float, output_scale: float = 1.0,
    acc_o: torch.Tensor | None = None,    # (B, T, H, 1, D) fp32 partial output
    acc_lse: torch.Tensor | None = None,  # (B, T, H, 1) fp32
    dbg: torch.Tensor | None = None,
    stream=None,
) -> None:
    """fp8 dual-pool attention with the reference's argument list; with
    acc_o/acc_lse the normalised partial and its log2-LSE go there instead of
    o/lse (the layout a cross-rank LSE merge consumes)."""
    B, T, heads, _ = q.shape
    if acc_o is not None:
        out_o = acc_o.view(B, T, heads, D)
        out_l = acc_lse.view(B, T, heads)
    else:
        out_o, out_l = o, lse
    run_sparse_mla(q, kv_win, kv_cmp, pt_win, pt_cmp, out_o, out_l, k_valid, win_valid, attn_sink,
                   softmax_scale, output_scale, fp8_p=True, stream=stream)
