"""Cross-rank LSE merge of attention partials: host runner.

Drop-in for mega_dsa_cp/tiles/lse_merge.py:175-197 of the reference
(mdc_lse_merge_launch, csrc/tile_lse_merge.cuh).  Partials may be fp32 (the
reference's layout) or bf16; the output may be fp32 or bf16.
"""

from __future__ import annotations

import torch

from .. import _native as N

N_THREADS = 256
H = 128
D = 512

_DT = {torch.float32: N.DT_F32, torch.bfloat16: N.DT_BF16}


def run_lse_merge(
    acc_o: torch.Tensor,    # (B, q_len, cp_max, H, D) fp32 | bf16
    acc_lse: torch.Tensor,  # (B, q_len, cp_max, H) fp32, log2 domain
    o: torch.Tensor,        # (B, q_len, H, D) fp32 | bf16
    lse: torch.Tensor | None,  # (B, q_len, H) fp32
    cp: int,
    stream=None,
) -> None:
    B, q_len, cp_max, heads, dim = acc_o.shape
    for t in (acc_o, acc_lse, o):
        assert t.is_cuda and t.is_contiguous()
    assert acc_lse.dtype == torch.float32 and acc_lse.shape == (B, q_len, cp_max, heads)
    assert o.shape == (B, q_len, heads, dim)
    p = N.LseMergeParams(
        acc_o=N.ptr(acc_o), acc_lse=N.ptr(acc_lse), o=N.ptr(o), lse=N.ptr(lse),
        rows=B * q_len, H=heads, D=dim, n_slices=cp, n_slices_max=cp_max,
        acc_dtype=_DT[acc_o.dtype], out_dtype=_DT[o.dtype],
    )
    N.call("mdc_lse_merge_launch", p, stream)
