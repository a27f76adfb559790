"""Host-side FP4 index-cache formats: quantisation, dequantisation, fused page
assembly and synthetic caches/queries.

Two block-scaled E2M1 formats are supported by the indexer kernel:

* ``mxfp4``: UE8M0 scale per 32 elements, 128-token pages of 8704 bytes
  (128 x 64 B of packed codes, then 512 B of scales in the tensor-core "atom"
  order byte = (tok % 32) * 16 + (tok // 32) * 4 + group) -- the layout of
  mega_dsa_cp/tiles/fp4.py:60-67,106-125 of the reference.
* ``nvfp4``: UE4M3 scale per 16 elements, pages of P x 64 B of codes followed
  by P x 8 B of token-major scales (P = 64 or 128).

Codes pack two per byte, even element in the low nibble.  Quantisation rounds
through bf16 first and resolves E2M1 ties towards the even code, so the
mxfp4 path is bit-identical to the reference (fp4.py:18-41).
"""

from __future__ import annotations

import torch

E2M1_LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
HEAD_DIM = 128
SF_VEC = 32
NV_SF_VEC = 16


def _codes(scaled: torch.Tensor) -> torch.Tensor:
    mag = scaled.abs()
    # midpoints between levels; a midpoint belongs to the neighbour with the even code
    code = (mag > 0.25).to(torch.int32) + (mag >= 0.75) + (mag > 1.25) + (mag >= 1.75) \
        + (mag > 2.5) + (mag >= 3.5) + (mag > 5.0)
    return (code | ((scaled < 0).to(torch.int32) << 3)).to(torch.uint8)


def _pack(nib: torch.Tensor) -> torch.Tensor:
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).contiguous()


def _unpack_values(packed: torch.Tensor) -> torch.Tensor:
    lut = torch.tensor(E2M1_LEVELS + tuple(-x for x in E2M1_LEVELS), dtype=torch.float32, device=packed.device)
    pair = torch.stack((lut[(packed & 0xF).long()], lut[(packed >> 4).long()]), dim=-1)
    return pair.flatten(-2)


def quant_mxfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(..., K) -> (packed (..., K/2) uint8, UE8M0 bytes (..., K/32) uint8)."""
    assert x.shape[-1] % SF_VEC == 0
    grp = x.bfloat16().float().unflatten(-1, (-1, SF_VEC))
    s = (grp.abs().amax(dim=-1) / 6.0).clamp(min=1e-4)
    bits = s.view(torch.int32)
    e = ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)  # ceil(log2 s)
    nib = _codes(grp * torch.exp2(-e.float()).unsqueeze(-1)).flatten(-2)
    return _pack(nib), (e + 127).clamp(0, 254).to(torch.uint8).contiguous()


def dequant_mxfp4(packed: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    scale = torch.exp2(sf.float() - 127.0).repeat_interleave(SF_VEC, dim=-1)
    return _unpack_values(packed) * scale


def quant_nvfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(..., K) -> (packed (..., K/2) uint8, UE4M3 bytes (..., K/16) uint8)."""
    assert x.shape[-1] % NV_SF_VEC == 0
    grp = x.bfloat16().float().unflatten(-1, (-1, NV_SF_VEC))
    s8 = (grp.abs().amax(dim=-1) / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    s = s8.float()
    scaled = torch.where(s.unsqueeze(-1) > 0, grp / s.clamp(min=2.0 ** -9).unsqueeze(-1), torch.zeros_like(grp))
    return _pack(_codes(scaled).flatten(-2)), s8.view(torch.uint8).contiguous()


def dequant_nvfp4(packed: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    scale = sf.view(torch.float8_e4m3fn).float().repeat_interleave(NV_SF_VEC, dim=-1)
    return _unpack_values(packed) * scale


def sf_to_atom(sf: torch.Tensor) -> torch.Tensor:
    """(T, 4) token-major UE8M0 scales -> (T/128, 512) atom order."""
    T, kg = sf.shape
    assert T % 128 == 0 and kg == HEAD_DIM // SF_VEC
    # token r of a block = 32 * mid + inner  ->  byte inner * 16 + mid * 4 + group
    return sf.reshape(T // 128, 4, 32, kg).transpose(1, 2).reshape(T // 128, 512).contiguous()


def page_bytes(fmt: str = "mxfp4", page_tokens: int = 128) -> int:
    return page_tokens * 64 + page_tokens * (4 if fmt == "mxfp4" else 8)


def fuse_pages(raw: torch.Tensor, fmt: str = "mxfp4", page_tokens: int = 128):
    """(num_pages * page_tokens, 128) float -> (fused (num_pages, page_bytes) uint8,
    token-major scales (num_pages, page_tokens, groups))."""
    n_pages = raw.shape[0] // page_tokens
    if fmt == "mxfp4":
        assert page_tokens == 128, "mxfp4 pages hold 128 tokens"
        packed, sf = quant_mxfp4(raw)
        tail = sf_to_atom(sf)
    elif fmt == "nvfp4":
        packed, sf = quant_nvfp4(raw)
        tail = sf.reshape(n_pages, -1)
    else:
        raise ValueError(f"unknown fmt {fmt!r}")
    fused = torch.cat([packed.reshape(n_pages, page_tokens * 64), tail], dim=1).contiguous()
    return fused, sf.reshape(n_pages, page_tokens, -1)


def make_index_cache(B: int, max_pages: int, device: str = "cuda", seed: int = 0,
                     fmt: str = "mxfp4", page_tokens: int = 128):
    """Random paged index-K cache, pages of request b at b*max_pages.. (the
    reference's helper, fp4.py:106-125).  Returns (fused pages, plain scales)."""
    g = torch.Generator(device=device).manual_seed(seed)
    raw = torch.randn(B * max_pages * page_tokens, HEAD_DIM, generator=g, device=device)
    return fuse_pages(raw, fmt, page_tokens)


def make_q(B: int, q_len: int = 2, heads: int = 64, device: str = "cuda", seed: int = 1):
    """Random FP4 indexer query: (packed (B,N,64), plain scales (B,N,4), atom
    scales (B, ceil(N/128)*512), weights (B,N)).  Rows beyond N in the last
    128-row scale block are padding."""
    g = torch.Generator(device=device).manual_seed(seed)
    N = q_len * heads
    raw = torch.randn(B, N, HEAD_DIM, generator=g, device=device)
    packed, sf = quant_mxfp4(raw)
    blocks = -(-N // 128)
    padded = torch.zeros(B, blocks * 128, 4, dtype=torch.uint8, device=device)
    padded[:, :N] = sf
    atom = torch.stack([sf_to_atom(padded[b]) for b in range(B)]).reshape(B, blocks * 512)
    w = torch.rand(B, N, generator=g, device=device) * 0.1
    return packed, sf, atom, w
