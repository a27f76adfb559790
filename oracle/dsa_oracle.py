"""CPU oracle for the context-parallel DSA decode path.  TEST INFRASTRUCTURE ONLY.

This module restates, on CPU torch, the reference algorithms that the CUDA
kernels of this repository implement.  It is the checker: only the test-suite,
the smoke entry point and the benchmark's CPU-baseline leg may import it; no
product module does.

Parity status: PINNED.  Every function that has a counterpart in the reference
is compared against outputs of the reference's own torch code (imported once,
in the build container) through the fixtures in ``tests/golden``; the script
``tests/golden/make_golden.py`` regenerates them.  Functions that extend the
reference to shapes it does not cover (NVFP4 scales, 64-token pages, bf16 MLA
with 576 QK dims, ratio-64 pooling, cp-way composition) are marked EXTENSION;
they are pinned indirectly: each reduces to the pinned function when its extra
parameters take the reference's values, and tests check that reduction.

Reference citations use paths inside the reference project.
"""

from __future__ import annotations

import math

import torch

# --------------------------------------------------------------------------
# FP4 (E2M1) block-scaled formats
# --------------------------------------------------------------------------

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
IDX_DIM = 128

FMT_MXFP4 = "mxfp4"  # E2M1 + UE8M0 scale per 32 elements
FMT_NVFP4 = "nvfp4"  # E2M1 + UE4M3 scale per 16 elements


def group_size(fmt: str) -> int:
    return 32 if fmt == FMT_MXFP4 else 16


def _e2m1_encode(q: torch.Tensor) -> torch.Tensor:
    """Scaled fp32 values -> 4-bit codes, round-to-nearest with ties to the
    even code (mega_dsa_cp/tiles/fp4.py:28-37): boundaries 0.25, 0.75, 1.25,
    1.75, 2.5, 3.5, 5.0 where the boundary itself goes to the even code."""
    mag = q.abs()
    # (boundary, inclusive?) in increasing order; each passed boundary adds 1
    steps = ((0.25, False), (0.75, True), (1.25, False), (1.75, True),
             (2.5, False), (3.5, True), (5.0, False))
    code = torch.zeros(mag.shape, dtype=torch.int32)
    for bound, inclusive in steps:
        code += ((mag >= bound) if inclusive else (mag > bound)).to(torch.int32)
    return (code | ((q < 0).to(torch.int32) << 3)).to(torch.uint8)


def _pack_nibbles(nib: torch.Tensor) -> torch.Tensor:
    """(..., K) codes -> (..., K/2) bytes, even element in the low nibble
    (mega_dsa_cp/tiles/fp4.py:38-39)."""
    return (nib[..., 0::2] | (nib[..., 1::2] << 4)).contiguous()


def _e2m1_decode(packed: torch.Tensor) -> torch.Tensor:
    """(..., K/2) bytes -> (..., K) fp32 unscaled values
    (mega_dsa_cp/tiles/fp4.py:46-55)."""
    table = torch.tensor(E2M1_VALUES + tuple(-v for v in E2M1_VALUES), dtype=torch.float32)
    lo = table[(packed & 0xF).long()]
    hi = table[(packed >> 4).long()]
    return torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


def _ue8m0_ceil_exponent(s: torch.Tensor) -> torch.Tensor:
    """ceil(log2 s) for positive fp32 s by bit inspection
    (mega_dsa_cp/tiles/compress_ref.py:199-200)."""
    bits = s.contiguous().view(torch.int32)
    return ((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFF) != 0).to(torch.int32)


def quant_mxfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """(..., K) float -> (packed (..., K/2) u8, scale bytes (..., K/32) u8).
    Follows mega_dsa_cp/tiles/fp4.py:18-41 with the integer exponent of
    compress_ref.py:186-216 (mathematically the same ceil(log2))."""
    xb = x.to(torch.bfloat16).to(torch.float32)
    g = xb.reshape(*xb.shape[:-1], -1, 32)
    s = (g.abs().amax(dim=-1) / 6.0).clamp(min=1e-4)
    e = _ue8m0_ceil_exponent(s)
    q = g / torch.exp2(e.to(torch.float32)).unsqueeze(-1)
    nib = _e2m1_encode(q).reshape(*x.shape)
    sf = (e + 127).clamp(0, 254).to(torch.uint8)
    return _pack_nibbles(nib), sf.contiguous()


def ue4m3_to_float(b: torch.Tensor) -> torch.Tensor:
    return b.contiguous().view(torch.float8_e4m3fn).to(torch.float32)


def quant_nvfp4(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """EXTENSION (NVFP4 analogue of quant_mxfp4): per-16 amax, scale =
    e4m3(amax/6) (round to nearest even, saturating, never negative), codes by
    the same E2M1 rounding.  Returns (packed (..., K/2), scale bytes (..., K/16))."""
    xb = x.to(torch.bfloat16).to(torch.float32)
    g = xb.reshape(*xb.shape[:-1], -1, 16)
    s = (g.abs().amax(dim=-1) / 6.0).clamp(max=448.0)
    sf8 = s.to(torch.float8_e4m3fn)
    sf = sf8.view(torch.uint8)
    sval = sf8.to(torch.float32)
    q = torch.where(sval.unsqueeze(-1) > 0, g / sval.clamp(min=2.0 ** -9).unsqueeze(-1),
                    torch.zeros_like(g))
    nib = _e2m1_encode(q).reshape(*x.shape)
    return _pack_nibbles(nib), sf.contiguous()


def dequant_fp4(packed: torch.Tensor, sf: torch.Tensor, fmt: str = FMT_MXFP4) -> torch.Tensor:
    """(packed (..., K/2), plain scales (..., K/group)) -> fp32 (..., K).
    MXFP4 branch = mega_dsa_cp/tiles/fp4.py:44-57."""
    vals = _e2m1_decode(packed)
    if fmt == FMT_MXFP4:
        scale = torch.exp2(sf.to(torch.float32) - 127.0)
    else:
        scale = ue4m3_to_float(sf)
    return vals * scale.repeat_interleave(group_size(fmt), dim=-1)


def sf_to_atom(sf: torch.Tensor) -> torch.Tensor:
    """(T, 4) plain MXFP4 scales -> (T/128, 512): byte (tok%32)*16 + (tok//32)*4 + g
    per 128-token block (mega_dsa_cp/tiles/fp4.py:60-67)."""
    T, kg = sf.shape
    out = torch.zeros(T // 128, 512, dtype=torch.uint8)
    tok = torch.arange(T)
    blk, r = tok // 128, tok % 128
    for g in range(kg):
        out[blk, (r % 32) * 16 + (r // 32) * 4 + g] = sf[:, g]
    return out


def atom_to_sf(atom: torch.Tensor, kg: int = 4) -> torch.Tensor:
    nblk = atom.shape[0]
    r = torch.arange(128)
    cols = [(r % 32) * 16 + (r // 32) * 4 + g for g in range(kg)]
    return torch.stack([atom[:, c] for c in cols], dim=-1).reshape(nblk * 128, kg)


def page_bytes(fmt: str, page_tokens: int) -> int:
    return page_tokens * 64 + page_tokens * (IDX_DIM // group_size(fmt))


def build_index_pages(raw: torch.Tensor, fmt: str, page_tokens: int):
    """raw (num_pages*page_tokens, 128) fp32 -> (fused pages u8 (num_pages, page_bytes),
    plain scales (num_pages, page_tokens, groups)).  MXFP4/128 reproduces the
    fused page of mega_dsa_cp/tiles/fp4.py:106-125 (data then atom-ordered
    scales); NVFP4 pages (EXTENSION) hold data then token-major scales."""
    n_tok = raw.shape[0]
    n_pages = n_tok // page_tokens
    if fmt == FMT_MXFP4:
        assert page_tokens == 128
        packed, sf = quant_mxfp4(raw)
        tail = sf_to_atom(sf)
    else:
        packed, sf = quant_nvfp4(raw)
        tail = sf.reshape(n_pages, page_tokens * 8)
    fused = torch.cat([packed.reshape(n_pages, page_tokens * 64), tail], dim=1).contiguous()
    return fused, sf.reshape(n_pages, page_tokens, -1)


def split_index_pages(fused: torch.Tensor, fmt: str, page_tokens: int):
    """Inverse view of build_index_pages: (packed (pages*tok, 64), plain sf)."""
    n_pages = fused.shape[0]
    data = fused[:, : page_tokens * 64].reshape(n_pages * page_tokens, 64)
    tail = fused[:, page_tokens * 64:]
    if fmt == FMT_MXFP4:
        sf = atom_to_sf(tail.reshape(-1, 512))
    else:
        sf = tail.reshape(n_pages * page_tokens, 8)
    return data, sf


def ref_logits(q: torch.Tensor, weights: torch.Tensor, fused: torch.Tensor,
               block_table: torch.Tensor, q_len: int, fmt: str = FMT_MXFP4,
               page_tokens: int = 128, heads: int = 64) -> torch.Tensor:
    """Indexer logits, fp32: out[b*q_len+t, s] = sum_h w[b,tH+h] * relu(q[b,tH+h] . k[s])
    with k gathered through the page table (mega_dsa_cp/tiles/fp4.py:70-103).
    q is the DEQUANTISED query (B, q_len*heads, 128) fp32 (from FP4 or bf16)."""
    B = q.shape[0]
    data, sf = split_index_pages(fused, fmt, page_tokens)
    k_all = dequant_fp4(data, sf, fmt).reshape(fused.shape[0], page_tokens, IDX_DIM)
    max_pages = block_table.shape[1]
    out = torch.zeros(B * q_len, max_pages * page_tokens, dtype=torch.float32)
    for b in range(B):
        k = k_all[block_table[b].long()].reshape(max_pages * page_tokens, IDX_DIM)
        for t in range(q_len):
            rows = slice(t * heads, (t + 1) * heads)
            dots = q[b, rows].to(torch.float32) @ k.T
            out[b * q_len + t] = (dots.clamp(min=0) * weights[b, rows].unsqueeze(1)).sum(dim=0)
    return out


# --------------------------------------------------------------------------
# Exact top-k with the total order (logit descending, id ascending)
# --------------------------------------------------------------------------

def sortable_u32(v: torch.Tensor) -> torch.Tensor:
    """fp32 -> int64 holding the monotone u32 key: negative -> ~bits, else
    bits ^ 0x80000000 (mega_dsa_cp/tiles/logits.py:69-89)."""
    u = v.contiguous().view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    return torch.where(u >= 0x80000000, u ^ 0xFFFFFFFF, u ^ 0x80000000)


def key64(v: torch.Tensor, ids: torch.Tensor) -> list:
    """Python-int 64-bit keys (sortable(v) << 32) | ~id (unsigned order;
    mega_dsa_cp/tiles/merge.py:45-79 stores the same key sign-flipped)."""
    hi = sortable_u32(v).tolist()
    lo = ((~ids.to(torch.int64)) & 0xFFFFFFFF).tolist()
    return [(h << 32) | l for h, l in zip(hi, lo)]


def topk_select_mask(v: torch.Tensor, ids: torch.Tensor, k: int) -> torch.Tensor:
    """Boolean mask of the k best entries of a 1-D list under (v desc, id asc),
    bit-level on v (so -0.0 < +0.0 and NaNs order by their bit pattern, as
    the radix key does)."""
    n = v.numel()
    if n <= k:
        return torch.ones(n, dtype=torch.bool)
    keys = key64(v, ids)
    order = sorted(range(n), key=keys.__getitem__, reverse=True)[:k]
    mask = torch.zeros(n, dtype=torch.bool)
    mask[torch.tensor(order, dtype=torch.long)] = True
    return mask


def merge_topk_ref(cand_v, cand_i, cand_c, top_k: int):
    """Exact top-k over L candidate lists per (b, t), emitted in padded input
    order (mega_dsa_cp/tiles/merge_ref.py:12-45)."""
    B, T, L, maxK = cand_v.shape
    out_v = torch.zeros(B, T, top_k, dtype=torch.float32)
    out_i = torch.zeros(B, T, top_k, dtype=torch.int32)
    out_c = torch.zeros(B, T, dtype=torch.int32)
    pos = torch.arange(maxK)
    for b in range(B):
        for t in range(T):
            live = (pos[None, :] < cand_c[b, t][:, None]).reshape(-1)
            v = cand_v[b, t].reshape(-1)[live]
            i = cand_i[b, t].reshape(-1)[live]
            if v.numel() == 0:
                continue
            m = topk_select_mask(v, i, top_k)
            n = int(m.sum())
            out_v[b, t, :n] = v[m]
            out_i[b, t, :n] = i[m]
            out_c[b, t] = n
    return out_v, out_i, out_c


def local_topk_ref(logits_row: torch.Tensor, lo: int, hi: int, limit: int, top_k: int,
                   id_mul: int = 1, id_add: int = 0):
    """Candidates of one (b, t, chunk): the top_k of logits_row[lo:min(hi,limit)]
    under (v desc, position asc), emitted in position order, ids = pos*id_mul+id_add.
    Set semantics of mega_dsa_cp/tiles/logits.py:819-865 (the reference's emit
    order is unspecified; this oracle and the CUDA tile use position order)."""
    hi = max(lo, min(hi, limit))
    seg = logits_row[lo:hi]
    pos = torch.arange(lo, hi, dtype=torch.int32)
    m = topk_select_mask(seg, pos, top_k)
    return seg[m], (pos[m] * id_mul + id_add).to(torch.int32)


# --------------------------------------------------------------------------
# LSE merge
# --------------------------------------------------------------------------

def lse_merge_ref(acc_o: torch.Tensor, acc_lse: torch.Tensor, cp: int):
    """acc_o (B,T,cp_max,H,D), acc_lse (B,T,cp_max,H) log2-domain ->
    (o (B,T,H,D), lse (B,T,H)); all-empty heads give o = 0, lse = -inf
    (mega_dsa_cp/tiles/lse_merge_ref.py:8-23)."""
    o_p = acc_o[:, :, :cp].to(torch.float32)
    l_p = acc_lse[:, :, :cp].to(torch.float32)
    top = l_p.amax(dim=2)
    anchor = torch.where(torch.isinf(top), torch.zeros_like(top), top)
    mass = torch.exp2(l_p - anchor.unsqueeze(2)).sum(dim=2)
    live = mass > 0
    neg_inf = torch.full_like(top, -math.inf)
    glse = torch.where(live, top + torch.log2(mass.clamp(min=1e-30)), neg_inf)
    share = torch.where(live.unsqueeze(2), torch.exp2(l_p - glse.unsqueeze(2)),
                        torch.zeros_like(l_p))
    return (o_p * share.unsqueeze(-1)).sum(dim=2), glse


# --------------------------------------------------------------------------
# Sparse MLA decode attention
# --------------------------------------------------------------------------

LOG2E = 1.4426950408889634
WIN_SLOTS = 128


def _gather_cmp(kcmp: torch.Tensor, ids: torch.Tensor, page_cmp: int) -> torch.Tensor:
    d = kcmp.shape[-1]
    if page_cmp == 1:
        return kcmp.reshape(-1, d)[ids.long()]
    return kcmp.reshape(-1, page_cmp, d)[ids.long()].reshape(-1, d)


def ref_mla(q, kwin, kcmp, pt_win, pt_cmp, k_valid, win_valid, sink, softmax_scale,
            output_scale: float = 1.0, d_v: int = 512, page_cmp: int = 1,
            fp8_p: bool = False, online_tile: int = 0):
    """Dual-pool sparse attention on fp32 views of the operands.

    q (B,T,H,Dqk); kwin (pages_win,128,Dqk) or None; kcmp (E*page_cmp, Dqk)
    gathered by pt_cmp (B*T, cols); slots [0,128) = window pool (valid below
    win_valid[row]), slots [128, k_valid[row]) = gathered pool; sink (H,) extra
    logit with zero value (-inf disables); V = first d_v columns of K.
    Returns (o (B,T,H,d_v), lse (B,T,H) in the log2 domain).

    online_tile == 0 is the one-shot softmax of mega_dsa_cp/tiles/hca_ref.py:189-245
    (d_v == Dqk == 512 and fp8_p=True are the reference's values); online_tile == 128
    is the tile-by-tile simulation of hca_ref.py:121-186, which quantises P to
    e4m3 at the running maximum.  EXTENSION: Dqk = 576 with d_v = 512, bf16 operands.
    """
    B, T, H, dqk = q.shape
    scale_log2 = softmax_scale * LOG2E
    o = torch.zeros(B, T, H, d_v)
    lse = torch.full((B, T, H), -math.inf)
    for b in range(B):
        for t in range(T):
            row = b * T + t
            sel = _gather_cmp(kcmp, pt_cmp[row], page_cmp)
            if kwin is not None:
                win = kwin[int(pt_win[row, 0])]
            else:
                win = torch.zeros(WIN_SLOTS, dqk)
            kall = torch.cat([win, sel], dim=0)
            n = kall.shape[0]
            if online_tile:
                n = min(n, -(-int(k_valid[row]) // online_tile) * online_tile)
                kall = kall[:n]
            s = q[b, t] @ kall.T
            slot = torch.arange(n)
            dead = torch.where(slot < WIN_SLOTS, slot >= win_valid[row], slot >= k_valid[row])
            s = s.masked_fill(dead[None, :], -math.inf)
            v = kall[:, :d_v]
            if not online_tile:
                peak = torch.maximum(s.amax(dim=-1), sink)
                p = torch.exp2((s - peak[:, None]) * scale_log2)
                p = torch.where(torch.isfinite(peak)[:, None], p, torch.zeros_like(p))
                if fp8_p:
                    p = p.to(torch.float8_e4m3fn).to(torch.float32)
                denom = p.sum(dim=-1)
                extra = torch.exp2((sink - peak) * scale_log2)
                denom = denom + torch.where(torch.isinf(sink), torch.zeros_like(extra), extra)
                acc = p @ v
            else:
                peak = sink.clone()
                acc = torch.zeros(H, d_v)
                denom = torch.where(torch.isinf(sink), torch.zeros(H), torch.ones(H))
                for j in range(0, n, online_tile):
                    st = s[:, j:j + online_tile]
                    new_peak = torch.maximum(peak, st.amax(dim=-1))
                    fix = torch.exp2((peak - new_peak) * scale_log2)
                    fix = torch.where(new_peak == peak, torch.ones_like(fix), fix)
                    p = torch.exp2((st - new_peak[:, None]) * scale_log2)
                    # nothing seen yet and nothing live in this tile: no mass (the
                    # reference's simulation yields NaN here, its kernel does not)
                    p = torch.where(torch.isfinite(new_peak)[:, None], p, torch.zeros_like(p))
                    if fp8_p:
                        p = p.to(torch.float8_e4m3fn).to(torch.float32)
                    acc = acc * fix[:, None] + p @ v[j:j + online_tile]
                    denom = denom * fix + p.sum(dim=-1)
                    peak = new_peak
            ok = denom > 0
            o[b, t] = torch.where(ok[:, None], acc / denom.clamp(min=1e-30)[:, None],
                                  torch.zeros_like(acc)) * output_scale
            lse[b, t] = torch.where(ok, torch.log2(denom.clamp(min=1e-30)) + scale_log2 * peak,
                                    torch.full_like(denom, -math.inf))
    return o, lse


# --------------------------------------------------------------------------
# KV compressor (softmax-gated pooling + post chain)
# --------------------------------------------------------------------------

HADAMARD_SCALE = 0.0883883461356163  # fp32 nearest of 1/sqrt(128)
ROPE_DIM = 64


def hadamard128_staged(x: torch.Tensor) -> torch.Tensor:
    """128-point Hadamard in the kernel's butterfly order: strides 1, 2 inside
    groups of 4 consecutive elements, then strides 4..64 across groups
    (mega_dsa_cp/tiles/compress_ref.py:43-58)."""
    v = x.reshape(*x.shape[:-1], 32, 4)
    p, q_, r, s = v.unbind(-1)
    u0, u1, u2, u3 = p + q_, p - q_, r + s, r - s
    v = torch.stack([u0 + u2, u1 + u3, u0 - u2, u1 - u3], dim=-1)
    lane = torch.arange(32)
    for bit in (1, 2, 4, 8, 16):
        partner = v[..., lane ^ bit, :]
        upper = ((lane & bit) != 0).reshape(-1, 1)
        v = torch.where(upper, partner - v, v + partner)
    return (v * HADAMARD_SCALE).reshape(x.shape)


def rms_norm(x, weight, eps):
    """mega_dsa_cp/tiles/compress_ref.py:77-80.  The mean of squares is accumulated in float64 and
    rounded to float32 once: within one ulp of the reference's float32 reduction, but independent
    of the order of the additions, which is what lets a CUDA kernel (tree reduction) and this
    restatement (vector reduction) agree bit for bit.  1 / sqrt is the IEEE division and square
    root; x * factor * weight are two float32 multiplications."""
    ms = x.double().pow(2).mean(dim=-1, keepdim=True).to(torch.float32)
    factor = 1.0 / torch.sqrt(ms + torch.tensor(eps, dtype=torch.float32))
    return x * factor * weight


def rope_tail(x: torch.Tensor, freqs: torch.Tensor, pos: int) -> torch.Tensor:
    """Rotate the last 64 dims, interleaved pairs, table row [cos0,sin0,cos1,...]
    (mega_dsa_cp/tiles/compress_ref.py:83-95)."""
    out = x.clone()
    tail = x[..., -ROPE_DIM:].to(torch.float32)
    row = freqs[pos].to(torch.float32)
    c, s = row[0::2], row[1::2]
    re, im = tail[..., 0::2], tail[..., 1::2]
    rot = torch.stack((re * c - im * s, re * s + im * c), dim=-1).reshape(tail.shape)
    out[..., -ROPE_DIM:] = rot
    return out


def make_freqs(max_pos: int) -> torch.Tensor:
    """(P, 64) rope table (mega_dsa_cp/tiles/compress_ref.py:98-108)."""
    inv = torch.exp(-math.log(10000.0) * torch.arange(0, ROPE_DIM, 2, dtype=torch.float32) / ROPE_DIM)
    ang = torch.outer(torch.arange(max_pos, dtype=torch.float32), inv)
    return torch.stack([ang.cos(), ang.sin()], dim=-1).flatten(-2)


def pool_partial(kv, score, bias):
    """One rank's (m, l, w) over its slots: kv/score/bias (k, hd)
    (mega_dsa_cp/tiles/compress_ref.py:126-133)."""
    s = score + bias
    m = s.max(dim=0).values
    e = torch.exp(s - m)
    return m, e.sum(dim=0), (e * kv).sum(dim=0)


def pool_merge(parts):
    """Merge (m, l, w) partials -> pooled (hd,) (compress_ref.py:136-145)."""
    m = torch.stack([p[0] for p in parts]).max(dim=0).values
    num = sum(p[2] * torch.exp(p[0] - m) for p in parts)
    den = sum(p[1] * torch.exp(p[0] - m) for p in parts)
    return num / den


def pool_full(kv, score, bias):
    """Single-machine softmax pooling over all slots (compress_ref.py:114-123)."""
    w = torch.softmax(score + bias, dim=0)
    return (w * kv).sum(dim=0)


def online_fold(state, kv, score, bias):
    """Fold one token into (m, l, kv_norm) (compress_ref.py:152-165); an empty
    state is (None, None, None)."""
    s = score + bias
    m, l, kn = state
    if m is None:
        return s.clone(), torch.ones_like(s), kv.clone()
    m2 = torch.maximum(m, s)
    keep = l * torch.exp(m - m2)
    add = torch.exp(s - m2)
    l2 = keep + add
    return m2, l2, (kn * keep + kv * add) / l2


def online_merge(states):
    """Merge per-rank online states at chunk close, any number of ranks
    (two-rank form: compress_ref.py:168-174)."""
    m = torch.stack([s[0] for s in states]).max(dim=0).values
    num = sum(s[2] * (s[1] * torch.exp(s[0] - m)) for s in states)
    den = sum(s[1] * torch.exp(s[0] - m) for s in states)
    return num / den


def post_attn_e4m3(x, norm_w, eps, freqs, pos, fp8_scale):
    """RMS norm -> rope(last 64 @ pos) -> e4m3 bytes (compress_ref.py:181-185)."""
    y = rope_tail(rms_norm(x, norm_w, eps), freqs, pos)
    return (y / fp8_scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def post_attn_bf16(x, norm_w, eps, freqs, pos):
    """EXTENSION: same chain with a bf16 pool entry instead of e4m3."""
    return rope_tail(rms_norm(x, norm_w, eps), freqs, pos).to(torch.bfloat16)


def post_indexer(x, norm_w, eps, freqs, pos, fmt: str = FMT_MXFP4):
    """RMS norm -> rope -> staged Hadamard-128 -> FP4 quant, bit-exact path
    (compress_ref.py:219-223); fmt=nvfp4 is the EXTENSION."""
    y = hadamard128_staged(rope_tail(rms_norm(x, norm_w, eps), freqs, pos))
    return quant_mxfp4(y) if fmt == FMT_MXFP4 else quant_nvfp4(y)


def synth_record(b: int, pos: int, hd: int, dual_role: bool, seed: int = 0) -> torch.Tensor:
    """Deterministic compressor input record (compress_ref.py:242-256)."""
    g = torch.Generator(device="cpu").manual_seed(seed * 1_000_003 + b * 65_537 + pos * 257 + hd)
    rec = torch.randn((4 if dual_role else 2) * hd, generator=g, dtype=torch.float32)
    rec[(2 if dual_role else 1) * hd:] *= 3.0
    return rec


def synth_bias(hd: int, slots: int, seed: int = 1234) -> torch.Tensor:
    """compress_ref.py:262-264."""
    g = torch.Generator(device="cpu").manual_seed(seed + hd + slots)
    return torch.randn(slots, hd, generator=g, dtype=torch.float32) * 0.5


def csa_entry_ref(records: torch.Tensor, bias: torch.Tensor, n: int, hd: int) -> torch.Tensor:
    """Pooled value of ratio-4 entry n from the full token stream.
    records (S, 4*hd) = [kv_ov | kv_nm | s_ov | s_nm] per token; the window is
    the 8 tokens 4n-4 .. 4n+3, slots 0-3 in the overlap role (absent for n = 0),
    slots 4-7 in the normal role (mega_dsa_cp/tiles/compress.py:165-178)."""
    kv, sc, bs = [], [], []
    for j in range(8):
        tok = 4 * n - 4 + j
        if tok < 0:
            continue
        role = j // 4
        kv.append(records[tok, role * hd:(role + 1) * hd])
        sc.append(records[tok, (2 + role) * hd:(3 + role) * hd])
        bs.append(bias[j])
    return pool_full(torch.stack(kv), torch.stack(sc), torch.stack(bs))


def online_entry_ref(records: torch.Tensor, bias: torch.Tensor, n: int, hd: int, ratio: int):
    """Pooled value of ratio-R entry n: softmax pooling over tokens nR..nR+R-1
    with bias row = position in chunk (what the online machine of
    compress_ref.py:152-174 converges to)."""
    rows = records[n * ratio:(n + 1) * ratio]
    return pool_full(rows[:, :hd], rows[:, hd:2 * hd], bias[:ratio])


# --------------------------------------------------------------------------
# Composed context-parallel decode step (EXTENSION: the reference never
# assembled this chain; it is the composition its design documents describe)
# --------------------------------------------------------------------------

def shard_tokens(x: torch.Tensor, cp: int, rank: int) -> torch.Tensor:
    """Token-interleaved shard: global token t lives on rank t % cp at local
    index t // cp."""
    return x[rank::cp]


def select_topk_ref(q_idx, w_idx, k_idx_deq, seq_len: int, top_k: int, cp: int = 1):
    """Selection of one sequence, one query token: the exact global top-k of the indexer logits
    under (v desc, id asc), computed hierarchically (per-rank top-k of the token-interleaved
    shards, then the merge), in the merge's emit order.  q_idx (64,128), w_idx (64,), k_idx_deq
    (S,128) dequantised index keys."""
    S = seq_len
    logits = ((q_idx @ k_idx_deq[:S].T).clamp(min=0) * w_idx[:, None]).sum(dim=0)
    cand_v, cand_i = [], []
    for r in range(cp):
        loc = logits[r::cp]
        v, i = local_topk_ref(loc, 0, loc.numel(), loc.numel(), top_k, id_mul=cp, id_add=r)
        cand_v.append(v)
        cand_i.append(i)
    maxk = max(v.numel() for v in cand_v)
    cv = torch.zeros(1, 1, cp, maxk)
    ci = torch.zeros(1, 1, cp, maxk, dtype=torch.int32)
    cc = torch.zeros(1, 1, cp, dtype=torch.int32)
    for r in range(cp):
        n = cand_v[r].numel()
        cv[0, 0, r, :n], ci[0, 0, r, :n], cc[0, 0, r] = cand_v[r], cand_i[r], n
    _, sel_i, sel_c = merge_topk_ref(cv, ci, cc, top_k)
    return sel_i[0, 0, :int(sel_c[0, 0])].long()


def decode_step_ref(q_idx, w_idx, k_idx_deq, q_mla, kv_mla, seq_len: int, top_k: int,
                    softmax_scale: float, cp: int = 1, d_v: int = 512):
    """One sequence, one query token.  q_idx (64,128), w_idx (64,), k_idx_deq
    (S,128) dequantised index keys, q_mla (H,Dqk), kv_mla (S,Dqk).
    Returns (selected global ids (sorted ascending), o (H,d_v), lse (H,)) where the
    selection is select_topk_ref's and the attention is computed per rank over its
    share of the selection and merged by LSE."""
    sel = select_topk_ref(q_idx, w_idx, k_idx_deq, seq_len, top_k, cp)
    o, l = attend_selected_ref(q_mla, kv_mla, sel, softmax_scale, cp=cp, d_v=d_v)
    return torch.sort(sel).values, o, l


def attend_selected_ref(q_mla, kv_mla, sel, softmax_scale: float, cp: int = 1, d_v: int = 512,
                        rows_are_selected: bool = False):
    """Sparse attention of one query token over the GIVEN global token ids `sel`
    (any order), computed the context-parallel way: rank r attends over the ids
    with id % cp == r in the order given, the cp partials are merged by LSE.
    q_mla (H,Dqk); kv_mla (S,Dqk) indexed by id, or with rows_are_selected one row
    per entry of sel (row j = the KV row of sel[j]).  Returns (o (H,d_v), log2-LSE
    (H,)).  Lets a test hold a kernel's attention to the oracle on the kernel's
    own selection."""
    sel = sel.long()
    H = q_mla.shape[0]
    acc_o = torch.zeros(1, 1, cp, H, d_v)
    acc_l = torch.full((1, 1, cp, H), -math.inf)
    sink = torch.full((H,), -math.inf)
    where = torch.arange(sel.numel())
    for r in range(cp):
        m = sel % cp == r
        mine = where[m] if rows_are_selected else sel[m]
        n = mine.numel()
        pt = torch.zeros(1, max(n, 1), dtype=torch.int32)
        pt[0, :n] = mine.to(torch.int32)
        o, l = ref_mla(q_mla[None, None].float(), None, kv_mla.float(), None, pt,
                       torch.tensor([WIN_SLOTS + n]), torch.tensor([0]), sink,
                       softmax_scale, d_v=d_v)
        acc_o[0, 0, r], acc_l[0, 0, r] = o[0, 0], l[0, 0]
    o, l = lse_merge_ref(acc_o, acc_l, cp)
    return o[0, 0], l[0, 0]
