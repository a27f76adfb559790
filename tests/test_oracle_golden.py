"""Pins oracle/dsa_oracle.py to the outputs of the reference's own torch code
(fixtures under tests/golden, produced by tests/golden/make_golden.py)."""

import math

import torch

from conftest import load_npz
from oracle import dsa_oracle as orc


def test_mxfp4_quant_dequant_bit_exact():
    g = load_npz("fp4")
    packed, sf = orc.quant_mxfp4(g["x"])
    assert torch.equal(packed, g["packed"])
    assert torch.equal(sf, g["sf"])
    assert torch.equal(orc.dequant_fp4(g["packed"], g["sf"], orc.FMT_MXFP4), g["deq"])
    assert torch.equal(orc.sf_to_atom(g["sf_plain"]), g["sf_atom"])
    assert torch.equal(orc.atom_to_sf(g["sf_atom"]), g["sf_plain"])


def test_logits_mxfp4_matches_reference():
    g = load_npz("logits_mxfp4")
    q = orc.dequant_fp4(g["q_packed"], g["q_sf"], orc.FMT_MXFP4)
    out = orc.ref_logits(q, g["w"], g["kv_fused"], g["bt"], q_len=2)
    # same fp32 matmul, same order: bitwise on CPU
    assert torch.allclose(out, g["logits"], rtol=1e-6, atol=1e-6)
    data, sf = orc.split_index_pages(g["kv_fused"], orc.FMT_MXFP4, 128)
    assert torch.equal(sf.reshape(4, 128, 4), g["kv_sf"])


def test_merge_topk_matches_reference_ordered_bitwise():
    g = load_npz("merge")
    for name in ("full", "var", "ties", "neginf", "tiny", "const"):
        ov, oi, oc = orc.merge_topk_ref(g[f"{name}_v"], g[f"{name}_i"], g[f"{name}_c"], int(g[f"{name}_k"]))
        assert torch.equal(oc, g[f"{name}_oc"]), name
        assert torch.equal(oi, g[f"{name}_oi"]), name
        assert torch.equal(ov.view(torch.int32), g[f"{name}_ov"].view(torch.int32)), name


def test_lse_merge_matches_reference():
    g = load_npz("lse_merge")
    for cp in (1, 3, 4):
        o, l = orc.lse_merge_ref(g["acc_o"], g["acc_lse"], cp)
        assert torch.equal(torch.isinf(l), torch.isinf(g[f"lse_cp{cp}"]))
        fin = torch.isfinite(l)
        assert torch.allclose(l[fin], g[f"lse_cp{cp}"][fin], rtol=0, atol=1e-6)
        assert torch.allclose(o, g[f"o_cp{cp}"], rtol=0, atol=1e-6)


def _hca_inputs(g):
    f8 = lambda t: t.view(torch.float8_e4m3fn).float()
    return f8(g["q"]), f8(g["kwin"]), f8(g["kcmp"]), f8(g["kcmp16"])


def test_mla_matches_reference_all_modes():
    g = load_npz("hca")
    q, kwin, kcmp, kcmp16 = _hca_inputs(g)
    pt_win = torch.arange(2, dtype=torch.int32).repeat_interleave(2).view(4, 1)
    H = q.shape[2]
    for tag, sink in (("nosink", torch.full((H,), -math.inf)), ("sink", g["sink_on"])):
        for suffix, kw in (("_fp8p", dict(fp8_p=True)), ("", dict(fp8_p=False)),
                           ("_online", dict(fp8_p=True, online_tile=128))):
            o, l = orc.ref_mla(q, kwin, kcmp, pt_win, g["pt_cmp"], g["k_valid"], g["win_valid"],
                               sink, float(g["scale"]), d_v=q.shape[-1], **kw)
            ro, rl = g[f"{tag}_o{suffix}"], g[f"{tag}_l{suffix}"]
            # the reference's online simulation turns a fully masked leading tile
            # into NaN (it never tests that case); those rows are left out
            good = ~torch.isnan(ro).any(dim=-1)
            assert bool(good.any())
            assert torch.equal(torch.isfinite(l)[good], torch.isfinite(rl)[good])
            fin = torch.isfinite(rl) & good
            assert torch.allclose(l[fin], rl[fin], rtol=0, atol=2e-6), (tag, suffix)
            assert torch.allclose(o[good], ro[good], rtol=1e-5, atol=1e-5), (tag, suffix)
    o, l = orc.ref_mla(q, kwin, kcmp16, pt_win, g["pt16"], g["k_valid16"], g["win_valid"],
                       g["sink_on"], float(g["scale"]), d_v=q.shape[-1], page_cmp=16)
    assert torch.allclose(o, g["paged_o"], rtol=1e-5, atol=1e-5)
    o, l = orc.ref_mla(q, kwin, kcmp16, pt_win, g["pt16"], g["k_valid16"], g["win_valid"],
                       g["sink_on"], float(g["scale"]), d_v=q.shape[-1], page_cmp=16,
                       fp8_p=True, online_tile=128)
    assert torch.allclose(o, g["paged_o_online"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(l, g["paged_l_online"], rtol=0, atol=2e-6)


def test_compressor_pieces_match_reference():
    g = load_npz("compress")
    assert torch.equal(orc.hadamard128_staged(g["x"]), g["had"])
    assert torch.allclose(orc.hadamard128_staged(g["x"]), g["had_m"], atol=1e-5)
    assert torch.equal(orc.make_freqs(64), g["freqs"])
    normed = orc.rms_norm(g["y"], g["w512"], 1e-6)
    assert torch.equal(normed, g["normed"])
    assert torch.allclose(orc.rope_tail(normed, g["freqs"], 17), g["roped"], rtol=0, atol=1e-7)
    e4 = orc.post_attn_e4m3(g["y"][0], g["w512"], 1e-6, g["freqs"], 17, 0.02)
    assert torch.equal(e4.view(torch.uint8), g["e4"])
    pk, sf = orc.post_indexer(g["yi"], g["w128"], 1e-6, g["freqs"], 12)
    assert torch.equal(pk, g["idx_packed"]) and torch.equal(sf, g["idx_sf"])
    pk, sf = orc.quant_mxfp4(g["qx"])
    assert torch.equal(pk, g["q_packed"]) and torch.equal(sf, g["q_sf"])
    full = orc.pool_full(g["kv"], g["sc"], g["ape"])
    assert torch.allclose(full, g["pool_full"], rtol=1e-6, atol=1e-7)
    p0 = orc.pool_partial(g["kv"][0::2], g["sc"][0::2], g["ape"][0::2])
    p1 = orc.pool_partial(g["kv"][1::2], g["sc"][1::2], g["ape"][1::2])
    for a, b in zip(p0, (g["p0_m"], g["p0_l"], g["p0_w"])):
        assert torch.equal(a, b)
    assert torch.equal(orc.pool_merge([p0, p1]), g["pool_merged"])
    assert torch.equal(orc.synth_bias(128, 8), g["ape"])
    assert torch.equal(orc.synth_bias(512, 16), g["bias128"])
    assert torch.equal(orc.synth_record(2, 7, 128, True, seed=0), g["rec_dual"])
    st = [(None, None, None), (None, None, None)]
    for p in range(12):
        rec = orc.synth_record(1, p, 512, False, seed=3)
        assert torch.equal(rec, g["recs"][p])
        st[p % 2] = orc.online_fold(st[p % 2], rec[:512], rec[512:], g["bias128"][p])
    for a, b in zip(st[0], (g["st0_m"], g["st0_l"], g["st0_k"])):
        assert torch.equal(a, b)
    assert torch.equal(orc.online_merge(st), g["merged128"])
    # the online machine converges to one-shot pooling over the chunk
    want = orc.online_entry_ref(g["recs"], g["bias128"], 0, 512, 12)
    assert torch.allclose(orc.online_merge(st), want, rtol=1e-5, atol=1e-5)


def test_nvfp4_extension_reduces_to_pinned_pieces():
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(64, 128, generator=gen) * torch.logspace(-0.5, 1, 64).unsqueeze(1)
    packed, sf = orc.quant_nvfp4(x)
    deq = orc.dequant_fp4(packed, sf, orc.FMT_NVFP4)
    assert sf.shape == (64, 8) and packed.shape == (64, 64)
    xb = x.bfloat16().float()
    grp = xb.reshape(64, 8, 16)
    # error bound: half an E2M1 step (1.0 at the top) plus the clamp after the scale itself rounded down
    scale = orc.ue4m3_to_float(sf).unsqueeze(-1)
    assert bool(((deq.reshape(64, 8, 16) - grp).abs() <= 1.5 * scale + 1e-6).all())
    # codes decode through the same E2M1 table the MXFP4 path is pinned on
    unit = orc.dequant_fp4(packed, torch.full_like(sf, 0x38), orc.FMT_NVFP4)  # 0x38 = 1.0 in e4m3
    assert set(unit.abs().unique().tolist()) <= set(orc.E2M1_VALUES)
    fused, sf_plain = orc.build_index_pages(x, orc.FMT_NVFP4, 64)
    assert fused.shape == (1, 4608)
    d2, s2 = orc.split_index_pages(fused, orc.FMT_NVFP4, 64)
    assert torch.equal(d2, packed) and torch.equal(s2, sf)


def test_decode_step_cp_invariance():
    """The composed step gives the same selection and output for every cp."""
    gen = torch.Generator().manual_seed(0)
    S, K = 1024, 128
    q_idx = torch.randn(64, 128, generator=gen).bfloat16().float()
    w = torch.randn(64, generator=gen) / 64
    kraw = torch.randn(S, 128, generator=gen)
    pk, sf = orc.quant_nvfp4(kraw)
    kd = orc.dequant_fp4(pk, sf, orc.FMT_NVFP4)
    q_mla = (torch.randn(16, 96, generator=gen) * 0.5).bfloat16().float()
    kv = (torch.randn(S, 96, generator=gen) * 0.5).bfloat16().float()
    base = orc.decode_step_ref(q_idx, w, kd, q_mla, kv, S, K, 1 / math.sqrt(96), cp=1, d_v=64)
    for cp in (2, 4, 8):
        sel, o, l = orc.decode_step_ref(q_idx, w, kd, q_mla, kv, S, K, 1 / math.sqrt(96), cp=cp, d_v=64)
        assert torch.equal(sel, base[0])
        assert torch.allclose(o, base[1], atol=1e-5) and torch.allclose(l, base[2], atol=1e-5)
