"""GPU parity tests of the four standalone tiles through the C ABI
(libmdc.so), against the CPU oracle and the golden fixtures."""

import math

import pytest
import torch

from conftest import load_npz
from dsa_inputs import indexer_case, mla_case, mla_oracle
from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _run_logits(case, blocks_per_chunk, fused_k=None, seq_lens=None, window_exclude=None, id_mul=1, id_add=0):
    from mega_dsa_cp_b200.tiles.logits import run_fp4_paged_mqa_logits

    B = case["q"].shape[0]
    T = case["q_len"]
    P = case["page_tokens"]
    max_pages = case["bt"].shape[1]
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    q_sf = None if case["q_sf"] is None else case["q_sf"].to(DEV)
    common = dict(fmt=case["fmt"], page_tokens=P, status=status)
    if fused_k is None:
        logits = torch.full((B * T, max_pages * P), float("nan"), device=DEV)
        run_fp4_paged_mqa_logits(case["fused"].to(DEV), case["q"].to(DEV), q_sf, case["w"].to(DEV),
                                 case["bt"].to(DEV), logits, blocks_per_chunk, **common)
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        return logits.cpu()
    n_chunks = -(-max_pages // blocks_per_chunk)
    cv = torch.full((B, T, n_chunks, fused_k), float("nan"), device=DEV)
    ci = torch.full((B, T, n_chunks, fused_k), -1, dtype=torch.int32, device=DEV)
    cc = torch.zeros((B, T, n_chunks), dtype=torch.int32, device=DEV)
    sl = None if seq_lens is None else seq_lens.to(DEV)
    run_fp4_paged_mqa_logits(case["fused"].to(DEV), case["q"].to(DEV), q_sf, case["w"].to(DEV),
                             case["bt"].to(DEV), None, blocks_per_chunk, seq_lens=sl,
                             cand_v=cv, cand_i=ci, cand_c=cc, top_k=fused_k,
                             window_exclude=window_exclude, id_mul=id_mul, id_add=id_add, **common)
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    return cv.cpu(), ci.cpu(), cc.cpu()


def _oracle_logits(case):
    return orc.ref_logits(case["q_deq"], case["w"], case["fused"], case["bt"], case["q_len"],
                          fmt=case["fmt"], page_tokens=case["page_tokens"])


def test_logits_golden_mxfp4_fp4q():
    """The reference's own format (MXFP4 pages of 128, FP4 query, q_len 2) on the
    golden inputs; tolerance of the reference's test (rtol 1e-3, atol 1e-4)."""
    g = load_npz("logits_mxfp4")
    case = {"fused": g["kv_fused"], "bt": g["bt"], "w": g["w"], "fmt": "mxfp4", "page_tokens": 128,
            "q_len": 2, "q": g["q_packed"], "q_sf": g["q_sf_atom"]}
    got = _run_logits(case, blocks_per_chunk=1)
    assert torch.allclose(got, g["logits"], rtol=1e-3, atol=1e-4), (got - g["logits"]).abs().max()


@pytest.mark.parametrize("fmt,P,T,q_fp4,B,S,bpc", [
    ("mxfp4", 128, 2, True, 4, 8192, 16),     # the reference test's shape
    ("nvfp4", 64, 1, False, 1, 4096, 16),     # BASELINE config 1 indexer
    ("nvfp4", 64, 1, False, 3, 8192, 37),     # ragged last chunk, odd pages per tile
    ("nvfp4", 128, 2, False, 2, 4096, 8),
    ("mxfp4", 128, 1, True, 2, 2048, 4),
    ("nvfp4", 64, 2, True, 2, 2048, 32),
])
def test_logits_vs_oracle(fmt, P, T, q_fp4, B, S, bpc):
    case = indexer_case(B, S, P, fmt, q_len=T, q_fp4=q_fp4, seed=1, pool_pages=B * (S // P) + 7)
    got = _run_logits(case, bpc)
    ref = _oracle_logits(case)
    assert not torch.isnan(got).any()
    # tolerance: dequantised-FP4 logits within 1e-3 relative (plus 1e-4 absolute for values near zero)
    assert torch.allclose(got, ref, rtol=1e-3, atol=1e-4), (got - ref).abs().max()


@pytest.mark.parametrize("fmt,P,T,K,bpc,S,seq,wex", [
    ("mxfp4", 128, 2, 512, 32, 8192, 8192, 128),   # the reference's fused test
    ("mxfp4", 128, 2, 1024, 32, 8192, 8000, 128),
    ("nvfp4", 64, 1, 2048, 128, 16384, 16384, 0),  # K = 2048 from 8192-token chunks
    ("nvfp4", 64, 1, 2048, 16, 4096, 4000, 0),     # chunk smaller than K: everything is a candidate
    ("nvfp4", 64, 1, 256, 64, 8192, 5000, 0),      # chunks beyond seq_len are empty
    ("nvfp4", 64, 1, 2048, 256, 32768, 31000, 0),  # 16384-token chunks (64 register keys per thread)
])
def test_fused_topk_exact_on_own_logits(fmt, P, T, K, bpc, S, seq, wex):
    B = 2
    case = indexer_case(B, S, P, fmt, q_len=T, q_fp4=(fmt == "mxfp4"), seed=2)
    logits = _run_logits(case, bpc)
    seq_lens = torch.tensor([seq, max(seq - 777, 1)], dtype=torch.int32)
    cv, ci, cc = _run_logits(case, bpc, fused_k=K, seq_lens=seq_lens, window_exclude=wex, id_mul=3, id_add=1)
    ref = _oracle_logits(case)
    n_chunks = cc.shape[-1]
    ct = bpc * P
    for b in range(B):
        limit = max(0, int(seq_lens[b]) - wex)
        for t in range(T):
            for c in range(n_chunks):
                ev, ei = orc.local_topk_ref(logits[b * T + t], c * ct, min((c + 1) * ct, S), limit, K, 3, 1)
                n = int(cc[b, t, c])
                assert n == ev.numel(), (b, t, c, n, ev.numel())
                # exact (bitwise, ordered) against the top-k of the kernel's own logits
                assert torch.equal(ci[b, t, c, :n], ei)
                assert torch.equal(cv[b, t, c, :n].view(torch.int32), ev.view(torch.int32))
                # and the same set as the oracle's logits would select, up to near-ties
                if n:
                    ov, oi = orc.local_topk_ref(ref[b * T + t], c * ct, min((c + 1) * ct, S), limit, K, 3, 1)
                    overlap = len(set(oi.tolist()) & set(ei.tolist())) / n
                    assert overlap >= 0.999, overlap


def _merge(v, i, c, K):
    from mega_dsa_cp_b200.tiles.merge import run_merge_topk

    B, q = v.shape[:2]
    ov = torch.zeros(B, q, K, dtype=torch.float32, device=DEV)
    oi = torch.zeros(B, q, K, dtype=torch.int32, device=DEV)
    oc = torch.zeros(B, q, dtype=torch.int32, device=DEV)
    dbg = torch.zeros(64, dtype=torch.int32, device=DEV)
    run_merge_topk(v.to(DEV), i.to(DEV), c.to(DEV), ov, oi, oc, dbg, top_k=K)
    torch.cuda.synchronize()
    assert dbg[0].item() == 0
    return ov.cpu(), oi.cpu(), oc.cpu()


def test_merge_golden_ordered_bitwise():
    g = load_npz("merge")
    for name in ("full", "var", "ties", "neginf", "tiny", "const"):
        K = int(g[f"{name}_k"])
        ov, oi, oc = _merge(g[f"{name}_v"], g[f"{name}_i"], g[f"{name}_c"], K)
        assert torch.equal(oc, g[f"{name}_oc"]), name
        assert torch.equal(oi, g[f"{name}_oi"]), name
        assert torch.equal(ov.view(torch.int32), g[f"{name}_ov"].view(torch.int32)), name


@pytest.mark.parametrize("B,q,L,maxK,K,mode", [
    (2, 2, 4, 512, 512, "full"), (2, 2, 4, 1024, 1024, "full"), (4, 2, 8, 512, 512, "var"),
    (2, 2, 4, 512, 512, "tiny"), (2, 2, 8, 512, 512, "ties"), (2, 2, 4, 512, 512, "const"),
    (2, 2, 8, 512, 512, "neginf"), (1, 2, 256, 128, 512, "full"), (2, 2, 1, 1024, 1024, "var"),
    (2, 1, 8, 2048, 2048, "full"), (1, 1, 6, 2048, 2048, "var"),
    (2, 1, 1, 2048, 2048, "full"), (2, 1, 4, 512, 2048, "full"), (2, 1, 4, 512, 2048, "neginf"),  # nothing to drop
])
def test_merge_vs_oracle_and_deterministic(B, q, L, maxK, K, mode):
    g = torch.Generator().manual_seed(B * 131 + L)
    v = torch.randn(B, q, L, maxK, generator=g)
    c = torch.full((B, q, L), maxK, dtype=torch.int32)
    if mode == "var":
        c = torch.randint(0, maxK + 1, (B, q, L), generator=g, dtype=torch.int32)
    if mode == "tiny":
        c = torch.randint(0, max(2, K // (4 * L) + 2), (B, q, L), generator=g, dtype=torch.int32)
    if mode == "ties":
        v = torch.randint(0, 16, (B, q, L, maxK), generator=g).float() / 8.0
    if mode == "const":
        v = torch.full((B, q, L, maxK), 0.5)
    if mode == "neginf":
        v = v.masked_fill(torch.rand(B, q, L, maxK, generator=g) < 0.3, -math.inf)
    ids = torch.empty(B, q, L, maxK, dtype=torch.int32)
    for b in range(B):
        for t in range(q):
            ids[b, t] = torch.randperm(1 << 24, generator=g)[: L * maxK].reshape(L, maxK).to(torch.int32)
    ids.view(-1)[0] = 0
    ids.view(-1)[1] = (1 << 31) - 1
    a = _merge(v, ids, c, K)
    b2 = _merge(v, ids, c, K)
    rv, ri, rc = orc.merge_topk_ref(v, ids, c, K)
    assert torch.equal(a[2], rc)
    assert torch.equal(a[1], ri)
    assert torch.equal(a[0].view(torch.int32), rv.view(torch.int32))
    assert all(torch.equal(x, y) for x, y in zip(a, b2))


def _lse(acc_o, acc_l, cp, out_dtype=torch.float32):
    from mega_dsa_cp_b200.tiles.lse_merge import run_lse_merge

    B, q, _, H, D = acc_o.shape
    o = torch.full((B, q, H, D), float("nan"), device=DEV, dtype=out_dtype)
    l = torch.full((B, q, H), float("nan"), device=DEV)
    run_lse_merge(acc_o.to(DEV), acc_l.to(DEV), o, l, cp)
    torch.cuda.synchronize()
    return o.cpu(), l.cpu()


def test_lse_merge_golden():
    g = load_npz("lse_merge")
    for cp in (1, 3, 4):
        o, l = _lse(g["acc_o"], g["acc_lse"], cp)
        ro, rl = g[f"o_cp{cp}"], g[f"lse_cp{cp}"]
        fin = torch.isfinite(rl)
        assert torch.equal(torch.isfinite(l), fin)
        assert (l - rl)[fin].abs().max() < 1e-5      # LSE / merge within 1e-5 in fp32
        assert (o - ro).abs().max() < 1e-5
        assert bool((o[~fin] == 0).all())


@pytest.mark.parametrize("B,q,cp,cp_max,mode,dt", [
    (4, 2, 2, 2, "full", torch.float32), (4, 2, 4, 8, "full", torch.float32),
    (4, 2, 2, 2, "sparse", torch.float32), (2, 2, 4, 4, "sparse", torch.float32),
    (2, 2, 2, 2, "allempty", torch.float32), (32, 2, 2, 2, "sparse", torch.float32),
    (8, 1, 8, 8, "sparse", torch.bfloat16), (3, 1, 8, 8, "full", torch.bfloat16),
])
def test_lse_merge_vs_oracle(B, q, cp, cp_max, mode, dt):
    g = torch.Generator().manual_seed(cp * 7 + B)
    H, D = 128, 512
    acc_o = (torch.randn(B, q, cp_max, H, D, generator=g) * 2.0).to(dt)
    acc_l = torch.randn(B, q, cp_max, H, generator=g) * 4.0 + 2.0
    if mode in ("sparse", "allempty"):
        acc_l = acc_l.masked_fill(torch.rand(B, q, cp_max, H, generator=g) < 0.35, -math.inf)
    if mode == "allempty":
        acc_l[:, :, :, : H // 4] = -math.inf
    o, l = _lse(acc_o, acc_l, cp, out_dtype=dt)
    ro, rl = orc.lse_merge_ref(acc_o.float(), acc_l, cp)
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(l), fin)
    assert (l - rl)[fin].abs().max() < 1e-5
    if dt == torch.float32:
        assert (o - ro).abs().max() < 1e-5
    else:
        assert torch.allclose(o.float(), ro, rtol=1e-2, atol=1e-2)  # bf16 output rounding
    assert bool((o.float()[~fin] == 0).all())


def _mla(case, sink, scale, out_dtype=torch.float32, n_splits=None, fp8_p=False, H=None):
    from mega_dsa_cp_b200.tiles.hca import run_sparse_mla

    B, T, Hh, _ = case["q"].shape
    o = torch.full((B, T, Hh, 512), float("nan"), device=DEV, dtype=out_dtype)
    l = torch.full((B, T, Hh), float("nan"), device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    d = lambda t: None if t is None else t.to(DEV)
    run_sparse_mla(d(case["q"]), d(case["kv_win"]), d(case["kv_cmp"]), d(case["pt_win"]), d(case["pt_cmp"]),
                   o, l, d(case["k_valid"]), d(case["win_valid"]), d(sink), scale,
                   n_splits=n_splits, fp8_p=fp8_p, status=status)
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    return o.cpu().float(), l.cpu()


@pytest.mark.parametrize("d_qk,H,n_sel,splits,win,sink_on", [
    (576, 128, [2048], 1, False, False),           # BASELINE config 1 attention
    (576, 128, [300, 37, 1, 0], 1, False, False),  # ragged, empty row
    (576, 64, [700, 64, 65], 4, False, False),     # KV splits + combine
    (512, 128, [500, 128], 1, True, True),         # window pool + sink
    (576, 128, [256, 255], None, True, False),
])
def test_sparse_mla_bf16_vs_oracle(d_qk, H, n_sel, splits, win, sink_on):
    rows = len(n_sel)
    case = mla_case(rows, 1, H, d_qk, 3000, n_sel, with_window=win, seed=5)
    scale = 1.0 / math.sqrt(576)
    sink = (torch.randn(H, generator=torch.Generator().manual_seed(1)) * 0.5 - 1.0) if sink_on else None
    o, l = _mla(case, sink, scale, n_splits=splits)
    ro, rl = mla_oracle(case, sink, scale)
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(l), fin)
    assert (l - rl)[fin].abs().max() < 1e-3 if fin.any() else True
    # attention output within 2e-2 absolute (bf16 probabilities in the P.V product)
    assert (o - ro).abs().max() < 2e-2, (o - ro).abs().max()
    assert bool((o[~fin] == 0).all())


def _fp8_case(gain):
    case = mla_case(2, 2, 128, 512, 2000, [512, 200, 384, 1], dtype=torch.float8_e4m3fn,
                    with_window=True, seed=9)
    case["win_valid"] = torch.tensor([128, 90, 1, 128], dtype=torch.int32)
    for k in ("q", "kv_cmp", "kv_win"):
        case[k] = (case[k].float() * gain).clamp(-448, 448).to(torch.float8_e4m3fn)
    return case


def test_sparse_mla_fp8_reference_mode():
    """fp8 operands, latent 512, window + sink, probabilities rounded through
    e4m3: the reference kernel's mode, against the online-softmax simulation
    with the reference test's tolerance (rtol = atol = 2e-2, LSE 1e-3).  The
    e4m3 rounding of P depends on the running maximum at the time a tile is
    processed; this kernel's tile is 64 slots, the reference's 128, so the
    simulation is run at 64 (a handful of elements may still flip one e4m3 step
    through exp2 round-off), and the 128-slot simulation is held to the same
    tolerance on all but a small fraction of elements."""
    sink = torch.randn(128, generator=torch.Generator().manual_seed(2)) * 0.5 - 1.0
    for gain in (200.0, 40.0):
        case = _fp8_case(gain)
        o, l = _mla(case, sink, 0.007, fp8_p=True, n_splits=1)
        ro, rl = mla_oracle(case, sink, 0.007, fp8_p=True, online_tile=64)
        bad = ((o - ro).abs() > 2e-2 + 2e-2 * ro.abs()).float().mean().item()
        assert bad < 1e-3, (gain, bad)
        assert torch.allclose(l, rl, rtol=1e-3, atol=1e-3)
        ro, rl = mla_oracle(case, sink, 0.007, fp8_p=True, online_tile=128)
        bad = ((o - ro).abs() > 2e-2 + 2e-2 * ro.abs()).float().mean().item()
        assert bad < 5e-2, (gain, bad)
        assert torch.allclose(l, rl, rtol=1e-3, atol=5e-3)


def test_sparse_mla_bf16_partial_output_and_paged_pool():
    case = mla_case(2, 1, 128, 576, 40, [16 * 30, 16 * 11 + 5], seed=11, page_cmp=16)
    scale = 1.0 / math.sqrt(576)
    o, l = _mla(case, None, scale, out_dtype=torch.bfloat16, n_splits=1)
    ro, rl = mla_oracle(case, None, scale)
    assert (o - ro).abs().max() < 2e-2
    assert (l - rl).abs().max() < 1e-3


def test_sparse_mla_dense_layer_and_window_only_layer():
    """The two layer variants that need no selection, through the same entry point: every compressed
    entry of the sequence in order (pages enumerated by dense_layer_tables), and the sliding window alone."""
    from mega_dsa_cp_b200.tiles.hca import dense_layer_tables

    g = torch.Generator().manual_seed(31)
    B, T, H, DQK, page = 3, 1, 128, 576, 16
    n_entries = torch.tensor([1024, 517, 16], dtype=torch.int32)           # 128 K / 128 = 1024 entries at most
    first = torch.tensor([0, 64, 130], dtype=torch.int32)
    case = mla_case(B, T, H, DQK, 200, [16] * B, with_window=True, seed=32, page_cmp=page)
    pt, k_valid = dense_layer_tables(n_entries, first, page)
    assert pt.shape == (B, 64) and pt[1, :33].tolist() == list(range(64, 97)) and int(pt[1, 33]) == 0
    case["pt_cmp"], case["k_valid"] = pt, k_valid
    case["win_valid"] = torch.tensor([128, 77, 0], dtype=torch.int32)
    scale = 1.0 / math.sqrt(DQK)
    sink = torch.randn(H, generator=g) * 0.5 - 1.0
    o, l = _mla(case, sink, scale, n_splits=None)
    ro, rl = mla_oracle(case, sink, scale)
    assert (o - ro).abs().max() < 2e-2 and (l - rl).abs().max() < 1e-3
    # window only: nothing beyond the 128 window slots
    case["k_valid"] = torch.full((B,), 128, dtype=torch.int32)
    case["pt_cmp"] = torch.zeros(B, 1, dtype=torch.int32)
    o, l = _mla(case, sink, scale, n_splits=1)
    ro, rl = mla_oracle(case, sink, scale)
    assert (o - ro).abs().max() < 2e-2 and (l - rl).abs().max() < 1e-3
    assert bool(torch.isfinite(l).all())      # the sink keeps the row with an empty window finite


@pytest.mark.parametrize("fmt,P,T,K,bpc,S,seq,wex", [
    ("nvfp4", 64, 1, 2048, 128, 32768, 32768, 0),    # BASELINE config 2 row: 4 chunks of 8192
    ("nvfp4", 64, 1, 2048, 64, 32768, 30011, 0),     # 8 chunks, ragged length
    ("nvfp4", 64, 1, 512, 32, 4096, 4096, 0),        # 2 chunks
    ("nvfp4", 64, 1, 2048, 16, 1024, 1024, 0),       # 1 chunk, fewer entries than k
    ("mxfp4", 128, 2, 1024, 32, 16384, 16000, 128),  # reference format, two query tokens, window excluded
])
def test_row_topk_equals_fused_plus_merge(fmt, P, T, K, bpc, S, seq, wex):
    """One-launch row mode (cluster-wide select) against fused candidates + merge: same
    entries in the same order, bit for bit."""
    from mega_dsa_cp_b200.tiles.logits import run_fp4_paged_mqa_logits
    from mega_dsa_cp_b200.tiles.merge import run_merge_topk

    B = 3
    case = indexer_case(B, S, P, fmt, q_len=T, q_fp4=(fmt == "mxfp4"), seed=5)
    seq_lens = torch.tensor([seq, max(seq - 1234, 1), min(seq, 700)], dtype=torch.int32)
    cv, ci, cc = _run_logits(case, bpc, fused_k=K, seq_lens=seq_lens, window_exclude=wex, id_mul=2, id_add=1)
    ov = torch.empty(B, T, K, device=DEV)
    oi = torch.empty(B, T, K, dtype=torch.int32, device=DEV)
    oc = torch.empty(B, T, dtype=torch.int32, device=DEV)
    run_merge_topk(cv.to(DEV), ci.to(DEV), cc.to(DEV), ov, oi, oc, None, top_k=K)
    rv = torch.full((B, T, K), float("nan"), device=DEV)
    ri = torch.full((B, T, K), -1, dtype=torch.int32, device=DEV)
    rc = torch.zeros(B, T, dtype=torch.int32, device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    q_sf = None if case["q_sf"] is None else case["q_sf"].to(DEV)
    for _ in range(2):  # twice: the second launch must not depend on what the first left behind
        run_fp4_paged_mqa_logits(case["fused"].to(DEV), case["q"].to(DEV), q_sf, case["w"].to(DEV), case["bt"].to(DEV),
                                 None, bpc, seq_lens=seq_lens.to(DEV), top_k=K, window_exclude=wex, id_mul=2, id_add=1,
                                 fmt=fmt, page_tokens=P, status=status, row_topk=(rv, ri, rc))
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    assert torch.equal(rc, oc)
    for b in range(B):
        for t in range(T):
            n = int(oc[b, t])
            assert torch.equal(ri[b, t, :n], oi[b, t, :n]), (b, t)
            assert torch.equal(rv[b, t, :n].view(torch.int32), ov[b, t, :n].view(torch.int32)), (b, t)


def test_row_topk_config2_full_size_exact_on_own_logits():
    """BASELINE config 2 at full size (B = 32 sequences of 32768 tokens, NVFP4 pages of 64,
    top-k 2048, one row-mode launch): on sampled sequences the ids and values are, bit for bit
    and in order, the top-k of the kernel's own logits under (value desc, position asc); every
    sequence returns exactly k entries, all distinct and in range.  Inputs are generated on the
    device (seeded) to keep the test short."""
    from mega_dsa_cp_b200.tiles.fp4 import fuse_pages
    from mega_dsa_cp_b200.tiles.logits import run_fp4_paged_mqa_logits

    B, S, P, K, bpc = 32, 32768, 64, 2048, 128
    g = torch.Generator(device=DEV).manual_seed(11)
    pages = S // P
    pool = B * pages
    cache = torch.cat([fuse_pages(torch.randn(pool // 8 * P, 128, generator=g, device=DEV), "nvfp4", P)[0]
                       for _ in range(8)])
    bt = torch.randperm(pool, generator=g, device=DEV).to(torch.int32).reshape(B, pages).contiguous()
    q = torch.randn(B, 64, 128, generator=g, device=DEV).to(torch.bfloat16)
    w = (torch.randn(B, 64, generator=g, device=DEV) / 64.0).contiguous()
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    logits = torch.full((B, S), float("nan"), device=DEV)
    run_fp4_paged_mqa_logits(cache, q, None, w, bt, logits, bpc, fmt="nvfp4", page_tokens=P, status=status)
    rv = torch.full((B, 1, K), float("nan"), device=DEV)
    ri = torch.full((B, 1, K), -1, dtype=torch.int32, device=DEV)
    rc = torch.zeros(B, 1, dtype=torch.int32, device=DEV)
    run_fp4_paged_mqa_logits(cache, q, None, w, bt, None, bpc, top_k=K, fmt="nvfp4", page_tokens=P, status=status,
                             row_topk=(rv, ri, rc))
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    assert not torch.isnan(logits).any()
    assert bool((rc == K).all())
    srt = torch.sort(ri[:, 0], dim=-1).values
    assert bool((srt[:, 1:] > srt[:, :-1]).all()) and int(srt.min()) >= 0 and int(srt.max()) < S
    # every selected value is the logit at its id, and nothing outside the selection beats the smallest selected value
    assert torch.equal(torch.gather(logits, 1, ri[:, 0].long()).view(torch.int32), rv[:, 0].view(torch.int32))
    masked = logits.clone()
    masked.scatter_(1, ri[:, 0].long(), float("-inf"))
    assert bool((masked.max(dim=1).values <= rv[:, 0].min(dim=1).values).all())
    lg, ri_c, rv_c = logits.cpu(), ri.cpu(), rv.cpu()
    for b in (0, 7, 13, 22, 31):
        ev, ei = orc.local_topk_ref(lg[b], 0, S, S, K, 1, 0)
        assert torch.equal(ri_c[b, 0], ei), b
        assert torch.equal(rv_c[b, 0].view(torch.int32), ev.view(torch.int32)), b
    # one sampled sequence against the oracle's logits (dequantised FP4, fp32): 1e-3 relative
    b = 13
    data, sf = orc.split_index_pages(cache[bt[b].long()].cpu(), "nvfp4", P)
    kd = orc.dequant_fp4(data, sf, "nvfp4").reshape(S, 128)
    ref = ((q[b].float().cpu() @ kd.T).clamp(min=0) * w[b].cpu()[:, None]).sum(dim=0)
    assert torch.allclose(lg[b], ref, rtol=1e-3, atol=1e-4), (lg[b] - ref).abs().max()
