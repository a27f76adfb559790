"""GPU tests of the KV compressor through the C ABI.  Several ranks are
emulated on one GPU by running their kernels one after the other on separate
buffers whose "peer offsets" are the address differences of those buffers: a
finalize launch then always finds its statistics already pushed, so no kernel
ever waits for a later launch."""

import pytest
import torch

from oracle import dsa_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


class FakeWorld:
    """cp ranks' event cells and arenas as plain tensors on one device."""

    def __init__(self, cp, n_events, arena_bytes):
        from mega_dsa_cp_b200.comm.buffers import SymmetricArena
        from mega_dsa_cp_b200.events.symm import EventBuffer

        ev = [torch.zeros(n_events * 16, dtype=torch.int64, device=DEV) for _ in range(cp)]
        ar = [torch.zeros(arena_bytes, dtype=torch.uint8, device=DEV) for _ in range(cp)]
        off = lambda ts, r: torch.tensor([t.data_ptr() - ts[r].data_ptr() for t in ts], dtype=torch.int64, device=DEV)
        self.events = [EventBuffer(n_events, r, cp, ev[r], off(ev, r)) for r in range(cp)]
        self.arenas = [SymmetricArena(arena_bytes, 1, r, cp, ar[r], off(ar, r), 0, None, {"stats": 0}) for r in range(cp)]


def test_hadamard_quant_micro_bit_exact():
    from mega_dsa_cp_b200.tiles.compress import launch_micro

    g = torch.Generator().manual_seed(1)
    x = torch.randn(64, 128, generator=g) * torch.logspace(-2, 2, 64).unsqueeze(1)
    out = torch.zeros(64, 68, dtype=torch.uint8, device=DEV)
    launch_micro(x.to(DEV), out)
    torch.cuda.synchronize()
    pk, sf = orc.quant_mxfp4(orc.hadamard128_staged(x))
    assert torch.equal(out[:, :64].cpu(), pk)
    assert torch.equal(out[:, 64:].cpu(), sf)


def _e4m3_rank(codes: torch.Tensor) -> torch.Tensor:
    """e4m3 bytes -> position on the value axis (adjacent representable values differ by 1; -0 = +0)."""
    c = codes.view(torch.uint8).int()
    mag = c & 0x7f
    return torch.where((c & 0x80) != 0, -mag, mag)


def _post_checks(st, b, slot, pooled_attn, pooled_idx, pos, norm_a, norm_i, freqs, fp8_scale, tag, tally):
    """The owner's entry against the oracle.  The pooled fp32 values (before the norm) within fp32
    round-off of single-machine pooling; then, with the kernel's OWN pooled value as the input of
    the oracle's post chain: the MXFP4 codes and the UE8M0 bytes bit for bit (the reference's bar,
    docs/phase1.3-compressor-tile.md:78-82: 0 of 38400 nibbles), every e4m3 code equal or the
    neighbouring code (the kernel multiplies by 1/scale where the oracle divides by scale)."""
    got = st.dbg_attn[b, slot].cpu()
    assert torch.allclose(got, pooled_attn, rtol=2e-4, atol=2e-5), (tag, (got - pooled_attn).abs().max())
    want = _e4m3_rank(orc.post_attn_e4m3(got, norm_a, 1e-6, freqs, pos, fp8_scale))
    have = _e4m3_rank(st.attn_pool[b, slot].cpu())
    assert int((want - have).abs().max()) <= 1, (tag, int((want - have).abs().max()))
    tally["e4m3"] += want.numel()
    tally["e4m3_off_by_one"] += int((want != have).sum())
    if pooled_idx is not None:
        gi = st.dbg_idx[b, slot].cpu()
        assert torch.allclose(gi, pooled_idx, rtol=2e-4, atol=2e-5), tag
        pk, sf = orc.post_indexer(gi, norm_i, 1e-6, freqs, pos)
        page = st.idx_pool[b, slot // 128].cpu()
        tok = slot % 128
        data = page[tok * 64:(tok + 1) * 64]
        sfb = page[8192 + (tok % 32) * 16 + (tok // 32) * 4: 8192 + (tok % 32) * 16 + (tok // 32) * 4 + 4]
        assert torch.equal(sfb, sf), (tag, sfb.tolist(), sf.tolist())
        assert torch.equal(data, pk), (tag, int((data != pk).sum()))
        tally["nibbles"] += 2 * pk.numel()


@pytest.mark.parametrize("cp", [1, 2, 4, 8])
def test_window_machine_roll(cp):
    """ratio 4, one token per step, B = 2, 26 steps: every closing step's entry
    against single-machine pooling of the full token stream."""
    from mega_dsa_cp_b200.tiles.compress import CompressorState, launch_finalize, launch_step, CSA_STATS_BYTES

    B, steps, E = 2, 26, 128   # 6 closing groups per sequence
    world = FakeWorld(cp, B, B * cp * CSA_STATS_BYTES)
    sts = [CompressorState(B, cp, r, 4, E) for r in range(cp)]
    ape_a, ape_i = orc.synth_bias(512, 8), orc.synth_bias(128, 8)
    g = torch.Generator().manual_seed(2)
    norm_a, norm_i = torch.rand(512, generator=g) + 0.5, torch.rand(128, generator=g) + 0.5
    freqs = orc.make_freqs(256)
    d = lambda t: t.to(DEV)
    dev = dict(ape_a=d(ape_a), ape_i=d(ape_i), na=d(norm_a), ni=d(norm_i), fr=d(freqs))
    rec_a = torch.stack([torch.stack([orc.synth_record(b, p, 512, True) for p in range(steps)]) for b in range(B)])
    rec_i = torch.stack([torch.stack([orc.synth_record(b, p, 128, True) for p in range(steps)]) for b in range(B)])
    tally = {"e4m3": 0, "e4m3_off_by_one": 0, "nibbles": 0}
    for s in range(steps):
        seq = torch.full((B,), s, dtype=torch.int32, device=DEV)
        na, ni = d(rec_a[:, s].contiguous()), d(rec_i[:, s].contiguous())
        for r in range(cp):
            launch_step(sts[r], seq, na, ni, dev["ape_a"], dev["ape_i"], world.arenas[r], "stats", world.events[r])
        for r in range(cp):
            launch_finalize(sts[r], seq, world.arenas[r], "stats", world.events[r], s, dev["na"], dev["ni"], 1e-6,
                            dev["fr"], fp8_scale=0.02)
        torch.cuda.synchronize()
        for r in range(cp):
            assert sts[r].status[0].item() == 0, sts[r].status.tolist()
        if (s + 1) % 4 == 0:
            n = s // 4
            owner, slot = n % cp, n // cp
            for b in range(B):
                pa = orc.csa_entry_ref(rec_a[b], ape_a, n, 512)
                pi = orc.csa_entry_ref(rec_i[b], ape_i, n, 128)
                _post_checks(sts[owner], b, slot, pa, pi, 4 * n, norm_a, norm_i, freqs, 0.02, (cp, s, b), tally)
            assert sts[owner].k_valid.tolist() == [slot + 1] * B
    assert tally["nibbles"] == 6 * B * 128 and tally["e4m3_off_by_one"] <= tally["e4m3"] // 100, tally


@pytest.mark.parametrize("cp,ratio", [(1, 64), (4, 64), (2, 128)])
def test_online_machine_roll(cp, ratio):
    from mega_dsa_cp_b200.tiles.compress import CompressorState, launch_finalize, launch_step, ONLINE_STATS_BYTES

    B, steps, E = 2, 2 * ratio + 5, 16
    world = FakeWorld(cp, B, B * cp * ONLINE_STATS_BYTES)
    sts = [CompressorState(B, cp, r, ratio, E, attn_dtype=torch.bfloat16) for r in range(cp)]
    bias = orc.synth_bias(512, ratio)
    g = torch.Generator().manual_seed(3)
    norm_a = torch.rand(512, generator=g) + 0.5
    freqs = orc.make_freqs(4 * ratio)
    d = lambda t: t.to(DEV)
    dbias, dn, dfr = d(bias), d(norm_a), d(freqs)
    rec = torch.stack([torch.stack([orc.synth_record(b, p, 512, False, seed=3) for p in range(steps)]) for b in range(B)])
    for s in range(steps):
        seq = torch.full((B,), s, dtype=torch.int32, device=DEV)
        nr = d(rec[:, s].contiguous())
        for r in range(cp):
            launch_step(sts[r], seq, nr, None, dbias, None, world.arenas[r], "stats", world.events[r])
        for r in range(cp):
            launch_finalize(sts[r], seq, world.arenas[r], "stats", world.events[r], s, dn, None, 1e-6, dfr)
        if (s + 1) % ratio == 0:
            torch.cuda.synchronize()
            n = s // ratio
            owner, slot = n % cp, n // cp
            assert sts[owner].status[0].item() == 0
            for b in range(B):
                want = orc.online_entry_ref(rec[b], bias, n, 512, ratio)
                got = sts[owner].dbg_attn[b, slot].cpu()
                assert torch.allclose(got, want, rtol=2e-4, atol=2e-5), (cp, s, b, (got - want).abs().max())
                ent = orc.post_attn_bf16(got, norm_a, 1e-6, freqs, n * ratio).float()
                have = sts[owner].attn_pool[b, slot].cpu().float()
                assert torch.equal(have, ent), (cp, s, b, (have - ent).abs().max())   # same fp32 chain, same bf16 rounding
            assert sts[owner].k_valid.tolist() == [slot + 1] * B
