"""KV compressor: host runners over mdc_compress_step_launch /
mdc_compress_finalize_launch (csrc/compress.cu).

Two pooling machines, both context-parallel (per-rank partial statistics ->
bulk push to the entry owner -> owner finalises):

* ratio 4: overlapping 8-slot window, attention (512) + indexer (128) streams;
  the owner writes an e4m3 (or bf16) attention entry and a Hadamard-rotated FP4
  indexer entry (with its block scale) into the fused index page.
* ratio 64 / 128: online per-channel softmax state [m | l | kv], attention
  stream only.

launch_step / launch_finalize take a CompressorState; launch_csa_step /
launch_csa_finalize / launch_c128_step / launch_c128_finalize / launch_micro
keep the names and argument order of mega_dsa_cp/tiles/compress.py (:253,
:526, :643, :795, :892) of the reference, generalised from cp = 2, q_len = 2
to any cp and q_len <= cp.  Inside the decode megakernel the same tiles run as
CMP_STEP / CMP_FIN tasks (layer.py).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .. import _native as N
from ..comm.buffers import SymmetricArena
from ..events.symm import EventBuffer

HD_ATTN, HD_IDX, ROPE_DIM, RING = 512, 128, 64, 8
REC_ATTN, REC_IDX, REC_ONLINE = 4 * HD_ATTN, 4 * HD_IDX, 2 * HD_ATTN
CSA_STATS_BYTES = 7696
ONLINE_STATS_BYTES = 6160
HADAMARD_SCALE = 0.0883883461356163


def stats_bytes(ratio: int) -> int:
    return CSA_STATS_BYTES if ratio == 4 else ONLINE_STATS_BYTES


@dataclass
class CompressorState:
    """Per-rank persistent state and pools of one compressor (ratio 4 or online)."""

    B: int
    cp: int
    rank: int
    ratio: int
    max_entries: int
    q_len: int = 1
    device: str = "cuda"
    attn_dtype: torch.dtype = torch.float8_e4m3fn
    idx_fmt: str = "mxfp4"
    idx_page_tokens: int = 128
    ring_attn: torch.Tensor = field(init=False, default=None)
    ring_idx: torch.Tensor = field(init=False, default=None)
    state: torch.Tensor = field(init=False, default=None)

    def __post_init__(self):
        dev, B, E = self.device, self.B, self.max_entries
        if self.ratio == 4:
            self.ring_attn = torch.zeros(B, RING, REC_ATTN, device=dev)
            self.ring_idx = torch.zeros(B, RING, REC_IDX, device=dev)
            pb = self.idx_page_tokens * (64 + (4 if self.idx_fmt == "mxfp4" else 8))
            self.idx_pool = torch.zeros(B, E // self.idx_page_tokens, pb, dtype=torch.uint8, device=dev)
            self.dbg_idx = torch.zeros(B, E, HD_IDX, device=dev)
        else:
            self.state = torch.zeros(B, 3, HD_ATTN, device=dev)
            self.state[:, 0] = -1.0e30
            self.idx_pool = None
            self.dbg_idx = None
        self.attn_pool = torch.zeros(B, E, HD_ATTN, device=dev).to(self.attn_dtype)
        self.dbg_attn = torch.zeros(B, E, HD_ATTN, device=dev)
        self.k_valid = torch.zeros(B, dtype=torch.int32, device=dev)
        self.status = torch.zeros(8, dtype=torch.int32, device=dev)


def _params(st: CompressorState, seq_len, arena: SymmetricArena, stats_region: str, events: EventBuffer,
            ev_base_id: int, phase: int, do_push: bool = True, wait_budget_ns: int = 2_000_000_000):
    p = N.CompressParams()
    p.B, p.cp, p.rank, p.q_len, p.ratio, p.phase = st.B, st.cp, st.rank, st.q_len, st.ratio, phase
    p.seq_len = N.ptr(seq_len)
    p.ring_attn, p.ring_idx, p.state = N.ptr(st.ring_attn), N.ptr(st.ring_idx), N.ptr(st.state)
    p.arena = N.PeerBufferC(arena.tensor.data_ptr(), arena.offsets.data_ptr(), arena.rank, arena.world_size, arena.mc_base)
    p.stats_off = arena.region_off(stats_region, 0)
    p.events = N.EventSetC(events.tensor.data_ptr(), events.offsets.data_ptr(), events.rank, events.world_size)
    p.ev_base_id, p.do_push, p.wait_budget_ns = ev_base_id, int(do_push), wait_budget_ns
    p.status = N.ptr(st.status)
    return p


def launch_step(st: CompressorState, seq_len, new_attn, new_idx, ape_attn, ape_idx, arena, stats_region, events,
                ev_base_id: int = 0, do_push: bool = True, stream=None) -> None:
    """Append this rank's new record(s), and on a closing step push this rank's
    statistics to the entry owner; bumps the sequence's event cell on all ranks."""
    p = _params(st, seq_len, arena, stats_region, events, ev_base_id, 0, do_push)
    p.new_attn, p.new_idx = N.ptr(new_attn), N.ptr(new_idx)
    p.ape_attn, p.ape_idx = N.ptr(ape_attn), N.ptr(ape_idx)
    N.call("mdc_compress_step_launch", p, stream)
    st._keep = (seq_len, new_attn, new_idx, ape_attn, ape_idx)


def launch_finalize(st: CompressorState, seq_len, arena, stats_region, events, phase: int, norm_w_attn, norm_w_idx,
                    norm_eps: float, freqs, fp8_scale: float = 1.0, ev_base_id: int = 0,
                    wait_budget_ns: int = 2_000_000_000, stream=None) -> None:
    """On the owner of a closing entry: wait for the cp statistics, merge,
    RMS-norm, rope, quantise, write the pools, bump k_valid."""
    p = _params(st, seq_len, arena, stats_region, events, ev_base_id, phase, True, wait_budget_ns)
    fill_finalize_params(p, st, norm_w_attn, norm_w_idx, norm_eps, freqs, fp8_scale)
    N.call("mdc_compress_finalize_launch", p, stream)


def fill_finalize_params(p, st: CompressorState, norm_w_attn, norm_w_idx, norm_eps: float, freqs, fp8_scale: float = 1.0):
    """The finalize-side fields of an mdc_compress_params for the state `st`."""
    p.norm_w_attn, p.norm_w_idx, p.freqs = N.ptr(norm_w_attn), N.ptr(norm_w_idx), N.ptr(freqs)
    p.freq_rows, p.norm_eps, p.inv_fp8_scale = freqs.shape[0], norm_eps, 1.0 / fp8_scale
    p.attn_pool_dtype = N.DT_E4M3 if st.attn_dtype == torch.float8_e4m3fn else N.DT_BF16
    p.attn_pool, p.idx_pool = N.ptr(st.attn_pool), N.ptr(st.idx_pool)
    p.idx_fmt = N.FMT_MXFP4 if st.idx_fmt == "mxfp4" else N.FMT_NVFP4
    p.idx_page_tokens, p.max_entries = st.idx_page_tokens, st.max_entries
    p.k_valid, p.dbg_attn, p.dbg_idx = N.ptr(st.k_valid), N.ptr(st.dbg_attn), N.ptr(st.dbg_idx)


# ---------------------------------------------------------------------------
# The reference's launchers, same names and argument order (mega_dsa_cp/tiles/compress.py:253-272,
# 526-551, 643-658, 795-816, 892-902).  There they are CuTe-DSL entry points compiled once and then
# called with raw pointers; here every "pointer" is a device address (int) or a torch tensor.  The
# reference hard-codes cp = 2, two new tokens per step and a record ring of 4 slots; those are the
# defaults of the trailing keyword arguments.
# ---------------------------------------------------------------------------
def _addr(x):
    return None if x is None else (x.data_ptr() if torch.is_tensor(x) else int(x))


def _raw_params(b_count, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank, ratio, cp, q_len):
    p = N.CompressParams()
    p.B, p.cp, p.rank, p.q_len, p.ratio = b_count, cp, int(my_rank), q_len, ratio
    p.seq_len = _addr(seq_len)
    p.arena = N.PeerBufferC(_addr(pay_base), _addr(pay_offsets), int(my_rank), cp, int(mc_base))
    p.stats_off = int(stats_off)
    p.events = N.EventSetC(_addr(ev_base), _addr(ev_offsets), int(my_rank), cp)
    p.wait_budget_ns = 2_000_000_000
    p.do_push = 1
    return p


def launch_csa_step(b_count, ring_attn, ring_idx, new_attn, new_idx, ape_attn, ape_idx, seq_len, pay_base, pay_offsets,
                    mc_base, stats_off, ev_base, ev_offsets, my_rank, do_push, stream=None, *, cp=2, q_len=2, ring_slots=4):
    p = _raw_params(b_count, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank, 4, cp, q_len)
    p.ring_attn, p.ring_idx, p.new_attn, p.new_idx = _addr(ring_attn), _addr(ring_idx), _addr(new_attn), _addr(new_idx)
    p.ape_attn, p.ape_idx, p.do_push, p.ring_slots = _addr(ape_attn), _addr(ape_idx), int(do_push), ring_slots
    N.call("mdc_compress_step_launch", p, stream)


def launch_csa_finalize(b_count, max_e, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank,
                        phase, norm_w_attn, norm_w_idx, norm_eps, freqs, inv_fp8_scale, cmp_pool, idxk_pool, k_valid,
                        dbg_attn, dbg_idx, do_body=1, stream=None, *, cp=2, q_len=2, freq_rows=1 << 20, status=None):
    if not do_body:
        return
    p = _raw_params(b_count, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank, 4, cp, q_len)
    p.phase, p.max_entries = int(phase), max_e
    p.norm_w_attn, p.norm_w_idx, p.freqs = _addr(norm_w_attn), _addr(norm_w_idx), _addr(freqs)
    p.freq_rows = freqs.shape[0] if torch.is_tensor(freqs) else freq_rows
    p.norm_eps, p.inv_fp8_scale = float(norm_eps), float(inv_fp8_scale)
    p.attn_pool_dtype, p.attn_pool, p.idx_pool = N.DT_E4M3, _addr(cmp_pool), _addr(idxk_pool)
    p.idx_fmt, p.idx_page_tokens = N.FMT_MXFP4, 128
    p.k_valid, p.dbg_attn, p.dbg_idx, p.status = _addr(k_valid), _addr(dbg_attn), _addr(dbg_idx), _addr(status)
    N.call("mdc_compress_finalize_launch", p, stream)


def launch_c128_step(b_count, state, new_c128, ape128, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base,
                     ev_offsets, my_rank, stream=None, *, cp=2, q_len=2, ratio=128):
    p = _raw_params(b_count, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank, ratio, cp, q_len)
    p.state, p.new_attn, p.ape_attn = _addr(state), _addr(new_c128), _addr(ape128)
    p.ev_base_id = b_count   # the reference's online machine uses the event cells b_count + b (compress.py:639-640)
    N.call("mdc_compress_step_launch", p, stream)


def launch_c128_finalize(b_count, max_e, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank,
                         phase, norm_w, norm_eps, freqs, inv_fp8_scale, c128_pool, k_valid, dbg, stream=None, *,
                         cp=2, q_len=2, ratio=128, freq_rows=1 << 20, status=None):
    p = _raw_params(b_count, seq_len, pay_base, pay_offsets, mc_base, stats_off, ev_base, ev_offsets, my_rank, ratio, cp, q_len)
    p.phase, p.max_entries = int(phase), max_e
    p.norm_w_attn, p.freqs = _addr(norm_w), _addr(freqs)
    p.freq_rows = freqs.shape[0] if torch.is_tensor(freqs) else freq_rows
    p.norm_eps, p.inv_fp8_scale = float(norm_eps), float(inv_fp8_scale)
    p.attn_pool_dtype, p.attn_pool = N.DT_E4M3, _addr(c128_pool)
    p.k_valid, p.dbg_attn, p.status = _addr(k_valid), _addr(dbg), _addr(status)
    p.ev_base_id = b_count
    N.call("mdc_compress_finalize_launch", p, stream)


def launch_micro(*args, stream=None) -> None:
    """Staged Hadamard-128 + MXFP4 of n rows: x (n, 128) fp32 -> out (n, 68) uint8 (64 B codes + 4 B
    scales).  Called as launch_micro(x, out) with tensors, or with the reference's argument list
    launch_micro(n_count, x, out68, dbg, stream) (compress.py:892-902; dbg is not written)."""
    import ctypes as C

    if len(args) >= 3 and isinstance(args[0], int):
        n, x, out = args[0], args[1], args[2]
        stream = args[4] if len(args) > 4 else stream
    else:
        x, out = args[0], args[1]
        stream = args[2] if len(args) > 2 else stream
        assert x.is_cuda and x.is_contiguous() and x.shape[1] == HD_IDX and out.shape == (x.shape[0], 68)
        n = x.shape[0]
    fn = N.lib().mdc_hadamard_quant_launch
    N.check(fn(C.c_void_p(_addr(x)), C.c_void_p(_addr(out)), C.c_int32(n), C.c_void_p(N.stream_ptr(stream))),
            "mdc_hadamard_quant_launch")
