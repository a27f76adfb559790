"""KV compressor: host runners over mdc_compress_step_launch /
mdc_compress_finalize_launch (csrc/compress.cu).

Two pooling machines, both context-parallel (per-rank partial statistics ->
bulk push to the entry owner -> owner finalises):

* ratio 4: overlapping 8-slot window, attention (512) + indexer (128) streams;
  the owner writes an e4m3 (or bf16) attention entry and a Hadamard-rotated FP4
  indexer entry (with its block scale) into the fused index page.
* ratio 64 / 128: online per-channel softmax state [m | l | kv], attention
  stream only.

Covers launch_csa_step / launch_csa_finalize / launch_c128_step /
launch_c128_finalize / launch_micro of mega_dsa_cp/tiles/compress.py
(:253, :526, :643, :795, :892) of the reference, generalised from cp = 2,
q_len = 2 to any cp and q_len <= cp.
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
    p.norm_w_attn, p.norm_w_idx, p.freqs = N.ptr(norm_w_attn), N.ptr(norm_w_idx), N.ptr(freqs)
    p.freq_rows, p.norm_eps, p.inv_fp8_scale = freqs.shape[0], norm_eps, 1.0 / fp8_scale
    p.attn_pool_dtype = N.DT_E4M3 if st.attn_dtype == torch.float8_e4m3fn else N.DT_BF16
    p.attn_pool, p.idx_pool = N.ptr(st.attn_pool), N.ptr(st.idx_pool)
    p.idx_fmt = N.FMT_MXFP4 if st.idx_fmt == "mxfp4" else N.FMT_NVFP4
    p.idx_page_tokens, p.max_entries = st.idx_page_tokens, st.max_entries
    p.k_valid, p.dbg_attn, p.dbg_idx = N.ptr(st.k_valid), N.ptr(st.dbg_attn), N.ptr(st.dbg_idx)
    N.call("mdc_compress_finalize_launch", p, stream)


# names of the reference's launchers
launch_csa_step = launch_c128_step = launch_step
launch_csa_finalize = launch_c128_finalize = launch_finalize


def launch_micro(x: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    """x (n, 128) fp32 -> out (n, 68) uint8: staged Hadamard-128 + MXFP4 (64 B codes + 4 B scales)."""
    assert x.is_cuda and x.is_contiguous() and x.shape[1] == HD_IDX and out.shape == (x.shape[0], 68)
    fn = N.lib().mdc_hadamard_quant_launch
    import ctypes as C

    N.check(fn(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()), C.c_int32(x.shape[0]),
               C.c_void_p(N.stream_ptr(stream))), "mdc_hadamard_quant_launch")
