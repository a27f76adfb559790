"""ctypes binding of libmdc.so (declared in include/mdc.h).

The CUDA library is the product: importing a launcher from here fails loudly
when libmdc.so is missing; there is no Python or CPU fallback for any kernel.
"""

from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MDC_LIB_PATH") or os.path.join(_PKG, "libmdc.so")

ABI_VERSION = 3
FMT_MXFP4, FMT_NVFP4 = 0, 1
Q_FP4, Q_BF16 = 0, 1
DT_F32, DT_BF16, DT_E4M3 = 0, 1, 2

p_void, i32, i64, f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float


class MdcError(RuntimeError):
    pass


class LogitsParams(C.Structure):
    _fields_ = [
        ("kv_pages", p_void), ("num_pages", i32), ("page_tokens", i32), ("fmt", i32), ("q_fmt", i32),
        ("q", p_void), ("q_sf", p_void), ("weights", p_void), ("block_table", p_void), ("max_pages", i32),
        ("seq_lens", p_void), ("logits", p_void), ("logits_stride", i64),
        ("cand_v", p_void), ("cand_i", p_void), ("cand_c", p_void), ("top_k", i32),
        ("B", i32), ("q_len", i32), ("heads", i32), ("blocks_per_chunk", i32), ("n_chunks", i32),
        ("window_exclude", i32), ("id_mul", i32), ("id_add", i32), ("status", p_void),
        ("row_v", p_void), ("row_i", p_void), ("row_c", p_void),
    ]


class MergeTopkParams(C.Structure):
    _fields_ = [
        ("cand_v", p_void), ("cand_i", p_void), ("cand_c", p_void), ("out_v", p_void), ("out_i", p_void),
        ("out_c", p_void), ("dbg", p_void),
        ("B", i32), ("q_len", i32), ("L", i32), ("maxK", i32), ("top_k", i32),
    ]


class LseMergeParams(C.Structure):
    _fields_ = [
        ("acc_o", p_void), ("acc_lse", p_void), ("o", p_void), ("lse", p_void),
        ("rows", i32), ("H", i32), ("D", i32), ("n_slices", i32), ("n_slices_max", i32),
        ("acc_dtype", i32), ("out_dtype", i32),
    ]


class SparseMlaParams(C.Structure):
    _fields_ = [
        ("q", p_void), ("kv_win", p_void), ("kv_cmp", p_void), ("pt_win", p_void), ("pt_cmp", p_void),
        ("k_valid", p_void), ("win_valid", p_void), ("attn_sink", p_void), ("o", p_void), ("lse", p_void),
        ("o_stride", i64), ("lse_stride", i64), ("ws_o", p_void), ("ws_lse", p_void),
        ("B", i32), ("q_len", i32), ("H", i32), ("d_qk", i32), ("d_v", i32),
        ("pages_win", i32), ("pages_cmp", i32), ("page_cmp", i32), ("pt_cols", i32),
        ("kv_dtype", i32), ("out_dtype", i32), ("n_splits", i32), ("fp8_p", i32),
        ("softmax_scale", f32), ("output_scale", f32), ("status", p_void),
    ]


class EventSetC(C.Structure):
    _fields_ = [("base", p_void), ("offsets", p_void), ("my_rank", i32), ("world", i32)]


class PeerBufferC(C.Structure):
    _fields_ = [("base", p_void), ("offsets", p_void), ("my_rank", i32), ("world", i32), ("mc_base", i64)]


class CompressParams(C.Structure):
    _fields_ = [
        ("B", i32), ("cp", i32), ("rank", i32), ("q_len", i32), ("ratio", i32), ("phase", i32),
        ("seq_len", p_void), ("ring_attn", p_void), ("ring_idx", p_void), ("new_attn", p_void), ("new_idx", p_void),
        ("ape_attn", p_void), ("ape_idx", p_void), ("state", p_void),
        ("arena", PeerBufferC), ("stats_off", i64), ("events", EventSetC), ("ev_base_id", i32), ("do_push", i32),
        ("wait_budget_ns", i64), ("norm_w_attn", p_void), ("norm_w_idx", p_void), ("freqs", p_void),
        ("freq_rows", i32), ("norm_eps", f32), ("inv_fp8_scale", f32), ("attn_pool_dtype", i32),
        ("attn_pool", p_void), ("idx_pool", p_void), ("idx_fmt", i32), ("idx_page_tokens", i32),
        ("max_entries", i32), ("ring_slots", i32), ("k_valid", p_void), ("dbg_attn", p_void), ("dbg_idx", p_void),
        ("status", p_void),
    ]


class LayerParams(C.Structure):
    _fields_ = [
        ("cp", i32), ("rank", i32), ("B", i32), ("top_k", i32), ("H", i32), ("n_chunks", i32),
        ("kv_seq_stride", i32), ("attn_splits", i32),
        ("logits", LogitsParams), ("mla", SparseMlaParams),
        ("cand_off", i64), ("inbox_off", i64), ("phase_bytes", i64), ("phases", i32),
        ("sel_v", p_void), ("sel_i", p_void), ("sel_c", p_void), ("out", p_void), ("out_lse", p_void),
        ("out_dtype", i32), ("l1_groups", i32), ("mid_v", p_void), ("mid_i", p_void), ("mid_c", p_void),
        ("cmp", CompressParams), ("q_stage", p_void), ("q_off", i64),
        ("kvw_k_idx", p_void), ("kvw_kv", p_void), ("kvw_glen", p_void), ("kvw_advance", i32),
        ("thr_hist", p_void), ("thr_done", p_void), ("kv_group", i32), ("cand_direct", i32), ("thr_exact", i32), ("thr_ev_base", i32), ("thr_off", i64), ("q_host_flag", p_void),
    ]


class MegaParams(C.Structure):
    _fields_ = [
        ("queue", p_void), ("row_words", i32), ("n_ctas", i32), ("scalars", p_void), ("arity", p_void),
        ("scopes", p_void), ("n_events", i32), ("events", EventSetC), ("arena", PeerBufferC),
        ("wait_budget_ns", i64), ("status", p_void), ("log", p_void), ("log_cap", i32),
        ("test_off", i64), ("test_slot_bytes", i32), ("layer", LayerParams),
        ("trace", p_void), ("trace_cap", i32), ("phase_ctl", p_void),
        ("dyn_task_off", p_void), ("dyn_n_tasks", i32), ("dyn_ctl", p_void),
    ]


class PingpongParams(C.Structure):
    _fields_ = [("events", EventSetC), ("role", i32), ("peer", i32), ("ev_ping", i32), ("ev_pong", i32), ("rounds", i32),
                ("base", C.c_uint64), ("wait_budget_ns", i64), ("out_ns", p_void), ("status", p_void)]


OP_NOP, OP_LOGITS, OP_MERGE_L1, OP_MERGE_L2, OP_ATTN, OP_LSE_MERGE, OP_MERGE_L1A = 0, 1, 2, 3, 4, 5, 6
OP_CMP_STEP, OP_CMP_FIN, OP_QPATH, OP_KVWRITE = 7, 8, 9, 10
OP_SLEEP, OP_LOG, OP_PUSH, OP_VERIFY = 16, 17, 18, 19
DEV_WAIT_TIMEOUT, DEV_COPY_TIMEOUT, DEV_BAD_INDEX, DEV_BAD_OP = 1, 2, 3, 4

_lib = None


def lib() -> C.CDLL:
    """The loaded library.  Raises MdcError when it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise MdcError(
                f"{LIB_PATH} is missing: build it with `python -m mega_dsa_cp_b200.build` "
                "(nvcc, sm_100a); this package has no fallback path")
        l = C.CDLL(LIB_PATH)
        l.mdc_abi_version.restype = C.c_int
        if l.mdc_abi_version() != ABI_VERSION:
            raise MdcError("libmdc.so ABI version mismatch; rebuild the library")
        l.mdc_status_string.restype = C.c_char_p
        l.mdc_status_string.argtypes = [C.c_int]
        l.mdc_last_cuda_error.restype = C.c_int
        for name in EXPORTS:
            if name != "mdc_status_string":
                getattr(l, name).restype = C.c_int
        _lib = l
    return _lib


# every symbol include/mdc.h declares (checked by the CPU test-suite)
EXPORTS = [
    "mdc_abi_version", "mdc_status_string", "mdc_last_cuda_error", "mdc_kernel_attrs",
    "mdc_logits_fp4_launch", "mdc_logits_fp4_smem_bytes", "mdc_merge_topk_launch",
    "mdc_lse_merge_launch", "mdc_sparse_mla_launch", "mdc_sparse_mla_smem_bytes",
    "mdc_sparse_mla_launch_static_ws",
    "mdc_megakernel_launch", "mdc_megakernel_check", "mdc_megakernel_smem_bytes", "mdc_megakernel_threads",
    "mdc_compress_step_launch", "mdc_compress_finalize_launch", "mdc_hadamard_quant_launch",
    "mdc_test_pingpong_launch",
]


def check(rc: int, what: str) -> None:
    if rc < 0:
        l = lib()
        msg = l.mdc_status_string(rc).decode()
        extra = f" (cudaError {l.mdc_last_cuda_error()})" if rc == -5 else ""
        raise MdcError(f"{what}: {msg}{extra}")


def ptr(t) -> int | None:
    """Device pointer of a torch tensor (None passes NULL)."""
    return None if t is None else t.data_ptr()


def stream_ptr(stream=None) -> int:
    """cudaStream_t of `stream` (a torch stream, a raw handle, or None = current)."""
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if hasattr(stream, "cuda_stream"):
        return stream.cuda_stream
    if hasattr(stream, "getPtr"):  # cuda.bindings.driver.CUstream
        return int(stream)
    return int(stream)


def call(name: str, params: C.Structure, stream=None) -> None:
    fn = getattr(lib(), name)
    check(fn(C.byref(params), C.c_void_p(stream_ptr(stream))), name)
