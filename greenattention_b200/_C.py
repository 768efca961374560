"""ctypes binding of ``libgreen_attention.so`` (the C ABI declared in ``include/green_attention.h``).

Takes the place of the reference's runtime build-and-load step (``green_attention/jit.py:139-183``): the
library is built ahead of time by ``greenattention_b200.build`` and loaded from the source tree. There is no
other implementation behind these calls: if the library is missing or a call fails, an exception is raised.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import POINTER, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_uint32, c_void_p

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libgreen_attention.so")
ABI_VERSION = 3

EXPORTS = (
    "ga_init", "ga_attn_workspace_bytes", "ga_attn_decode", "ga_attn_extend", "ga_attn_decode_noalloc", "ga_attn_merge",
    "ga_attn_exchange_merge",
    "ga_gdn_recurrent", "ga_gdn_verify", "ga_fp8_tensor_peak", "ga_last_launch_count", "ga_attn_workspace_status", "ga_attn_workspace_clear_status", "ga_last_error",
    "ga_abi_version", "ga_sm_count",
)


class GreenAttentionError(RuntimeError):
    """A call into the CUDA library failed, or the library is not built."""


class GaAttnParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("q_is_bf16", c_int32), ("q_stride_tok", c_int64), ("q_stride_head", c_int64),
        ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("k_stride_page", c_int64), ("k_stride_tok", c_int64), ("k_stride_head", c_int64),
        ("v_stride_page", c_int64), ("v_stride_tok", c_int64), ("v_stride_head", c_int64),
        ("num_pages", c_int32), ("page_size", c_int32),
        ("q_heads", c_int32), ("kv_heads", c_int32), ("head_dim", c_int32),
        ("page_table", c_void_p), ("pt_stride_row", c_int64), ("pt_stride_col", c_int64), ("pt_cols", c_int32),
        ("cache_seqlens", c_void_p), ("cu_seqlens_q", c_void_p),
        ("k_descale", c_void_p), ("kd_stride_b", c_int64), ("kd_stride_h", c_int64),
        ("v_descale", c_void_p), ("vd_stride_b", c_int64), ("vd_stride_h", c_int64),
        ("out", c_void_p), ("out_is_f32", c_int32), ("o_stride_tok", c_int64), ("o_stride_head", c_int64),
        ("lse", c_void_p), ("total_q", c_int64),
        ("batch", c_int32), ("max_seqlen_q", c_int32), ("window_left", c_int32), ("softmax_scale", c_float),
        ("workspace", c_void_p), ("workspace_bytes", c_size_t),
    ]


class GaMergeParams(ctypes.Structure):
    _fields_ = [
        ("o_parts", c_void_p), ("lse_parts", c_void_p), ("o_part_stride", c_int64), ("lse_part_stride", c_int64),
        ("parts", c_int32), ("rows", c_int32), ("head_dim", c_int32),
        ("out", c_void_p), ("lse", c_void_p),
    ]


class GaExchangeParams(ctypes.Structure):
    _fields_ = [
        ("mine", c_void_p), ("peer_bufs", c_void_p), ("peer_flags", c_void_p), ("epoch", c_void_p),
        ("rank", c_int32), ("world", c_int32), ("rows", c_int32), ("head_dim", c_int32),
        ("out", c_void_p), ("lse", c_void_p), ("status", c_void_p), ("wait_polls", c_uint32),
    ]


class GaGdnParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p),
        ("q_stride_seq", c_int64), ("q_stride_tok", c_int64), ("k_stride_seq", c_int64),
        ("k_stride_tok", c_int64), ("v_stride_seq", c_int64), ("v_stride_tok", c_int64),
        ("a", c_void_p), ("b", c_void_p),
        ("a_stride_seq", c_int64), ("a_stride_tok", c_int64), ("b_stride_seq", c_int64), ("b_stride_tok", c_int64),
        ("A_log", c_void_p), ("dt_bias", c_void_p), ("dt_bias_is_bf16", c_int32),
        ("state", c_void_p), ("state_is_bf16", c_int32), ("state_stride_slot", c_int64),
        ("cache_indices", c_void_p), ("cache_indices_is_i64", c_int32),
        ("accept_lens", c_void_p), ("query_start_loc", c_void_p),
        ("out", c_void_p), ("out_is_f32", c_int32), ("o_stride_seq", c_int64), ("o_stride_tok", c_int64),
        ("batch", c_int32), ("tokens", c_int32),
        ("h", c_int32), ("hv", c_int32), ("k_dim", c_int32), ("v_dim", c_int32),
        ("l2norm_qk", c_int32), ("round_beta_bf16", c_int32), ("pad_reads_zero", c_int32), ("scale", c_float),
    ]


class GaGdnVerifyParams(ctypes.Structure):
    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("a", c_void_p), ("b", c_void_p),
        ("q_stride_tok", c_int64), ("k_stride_tok", c_int64), ("v_stride_tok", c_int64),
        ("a_stride_tok", c_int64), ("b_stride_tok", c_int64),
        ("A_log", c_void_p), ("dt_bias", c_void_p), ("dt_bias_is_bf16", c_int32),
        ("checkpoint_state", c_void_p), ("state_is_bf16", c_int32), ("state_stride_slot", c_int64),
        ("d_cache", c_void_p), ("rawv_cache", c_void_p), ("k_cache", c_void_p), ("rawk_cache", c_void_p),
        ("g_cache", c_void_p),
        ("d_stride_slot", c_int64), ("rawv_stride_slot", c_int64), ("k_stride_slot", c_int64),
        ("rawk_stride_slot", c_int64), ("g_stride_slot", c_int64),
        ("ssm_state_indices", c_void_p), ("state_indices_is_i64", c_int32),
        ("replay_indices", c_void_p), ("replay_indices_is_i64", c_int32),
        ("query_start_loc", c_void_p), ("write_pos", c_void_p), ("cache_base", c_void_p), ("is_flush", c_void_p),
        ("out", c_void_p), ("o_stride_tok", c_int64),
        ("batch", c_int32), ("h", c_int32), ("hv", c_int32), ("k_dim", c_int32), ("v_dim", c_int32),
        ("ring_len", c_int32), ("scale", c_float),
    ]


_lock = threading.Lock()
_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library; raises ``GreenAttentionError`` when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise GreenAttentionError(
                f"{LIB_PATH} is missing: run `python -m greenattention_b200.build` (needs nvcc; no GPU required)"
            )
        handle = ctypes.CDLL(LIB_PATH)
        handle.ga_init.argtypes = [c_int]
        handle.ga_init.restype = c_int
        handle.ga_attn_workspace_bytes.argtypes = [c_int, c_int]
        handle.ga_attn_workspace_bytes.restype = c_size_t
        for name, ptype in (("ga_attn_decode", GaAttnParams), ("ga_attn_extend", GaAttnParams),
                            ("ga_attn_decode_noalloc", GaAttnParams),
                            ("ga_attn_merge", GaMergeParams), ("ga_attn_exchange_merge", GaExchangeParams),
                            ("ga_gdn_recurrent", GaGdnParams),
                            ("ga_gdn_verify", GaGdnVerifyParams)):
            fn = getattr(handle, name)
            fn.argtypes = [POINTER(ptype), c_void_p]
            fn.restype = c_int
        handle.ga_fp8_tensor_peak.argtypes = [c_void_p, c_void_p, POINTER(c_float)]
        handle.ga_fp8_tensor_peak.restype = c_int
        handle.ga_last_launch_count.argtypes = []
        handle.ga_last_launch_count.restype = c_int
        handle.ga_attn_workspace_status.argtypes = [c_void_p, c_void_p, POINTER(c_int)]
        handle.ga_attn_workspace_status.restype = c_int
        handle.ga_attn_workspace_clear_status.argtypes = [c_void_p, c_void_p]
        handle.ga_attn_workspace_clear_status.restype = c_int
        handle.ga_last_error.argtypes = []
        handle.ga_last_error.restype = c_char_p
        handle.ga_abi_version.argtypes = []
        handle.ga_abi_version.restype = c_int
        handle.ga_sm_count.argtypes = [c_int]
        handle.ga_sm_count.restype = c_int
        if handle.ga_abi_version() != ABI_VERSION:
            raise GreenAttentionError(
                f"{LIB_PATH} has ABI {handle.ga_abi_version()}, this package expects {ABI_VERSION}: rebuild it"
            )
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise GreenAttentionError(f"{what}: {lib().ga_last_error().decode(errors='replace')}")


def init(device_index: int) -> None:
    check(lib().ga_init(int(device_index)), f"ga_init({device_index})")
