"""Front-end of the FP8-KV paged attention kernels (ops ``decode``, ``verify`` and ``extend``).

Keeps the call contract of the reference module of the same name (``green_attention/attn_decode.py:152-400``):

* ``q [total_q, q_heads, head_dim]`` e4m3 or bf16 (a bf16 query is rounded to e4m3 in the kernel), last
  stride 1; K/V cache e4m3 ``[pages, page_size, kv_heads, head_dim]`` with a power-of-two page size, paged by an
  int32 ``page_table [batch, max_pages]``; int32 ``cache_seqlens [batch]`` and ``cu_seqlens_q [batch + 1]``;
* causal (bottom-right aligned) for more than one query token; optional left window ``window_size=(W, 0)``:
  the query at position ``p`` attends keys ``[p - W, p]``; no softcap / right window / sinks / rotary / KV append;
* ``k_descale`` / ``v_descale`` fp32 ``[batch | 1, kv_heads]`` with any strides;
* output bf16 ``[total_q, q_heads, head_dim]`` (``out=`` is written in place); with ``return_softmax_lse`` the
  call returns ``(out, lse)`` with ``lse`` fp32 ``[q_heads, total_q]`` in natural log.

``select`` / ``select_extend`` validate a call from shapes, dtypes and Python scalars only and return either a
launcher or a reason string. What differs from the reference is the kernel set behind them: instead of three
compile-time (head_dim, GQA) instances, the sm_100a kernels take head_dim 128 or 256 with any GQA whose
``GQA * max_seqlen_q`` fits 128 rows, and the window is a run-time argument. The split plan is made on the
device from the live ``cache_seqlens`` (the grid is one CTA per SM whatever the lengths), so ``plan_splits``
survives only as the host-side bound the reference exposes (``attn_decode.py:123-134``).
"""

from __future__ import annotations

import ctypes
import logging
import os
from typing import Callable, Optional, Union

import torch

from greenattention_b200 import _C, dispatch

TILE_N = 64                # KV tokens per pipeline stage of the kernels
SPLIT_TILE_TOKENS = 256    # plan_splits: at most one split per 256 tokens of context
WINDOW_SPLIT_MAX_FILL = 0.4
HEAD_DIMS = (128, 256, 512)
WIDE_HEAD_DIM = 512        # four 128-byte slabs per head: decode only, at most WIDE_HEAD_ROWS rows per kv head
WIDE_HEAD_ROWS = 8
MAX_ROWS = 128             # GQA * query tokens per (request, kv head) a decode / verify launch can hold
MAX_Q = dispatch.MAX_VERIFY_Q
MAX_BATCH = int(os.environ.get("GREEN_ATTN_MAX_BATCH", "4096"))  # requests per call the workspace is sized for

_ALLOWED = frozenset(
    (
        "q", "k_cache", "v_cache", "page_table", "cache_seqlens", "cu_seqlens_q", "max_seqlen_q",
        "softmax_scale", "causal", "window_size", "softcap", "return_softmax_lse", "num_splits", "out",
        "scheduler_metadata", "k_descale", "v_descale", "max_seqlen_k", "cu_seqlens_k_new", "pack_gqa",
        "sm_margin", "rel_bias_prep_cache",
    )
)
FP8 = torch.float8_e4m3fn
logger = logging.getLogger(__name__)

STATUS_NAMES = {
    1: "a bounded wait for a full ring stage ran out", 2: "a bounded wait for a free ring stage ran out",
    3: "a page id was out of range", 4: "a bounded wait for tensor memory ran out",
    5: "a cache_seqlens entry exceeded page_table.shape[1] * page_size",
}


class _State:
    workspaces: dict = {}  # device index -> uint8 workspace tensor
    sm_count: dict = {}


_S = _State()


def _is_sm100(device: torch.device) -> bool:
    return torch.cuda.get_device_capability(device)[0] == 10


def ensure_ready(device: Union[torch.device, int, None] = None) -> None:
    """Load the library, run its per-device set-up and allocate the split workspace. Idempotent; must run
    before CUDA-graph capture (same rule as the reference's ``ensure_ready``, ``attn_decode.py:100-115``)."""
    if not torch.cuda.is_available():
        raise _C.GreenAttentionError("no CUDA device: the green kernels have no CPU path")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    if dev.index in _S.workspaces:
        return
    _C.init(dev.index)
    lib = _C.lib()
    nbytes = lib.ga_attn_workspace_bytes(dev.index, MAX_BATCH)
    _S.workspaces[dev.index] = torch.zeros(nbytes, dtype=torch.uint8, device=dev)
    _S.sm_count[dev.index] = lib.ga_sm_count(dev.index)


def workspace(device: torch.device) -> torch.Tensor:
    return _S.workspaces[device.index]


def workspace_status(device: torch.device, builtin: bool = False) -> int:
    """Status word the kernels leave behind (0 = fine; see ``STATUS_NAMES``). It is sticky: one read covers every
    call since the last ``clear_status``. ``builtin`` reads the word of the array ``decode_noalloc`` works on
    (that entry point clears it at the start of each call). Synchronises the current stream."""
    val = ctypes.c_int(0)
    with torch.cuda.device(device):
        _C.check(
            _C.lib().ga_attn_workspace_status(
                None if builtin else workspace(device).data_ptr(), torch.cuda.current_stream(device).cuda_stream,
                ctypes.byref(val)),
            "ga_attn_workspace_status",
        )
    return val.value


def clear_status(device: torch.device) -> None:
    with torch.cuda.device(device):
        _C.check(
            _C.lib().ga_attn_workspace_clear_status(
                workspace(device).data_ptr(), torch.cuda.current_stream(device).cuda_stream),
            "ga_attn_workspace_clear_status",
        )


def check_status(device: Union[torch.device, None] = None, reset: bool = True) -> int:
    """Read the status word, log a non-zero value as an error and (by default) clear it. The launch path never
    synchronises, so a serving loop calls this at points where a sync is cheap: ``dispatch.prewarm`` does, and a
    scheduler may between batches. Returns the value read."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index not in _S.workspaces:
        return 0
    val = workspace_status(dev)
    if val != 0:
        logger.error("green_attention: kernel status %d on %s: %s; outputs of calls since the last check are "
                     "not trustworthy", val, dev, STATUS_NAMES.get(val, "unknown"))
        if reset:
            clear_status(dev)
    return val


def fp8_tensor_peak_tflops(device: Union[torch.device, None] = None) -> float:
    """Dense FP8 tensor-core peak of the device (TFLOP/s), measured with a tcgen05 issue loop."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    ensure_ready(dev)
    val = ctypes.c_float(0.0)
    _C.check(
        _C.lib().ga_fp8_tensor_peak(workspace(dev).data_ptr(), torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(val)),
        "ga_fp8_tensor_peak",
    )
    return float(val.value)


def _prewarm(backend) -> None:
    ensure_ready()
    check_status()


def plan_splits(batch: int, max_ctx: int, sm_count: int = 148, units: int = 8, windowed: bool = False) -> int:
    """Host-side upper bound on KV splits per (request, kv head): ``clamp(ceil(2*SMs / (batch*units)), 1,
    ceil(ctx / 256))``, and 1 for a windowed call once ``batch*units`` exceeds 0.4 of the SMs. The kernels do
    not consume it (they balance tiles across SMs on the device); it is kept for callers that size buffers."""
    work = batch * units
    if windowed and work > WINDOW_SPLIT_MAX_FILL * sm_count:
        return 1
    by_occupancy = (2 * sm_count + work - 1) // work
    by_context = max((max_ctx + SPLIT_TILE_TOKENS - 1) // SPLIT_TILE_TOKENS, 1)
    return max(1, min(by_occupancy, by_context))


# ------------------------------------------------------------------ validation


def _descale_reason(t, batch: int, kvh: int, name: str) -> Optional[str]:
    if t is None:
        return None
    if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != kvh or t.shape[0] not in (batch, 1):
        return f"{name} must be fp32 [batch|1, {kvh}]"
    return None


def _window_left(kw: dict) -> Union[int, str]:
    """Left window from FA's ``window_size=(left, right)``; right must be -1 or 0 (0 only with causal)."""
    ws = kw.get("window_size", (-1, -1))
    if ws is None:
        return -1
    if len(ws) != 2:
        return "window"
    left = -1 if ws[0] is None else int(ws[0])
    right = -1 if ws[1] is None else int(ws[1])
    if right not in (-1, 0):
        return f"window right {right} must be -1 or 0"
    if right == 0 and not kw.get("causal", False):
        return "window right 0 without causal"
    return left


def _shape_reason(kw: dict) -> Optional[str]:
    for name, val in kw.items():
        if val is not None and name not in _ALLOWED:
            return f"unsupported arg {name}"
    need = ("q", "k_cache", "v_cache", "page_table", "cache_seqlens", "cu_seqlens_q")
    if any(kw.get(n) is None for n in need):
        return "not a paged varlen call"
    if not isinstance(kw["cache_seqlens"], torch.Tensor):
        return "cache_seqlens must be a tensor"
    q, kc = kw["q"], kw["k_cache"]
    if q.dim() != 3 or q.stride(2) != 1 or kc.dim() != 4:
        return "q shape/stride"
    return None


def _paged_reason(kw: dict) -> Optional[str]:
    q, kc, vc = kw["q"], kw["k_cache"], kw["v_cache"]
    pt, cs, cu = kw["page_table"], kw["cache_seqlens"], kw["cu_seqlens_q"]
    hd, kvh = q.shape[2], kc.shape[2]
    # The C ABI takes raw addresses: a tensor on the host or on another GPU would be an illegal address in the
    # kernel, so every tensor argument must live where q lives.
    for name in ("k_cache", "v_cache", "page_table", "cache_seqlens", "cu_seqlens_q", "k_descale", "v_descale", "out"):
        t = kw.get(name)
        if isinstance(t, torch.Tensor) and t.device != q.device:
            return f"{name} is on {t.device}, q on {q.device}"
    if q.dtype not in (FP8, torch.bfloat16):
        return f"q dtype {q.dtype}"
    if kc.dtype != FP8 or vc.dtype != FP8:
        return "kv dtype is not e4m3"
    for t in (kc, vc):
        if t.dim() != 4 or t.shape[3] != hd or t.stride(3) != 1:
            return "kv layout"
        if any(s % 16 for s in t.stride()[:3]) or t.data_ptr() % 16:
            return "kv strides not 16-byte aligned"
    if tuple(kc.shape[:3]) != tuple(vc.shape[:3]):
        return "k/v page geometry differ"
    page = kc.shape[1]
    if page & (page - 1):
        return "page_size not a power of two"
    if pt.dtype != torch.int32 or pt.dim() != 2 or cs.dtype != torch.int32 or cs.dim() != 1 or cs.stride(0) != 1:
        return "page_table/cache_seqlens dtype/layout"
    if cu.dtype != torch.int32 or cu.dim() != 1 or cu.stride(0) != 1:
        return "cu_seqlens_q dtype/layout"
    batch = cs.shape[0]
    if batch == 0 or pt.shape[0] != batch or cu.shape[0] != batch + 1:
        return "batch mismatch"
    if batch > MAX_BATCH:
        return f"batch {batch} exceeds the workspace capacity {MAX_BATCH} (GREEN_ATTN_MAX_BATCH)"
    why = _descale_reason(kw.get("k_descale"), batch, kvh, "k_descale") or _descale_reason(
        kw.get("v_descale"), batch, kvh, "v_descale"
    )
    if why:
        return why
    vec = 4  # elements per vector access of q / out rows
    if q.stride(0) % vec or q.stride(1) % vec or q.data_ptr() % (8 if q.dtype == torch.bfloat16 else 4):
        return "q alignment"
    out = kw.get("out")
    if out is not None:
        if out.dtype != torch.bfloat16 or tuple(out.shape) != tuple(q.shape) or out.stride(2) != 1:
            return "out layout"
        if out.stride(0) % vec or out.stride(1) % vec or out.data_ptr() % 8:
            return "out alignment"
    if not q.is_cuda or q.device.index not in _S.workspaces:
        return "kernel not prewarmed for this device"
    return None


def _common_reason(kw: dict, op: str) -> Union[str, tuple]:
    why = _shape_reason(kw)
    if why:
        return why
    q, kc = kw["q"], kw["k_cache"]
    hd, qh, kvh = q.shape[2], q.shape[1], kc.shape[2]
    if hd not in HEAD_DIMS or not kvh or qh % kvh:
        return f"q shape: no {op} kernel for (head_dim={hd}, q_heads={qh}, kv_heads={kvh})"
    if qh // kvh > MAX_ROWS:
        return f"q shape: GQA {qh // kvh} exceeds {MAX_ROWS} rows"
    mq = kw.get("max_seqlen_q")
    if not isinstance(mq, int) or isinstance(mq, bool) or mq < 1:
        return f"max_seqlen_q {mq} is not a positive int"
    if mq > 1 and not kw.get("causal", False):
        return f"non-causal {op}"
    if kw.get("softcap", 0.0):
        return "softcap"
    wl = _window_left(kw)
    if isinstance(wl, str):
        return wl
    return (hd, qh, kvh, mq, wl)


def select(kw: dict) -> Union[Callable, str]:
    """Decode / verify: at most ``MAX_ROWS // GQA`` (and ``MAX_VERIFY_Q``) query tokens per request."""
    head = _common_reason(kw, "decode")
    if isinstance(head, str):
        return head
    hd, qh, kvh, mq, wl = head
    limit = min(MAX_Q, MAX_ROWS // (qh // kvh))
    if mq > limit:
        return f"max_seqlen_q {mq} outside 1..{limit}"
    if hd == WIDE_HEAD_DIM and mq * (qh // kvh) > WIDE_HEAD_ROWS:
        # the reference's (512, 8) instance takes up to 8 query tokens (attn_decode.py:58-62); here only the
        # decode step of that shape is built
        return f"q shape: head_dim {hd} is built for at most {WIDE_HEAD_ROWS} rows per kv head ({mq} x GQA {qh // kvh})"
    why = _paged_reason(kw)
    if why:
        return why
    return lambda **call_kw: _run("decode", window_left=wl, **call_kw)


def select_extend(kw: dict) -> Union[Callable, str]:
    """Prefill / extend over the FP8 cache: any query length, causal, optional left window."""
    head = _common_reason(kw, "extend")
    if isinstance(head, str):
        return head
    if head[0] == WIDE_HEAD_DIM:
        return f"q shape: no extend kernel for head_dim {head[0]}"
    wl = head[4]
    why = _paged_reason(kw)
    if why:
        return why
    return lambda **call_kw: _run("extend", window_left=wl, **call_kw)


# ------------------------------------------------------------------ launch


def _run(
    kind: str, *, q, k_cache, v_cache, page_table, cache_seqlens, cu_seqlens_q, max_seqlen_q, window_left=-1,
    softmax_scale=None, return_softmax_lse=False, out=None, k_descale=None, v_descale=None, _out_f32=False,
    _lse=None, **_,
):
    dev = q.device
    ws = _S.workspaces[dev.index]
    total_q, qh, hd = q.shape
    if out is None:
        out = torch.empty(q.shape, dtype=torch.float32 if _out_f32 else torch.bfloat16, device=dev)
    lse = _lse
    if lse is None and return_softmax_lse:
        lse = torch.empty((qh, total_q), dtype=torch.float32, device=dev)
    p = _C.GaAttnParams()
    p.q = q.data_ptr()
    p.q_is_bf16 = int(q.dtype == torch.bfloat16)
    p.q_stride_tok, p.q_stride_head = q.stride(0), q.stride(1)
    p.k_cache, p.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    p.k_stride_page, p.k_stride_tok, p.k_stride_head = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
    p.v_stride_page, p.v_stride_tok, p.v_stride_head = v_cache.stride(0), v_cache.stride(1), v_cache.stride(2)
    p.num_pages, p.page_size = k_cache.shape[0], k_cache.shape[1]
    p.q_heads, p.kv_heads, p.head_dim = qh, k_cache.shape[2], hd
    p.page_table = page_table.data_ptr()
    p.pt_stride_row, p.pt_stride_col = page_table.stride(0), page_table.stride(1)
    p.pt_cols = page_table.shape[1]
    p.cache_seqlens, p.cu_seqlens_q = cache_seqlens.data_ptr(), cu_seqlens_q.data_ptr()
    if k_descale is not None:
        p.k_descale = k_descale.data_ptr()
        p.kd_stride_b = k_descale.stride(0) if k_descale.shape[0] > 1 else 0
        p.kd_stride_h = k_descale.stride(1)
    if v_descale is not None:
        p.v_descale = v_descale.data_ptr()
        p.vd_stride_b = v_descale.stride(0) if v_descale.shape[0] > 1 else 0
        p.vd_stride_h = v_descale.stride(1)
    p.out = out.data_ptr()
    p.out_is_f32 = int(out.dtype == torch.float32)
    p.o_stride_tok, p.o_stride_head = out.stride(0), out.stride(1)
    p.lse = lse.data_ptr() if lse is not None else None
    p.total_q = total_q
    p.batch = cache_seqlens.shape[0]
    p.max_seqlen_q = int(max_seqlen_q)
    p.window_left = int(window_left)
    p.softmax_scale = float(hd**-0.5 if softmax_scale is None else softmax_scale)
    p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
    stream = torch.cuda.current_stream(dev).cuda_stream
    lib = _C.lib()
    fn = {"decode": lib.ga_attn_decode, "extend": lib.ga_attn_extend,
          "decode_noalloc": lib.ga_attn_decode_noalloc}[kind]
    with torch.cuda.device(dev):  # the library launches on the current device
        _C.check(fn(ctypes.byref(p), stream), f"ga_attn_{kind}")
    return (out, lse) if return_softmax_lse else out


def decode_noalloc(**kw):
    """Decode / verify through ``ga_attn_decode_noalloc``: the variant for hosts that cannot hand the library a
    workspace (no device allocator of their own, or allocation banned after start-up). Same arguments and
    result as the launcher ``select`` returns, within that entry point's limits (batch <= 1024, GQA * query
    tokens <= 16); larger calls raise. Calls on one device share a built-in scratch array and must not overlap."""
    fn = select(kw)
    if not callable(fn):
        raise dispatch.Declined(f"decode_noalloc: {fn}")
    if kw["q"].shape[2] == WIDE_HEAD_DIM:
        raise dispatch.Declined(f"decode_noalloc: the built-in scratch does not hold head_dim {WIDE_HEAD_DIM} partials")
    wl = _window_left(kw)
    return _run("decode_noalloc", window_left=wl, **{k: v for k, v in kw.items() if k != "window_size"})


def decode_partial(into: Optional[torch.Tensor] = None, **kw):
    """Decode over this device's shard of one request's KV range: returns ``(o fp32 [total_q, QH, HD]
    normalised, lse fp32 [QH, total_q])`` for ``merge_partials`` (the per-GPU step of a sequence whose KV
    range is split across GPUs). One query token per request and no window: the kernel places the causal
    diagonal and a window relative to the keys it is given, which is only right for a whole sequence.

    ``into``: a contiguous fp32 buffer of ``total_q * QH * (HD + 1)`` elements that receives O followed by the
    LSE (the packed form the exchange sends); the returned tensors are views of it, so nothing is copied
    between the kernel and the collective."""
    kw = {k: v for k, v in kw.items() if k != "out"}
    fn = select(kw)
    if not callable(fn):
        raise dispatch.Declined(f"decode_partial: {fn}")
    wl = _window_left(kw)
    if isinstance(wl, str) or wl >= 0:
        raise dispatch.Declined("decode_partial: a left window cannot be applied to a KV-range shard")
    q = kw["q"]
    if kw["max_seqlen_q"] != 1 or q.shape[0] != kw["cache_seqlens"].shape[0]:
        raise dispatch.Declined("decode_partial: one query token per request")
    out = lse = None
    if into is not None:
        tq, qh, hd = q.shape
        if (into.dtype != torch.float32 or into.dim() != 1 or into.numel() != tq * qh * (hd + 1)
                or not into.is_contiguous() or into.device != q.device or into.data_ptr() % 16):
            raise dispatch.Declined("decode_partial: `into` must be a 16-byte aligned fp32 buffer of total_q*QH*(HD+1) elements on q's device")
        out = into[: tq * qh * hd].view(tq, qh, hd)
        lse = into[tq * qh * hd:].view(qh, tq)
    kw = dict(kw, return_softmax_lse=True)
    return _run("decode", window_left=-1, _out_f32=True, out=out, _lse=lse, **kw)


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor, return_lse: bool = False):
    """LSE-weighted merge of ``o_parts [parts, rows, HD]`` fp32 / ``lse_parts [parts, rows]`` (natural log),
    all resident on this device, into bf16 ``[rows, HD]`` (math of ``kernel.cuh:665-749``). The tensors may be
    strided in their first dimension (views of one gathered buffer of packed partials are read where they are);
    the other dimensions must be dense."""
    parts, rows, hd = o_parts.shape
    if o_parts.stride(2) != 1 or o_parts.stride(1) != hd or o_parts.dtype != torch.float32:
        o_parts = o_parts.float().contiguous()
    if lse_parts.stride(1) != 1 or lse_parts.dtype != torch.float32:
        lse_parts = lse_parts.float().contiguous()
    if lse_parts.device != o_parts.device or not o_parts.is_cuda:
        raise dispatch.Declined("merge_partials: partials must be CUDA tensors on one device")
    out = torch.empty((rows, hd), dtype=torch.bfloat16, device=o_parts.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=o_parts.device) if return_lse else None
    m = _C.GaMergeParams()
    m.o_parts, m.lse_parts = o_parts.data_ptr(), lse_parts.data_ptr()
    m.o_part_stride = o_parts.stride(0) if parts > 1 else 0
    m.lse_part_stride = lse_parts.stride(0) if parts > 1 else 0
    m.parts, m.rows, m.head_dim = parts, rows, hd
    m.out = out.data_ptr()
    m.lse = lse.data_ptr() if lse is not None else None
    with torch.cuda.device(o_parts.device):
        _C.check(
            _C.lib().ga_attn_merge(ctypes.byref(m), torch.cuda.current_stream(o_parts.device).cuda_stream), "ga_attn_merge"
        )
    return (out, lse) if return_lse else out


dispatch.register("decode", select, prewarm=_prewarm)
dispatch.register("verify", select)
# A verify-sized call whose rows do not fit one decode launch still has the extend kernel.
dispatch.register("verify", select_extend)
dispatch.register("extend", select_extend)
