"""Front-end of the Gated-DeltaNet recurrent kernel (ops ``gdn_decode`` and ``gdn_verify``).

Call forms kept from the reference (``green_attention/gdn_recurrent.py:120-214``, ``docs/gdn-contract.md:46-67``):

* packed decode: ``mixed_qkv [B, 2*H*K + HV*V]`` bf16 (q, k, v concatenated), ``a, b [B, HV]`` bf16, ``A_log [HV]``
  fp32, ``dt_bias [HV]`` fp32/bf16, ``ssm_states [slots, HV, V, K]`` fp32/bf16 updated in place,
  ``cache_indices [B]`` int32/int64 (``< 0`` = PAD: zero output row, state untouched); returns the
  ``[1, B, HV, V]`` transposed view of a ``[B, 1, HV, V]`` allocation; ``beta`` is rounded to bf16;
* split decode: ``q, k [1, N, H, K]``, ``v [1, N, HV, V]``, ``query_start_loc [B + 1]`` int32 (PAD: computed from a
  zero state, not stored; a request whose length is not 1: zero output, state untouched); returns ``[1, N, HV, V]``.

Added for speculative decoding with in-place commit (``gdn_spec_decode`` / op ``gdn_verify``): ``T <= 8`` chained
draft tokens per request, outputs for every token, and the stored state replaced by the state after
``accept_lens[n]`` tokens (0 = untouched, bit for bit).

Geometry is read from the tensors (``K = V = 128``, any ``HV`` that is a multiple of ``H``) instead of the
reference's compile-time ``H, HV = 16, 48``.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from greenattention_b200 import _C, dispatch

K = V = 128
MAX_SPEC = 8
_ready: set = set()


def ensure_ready(device=None) -> None:
    if not torch.cuda.is_available():
        raise _C.GreenAttentionError("no CUDA device: the green kernels have no CPU path")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = torch.cuda.current_device() if dev.index is None else dev.index
    if idx not in _ready:
        _C.init(idx)
        _ready.add(idx)


def _prewarm(backend=None) -> None:
    ensure_ready()


def _on_green_sm100() -> bool:
    from greenattention_b200 import gdn

    return gdn._green_on_sm100()


def _launch(
    *, q, k, v, a, b, A_log, dt_bias, state, idx, accept, qsl, out, tokens, batch, h, hv,
    q_str, k_str, v_str, a_str, b_str, o_str, l2norm=True, round_beta=False, pad_reads_zero=False, scale=None,
):
    p = _C.GaGdnParams()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.q_stride_seq, p.q_stride_tok = q_str
    p.k_stride_seq, p.k_stride_tok = k_str
    p.v_stride_seq, p.v_stride_tok = v_str
    p.a, p.b = a.data_ptr(), b.data_ptr()
    p.a_stride_seq, p.a_stride_tok = a_str
    p.b_stride_seq, p.b_stride_tok = b_str
    p.A_log = A_log.data_ptr()
    p.dt_bias = dt_bias.data_ptr()
    p.dt_bias_is_bf16 = int(dt_bias.dtype == torch.bfloat16)
    p.state = state.data_ptr()
    p.state_is_bf16 = int(state.dtype == torch.bfloat16)
    p.state_stride_slot = state.stride(0)
    p.cache_indices = idx.data_ptr()
    p.cache_indices_is_i64 = int(idx.dtype == torch.int64)
    p.accept_lens = accept.data_ptr() if accept is not None else None
    p.query_start_loc = qsl.data_ptr() if qsl is not None else None
    p.out = out.data_ptr()
    p.out_is_f32 = int(out.dtype == torch.float32)
    p.o_stride_seq, p.o_stride_tok = o_str
    p.batch, p.tokens, p.h, p.hv, p.k_dim, p.v_dim = batch, tokens, h, hv, K, V
    p.l2norm_qk, p.round_beta_bf16, p.pad_reads_zero = int(l2norm), int(round_beta), int(pad_reads_zero)
    p.scale = float(K**-0.5 if scale is None else scale)
    _C.check(
        _C.lib().ga_gdn_recurrent(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream), "ga_gdn_recurrent"
    )
    return out


def _common_reasons(q, k, v, a, b, A_log, dt_bias, state, idx, hv) -> list:
    why = []
    if any(t.dtype is not torch.bfloat16 for t in (q, k, v)):
        why.append("q/k/v dtype")
    if a.dtype is not torch.bfloat16 or b.dtype is not torch.bfloat16:
        why.append("a/b dtype")
    if A_log.dtype is not torch.float32 or A_log.numel() != hv:
        why.append("A_log")
    if dt_bias.numel() != hv or dt_bias.dtype not in (torch.float32, torch.bfloat16):
        why.append("dt_bias")
    if idx.ndim != 1 or idx.dtype not in (torch.int32, torch.int64):
        why.append(f"cache_indices {idx.dtype} {tuple(idx.shape)}")
    if state.dtype not in (torch.float32, torch.bfloat16):
        why.append(f"state dtype {state.dtype}")
    if state.ndim != 4 or tuple(state.shape[1:]) != (hv, V, K):
        why.append(f"state shape {tuple(state.shape)}")
    elif state.stride(1) != V * K or state.stride(2) != K or state.stride(3) != 1 or state.stride(0) % 4:
        why.append("state strides")
    if a.stride(-1) != 1 or b.stride(-1) != 1:
        why.append("a/b last stride")
    return why


def _select_packed(kwargs):
    if not _on_green_sm100():
        return "not on the green backend of an sm_100 device"
    mq, a, b = kwargs.get("mixed_qkv"), kwargs.get("a"), kwargs.get("b")
    state, idx = kwargs.get("ssm_states"), kwargs.get("cache_indices")
    if not isinstance(mq, torch.Tensor) or not isinstance(state, torch.Tensor):
        return "missing tensor"
    for ring in ("replayssm_d", "replayssm_k", "replayssm_g", "replayssm_write_pos"):
        if kwargs.get(ring) is not None:
            return f"replayssm buffered decode ({ring}) unsupported"
    if state.ndim != 4:
        return f"state shape {tuple(state.shape)}"
    hv = state.shape[1]
    width = mq.shape[-1] - hv * V if mq.ndim == 2 else -1
    if mq.ndim != 2 or mq.stride(-1) != 1 or width <= 0 or width % (2 * K) or hv % (width // (2 * K)):
        return f"mixed_qkv {tuple(mq.shape)}"
    h = width // (2 * K)
    why = _common_reasons(mq, mq, mq, a, b, kwargs.get("A_log"), kwargs.get("dt_bias"), state, idx, hv)
    if kwargs.get("num_v_heads", hv) != hv or kwargs.get("head_v_dim", V) != V:
        why.append("num_v_heads/head_v_dim")
    if why:
        return "; ".join(why)
    scale = kwargs.get("scale")
    B = mq.shape[0]

    def run(mixed_qkv, a, b, A_log, dt_bias, ssm_states, cache_indices, **kw):
        out = mixed_qkv.new_empty(B, 1, hv, V)
        row = mixed_qkv.stride(0)
        _launch(
            q=mixed_qkv, k=mixed_qkv[:, h * K:], v=mixed_qkv[:, 2 * h * K:], a=a, b=b, A_log=A_log, dt_bias=dt_bias,
            state=ssm_states, idx=cache_indices, accept=None, qsl=None, out=out, tokens=1, batch=B, h=h, hv=hv,
            q_str=(row, 0), k_str=(row, 0), v_str=(row, 0), a_str=(a.stride(0), 0), b_str=(b.stride(0), 0),
            o_str=(out.stride(0), 0), round_beta=True, pad_reads_zero=False, scale=scale,
        )
        return out.transpose(0, 1)

    return run


def _select_split(kwargs):
    if not _on_green_sm100():
        return "not on the green backend of an sm_100 device"
    q, k, v = kwargs.get("q"), kwargs.get("k"), kwargs.get("v")
    a, b = kwargs.get("a"), kwargs.get("b")
    state, idx, cu = kwargs.get("ssm_states"), kwargs.get("cache_indices"), kwargs.get("query_start_loc")
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v, state, cu)):
        return "missing tensor"
    if state.ndim != 4 or q.ndim != 4 or v.ndim != 4:
        return "q/v/state rank"
    hv, h = state.shape[1], q.shape[2]
    why = _common_reasons(q, k, v, a, b, kwargs.get("A_log"), kwargs.get("dt_bias"), state, idx, hv)
    if q.shape[0] != 1 or q.shape[1] != cu.numel() - 1 or q.shape[3] != K or hv % max(h, 1):
        why.append(f"q shape {tuple(q.shape)}")
    if k.shape != q.shape or v.shape[:2] != q.shape[:2] or tuple(v.shape[2:]) != (hv, V):
        why.append("k/v shape")
    for name, t, dim in (("q", q, K), ("k", k, K), ("v", v, V)):
        if t.stride(2) != dim or t.stride(3) != 1:
            why.append(f"{name} strides {t.stride()}")
    if cu.dtype is not torch.int32:
        why.append(f"query_start_loc dtype {cu.dtype}")
    if why:
        return "; ".join(why)
    scale = kwargs.get("scale")
    B = q.shape[1]

    def run(q, k, v, a, b, A_log, dt_bias, ssm_states, cache_indices, query_start_loc, **kw):
        out = q.new_empty(1, B, hv, V)
        _launch(
            q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=ssm_states, idx=cache_indices,
            accept=None, qsl=query_start_loc, out=out, tokens=1, batch=B, h=h, hv=hv,
            q_str=(q.stride(1), 0), k_str=(k.stride(1), 0), v_str=(v.stride(1), 0),
            a_str=(a.stride(0), 0), b_str=(b.stride(0), 0), o_str=(out.stride(1), 0),
            round_beta=False, pad_reads_zero=True, scale=scale,
        )
        return out

    return run


def _select_spec(kwargs):
    """Speculative step with accepted-prefix commit: q, k ``[B, T, H, K]``, v ``[B, T, HV, V]``, a, b ``[B, T, HV]``,
    ``accept_lens [B]`` int32 (optional), ``out`` optional (bf16 or fp32 ``[B, T, HV, V]``)."""
    if "accept_lens" not in kwargs and "ssm_states" not in kwargs:
        return "non-replayssm target_verify unsupported; speculative commit needs ssm_states/accept_lens"
    if not _on_green_sm100():
        return "not on the green backend of an sm_100 device"
    q, k, v, a, b = (kwargs.get(n) for n in ("q", "k", "v", "a", "b"))
    state, idx, acc = kwargs.get("ssm_states"), kwargs.get("cache_indices"), kwargs.get("accept_lens")
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v, a, b, state, idx)):
        return "missing tensor"
    if q.ndim != 4 or v.ndim != 4 or a.ndim != 3 or state.ndim != 4:
        return "q/v/a/state rank"
    B, T, h, _ = q.shape
    hv = state.shape[1]
    why = _common_reasons(q, k, v, a, b, kwargs.get("A_log"), kwargs.get("dt_bias"), state, idx, hv)
    if not 1 <= T <= MAX_SPEC:
        why.append(f"{T} draft tokens outside 1..{MAX_SPEC}")
    if q.shape[3] != K or k.shape != q.shape or tuple(v.shape) != (B, T, hv, V) or hv % max(h, 1):
        why.append("q/k/v shape")
    for name, t, dim in (("q", q, K), ("k", k, K), ("v", v, V)):
        if t.stride(2) != dim or t.stride(3) != 1:
            why.append(f"{name} strides {t.stride()}")
    if tuple(a.shape) != (B, T, hv) or tuple(b.shape) != (B, T, hv):
        why.append("a/b shape")
    if acc is not None and (acc.dtype is not torch.int32 or tuple(acc.shape) != (B,) or acc.stride(0) != 1):
        why.append("accept_lens must be int32 [B]")
    if idx.numel() != B:
        why.append("cache_indices batch")
    out = kwargs.get("out")
    if out is not None and (
        tuple(out.shape) != (B, T, hv, V) or out.dtype not in (torch.bfloat16, torch.float32)
        or out.stride(3) != 1 or out.stride(2) != V
    ):
        why.append("out layout")
    if why:
        return "; ".join(why)

    def run(q, k, v, a, b, A_log, dt_bias, ssm_states, cache_indices, accept_lens=None, scale=None, out=None,
            out_dtype=torch.bfloat16, use_qk_l2norm_in_kernel=True, **kw):
        if out is None:
            out = torch.empty((B, T, hv, V), dtype=out_dtype, device=q.device)
        return _launch(
            q=q, k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, state=ssm_states, idx=cache_indices,
            accept=accept_lens, qsl=None, out=out, tokens=T, batch=B, h=h, hv=hv,
            q_str=(q.stride(0), q.stride(1)), k_str=(k.stride(0), k.stride(1)), v_str=(v.stride(0), v.stride(1)),
            a_str=(a.stride(0), a.stride(1)), b_str=(b.stride(0), b.stride(1)),
            o_str=(out.stride(0), out.stride(1)), l2norm=use_qk_l2norm_in_kernel, scale=scale,
        )

    return run


def gdn_spec_decode(**kwargs) -> torch.Tensor:
    """Run the speculative GDN step (see ``_select_spec``); raises ``dispatch.Declined`` with the reason."""
    run = _select_spec(kwargs)
    if not callable(run):
        raise dispatch.Declined(f"gdn_spec_decode: {run}")
    return run(**kwargs)


dispatch.register("gdn_decode", _select_packed, _prewarm)
dispatch.register("gdn_decode", _select_split)
dispatch.register("gdn_verify", _select_spec)
