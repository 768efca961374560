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

Replay-SSM verify (``gdn_replayssm_verify`` and the AROUND hook on SGLang's ``gdn_replayssm_spec_decode``): up to 4
chained tokens against a read-only checkpoint state plus the ring of deltas committed since, new deltas into the
ring, state untouched (``docs/gdn-contract.md:75-132`` of the reference).

Geometry is read from the tensors (``K = V = 128``, any ``HV`` that is a multiple of ``H``) instead of the
reference's compile-time ``H, HV = 16, 48``.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from greenattention_b200 import _C, dispatch

# Names this module expects SGLang to define (file under python/sglang/ -> symbols); the hook itself is
# registered by ``plugin.register``.
SGLANG_READS = {
    "srt/plugins/hook_registry.py": ("HookRegistry", "HookType", "AROUND"),
    "kernels/ops/attention/linear/gdn_replayssm_spec_decode.py": ("gdn_replayssm_spec_decode",),
}

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
    _require_cuda(q)
    bad_dev = _device_reason(q, dict(out=out, accept_lens=accept, query_start_loc=qsl))
    if bad_dev:
        raise dispatch.Declined(f"gdn: {bad_dev}")
    with torch.cuda.device(q.device):  # the library launches on the current device
        _C.check(
            _C.lib().ga_gdn_recurrent(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream), "ga_gdn_recurrent"
        )
    return out


def _device_reason(anchor: torch.Tensor, tensors: dict) -> Optional[str]:
    """The C ABI takes raw addresses and launches on ``anchor``'s device, so every tensor must live there (a
    length or index tensor left on the host would be an illegal address inside the kernel). Selectors look at
    placement only relative to ``anchor``; the launchers refuse host tensors outright (``_require_cuda``)."""
    for name, t in tensors.items():
        if isinstance(t, torch.Tensor) and t.device != anchor.device:
            return f"{name} is on {t.device}, expected {anchor.device}"
    return None


def _require_cuda(t: torch.Tensor) -> None:
    if not t.is_cuda:
        raise _C.GreenAttentionError(f"tensors are on {t.device}: the green kernels have no CPU path")


def _common_reasons(q, k, v, a, b, A_log, dt_bias, state, idx, hv) -> list:
    why = []
    bad_dev = _device_reason(q, dict(k=k, v=v, a=a, b=b, A_log=A_log, dt_bias=dt_bias, ssm_states=state, cache_indices=idx))
    if bad_dev:
        why.append(bad_dev)
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


# --------------------------------------------------------------------------- Replay-SSM verify

REPLAY_TARGET = (
    "sglang.kernels.ops.attention.linear.gdn_replayssm_spec_decode."
    "gdn_replayssm_spec_decode"
)
RING_LENS = (16, 32)
MAX_REPLAY_SPEC = 4


def _verify_supported(call) -> Optional[str]:
    """Why the Replay-SSM verify kernel cannot serve ``call`` (keyword arguments of
    ``gdn_replayssm_spec_decode``), or None. Same limits as the reference states for its own kernel
    (``green_attention/gdn_recurrent.py:269-352``, ``docs/gdn-contract.md:130-132``), with the head counts read
    from the tensors instead of fixed at 16 / 48."""
    if call.get("launch_mode") != "verify":
        return f"launch_mode {call.get('launch_mode')!r}"
    st = call.get("checkpoint_state")
    if not isinstance(st, torch.Tensor) or st.ndim != 4:
        return "no checkpoint_state [slots, HV, V, K]"
    if st.dtype not in (torch.float32, torch.bfloat16):
        return f"state dtype {st.dtype}"
    hv = st.shape[1]
    q, k, v = call.get("q"), call.get("k"), call.get("v")
    if not all(isinstance(t, torch.Tensor) for t in (q, k, v, call.get("a"), call.get("b"))):
        return "missing activation tensor"
    h = q.shape[1] if q.ndim == 3 else q.shape[-1] // K
    if tuple(st.shape[2:]) != (V, K) or st.stride(3) != 1 or st.stride(2) != K or st.stride(1) != V * K:
        return f"state layout {tuple(st.shape)} {st.stride()}"
    if h <= 0 or hv % h:
        return f"{hv} value heads over {h} key heads"
    L = int(call.get("max_cache_len") or 0)
    for name, shape, dt in (
        ("d_cache", (hv, L, V), torch.bfloat16), ("rawv_cache", (hv, L, V), torch.bfloat16),
        ("k_cache", (h, L, K), torch.bfloat16), ("rawk_cache", (h, L, K), torch.bfloat16),
        ("g_cache", (hv, L), torch.float32),
    ):
        t = call.get(name)
        if not isinstance(t, torch.Tensor):
            return f"missing {name}"
        if L not in RING_LENS:
            return f"max_cache_len {L} not in {RING_LENS}"
        if t.dtype is not dt:
            return f"{name} dtype {t.dtype}"
        if t.ndim != len(shape) + 1 or tuple(t.shape[1:]) != shape:
            return f"{name} shape {tuple(t.shape)}"
        if not t[0].is_contiguous() or t.stride(0) % 8:
            return f"{name} strides {t.stride()}"
    if call.get("beta_cache") is not None:
        return "beta_cache unsupported"
    if int(call.get("max_spec_len") or 0) > MAX_REPLAY_SPEC:
        return f"max_spec_len {call.get('max_spec_len')}"
    if call.get("use_qk_l2norm_in_kernel") is not True:
        return "use_qk_l2norm_in_kernel must be True"
    if call.get("null_block_id", -1) != -1:
        return f"null_block_id {call.get('null_block_id')}"
    why = []
    for name, t, n, dim in (("q", q, h, K), ("k", k, h, K), ("v", v, hv, V)):
        if t.dtype is not torch.bfloat16:
            why.append(f"{name} dtype {t.dtype}")
        if t.ndim == 3:  # [T, n, dim] with dense heads
            if tuple(t.shape[1:]) != (n, dim) or t.stride(2) != 1 or t.stride(1) != dim or t.stride(0) % 8:
                why.append(f"{name} layout {tuple(t.shape)} {t.stride()}")
        elif t.ndim == 2:  # flattened [T, n * dim]
            if t.shape[1] != n * dim or t.stride(1) != 1 or t.stride(0) % 8:
                why.append(f"{name} layout {tuple(t.shape)} {t.stride()}")
        else:
            why.append(f"{name} layout {tuple(t.shape)}")
    T = q.shape[0]
    for name in ("a", "b"):
        t = call[name]
        if t.dtype is not torch.bfloat16 or t.shape[0] != T or t.shape[-1] != hv or t.stride(-1) != 1:
            why.append(f"{name} {t.dtype} {tuple(t.shape)}")
    A_log, dt_bias = call.get("A_log"), call.get("dt_bias")
    if not isinstance(A_log, torch.Tensor) or A_log.dtype is not torch.float32 or A_log.numel() != hv:
        why.append("A_log must be fp32 [HV]")
    if not isinstance(dt_bias, torch.Tensor) or dt_bias.dtype not in (torch.float32, torch.bfloat16) or dt_bias.numel() != hv:
        why.append("dt_bias must be fp32/bf16 [HV]")
    if why:
        return "; ".join(why)
    ri, si, qsl = call.get("replay_indices"), call.get("ssm_state_indices"), call.get("query_start_loc")
    for name, t in (("ssm_state_indices", si), ("replay_indices", ri)):
        if not isinstance(t, torch.Tensor) or t.dtype not in (torch.int32, torch.int64) or not t.is_contiguous():
            return f"{name} must be a contiguous int32/int64 tensor"
    B = int(ri.numel())
    if si.numel() != B or not isinstance(qsl, torch.Tensor) or qsl.dtype is not torch.int32 or qsl.numel() != B + 1:
        return "ssm_state_indices / query_start_loc do not match replay_indices"
    for name, dt in (("write_pos", torch.int32), ("cache_base", torch.int32), ("is_flush", torch.int8)):
        t = call.get(name)
        if not isinstance(t, torch.Tensor) or t.dtype is not dt or not t.is_contiguous():
            return f"{name} must be a contiguous {dt} tensor"
    scale = call.get("scale")
    if scale is not None and abs(float(scale) - K**-0.5) > 1e-9:
        return f"scale {scale}"
    out = call.get("out")
    if not isinstance(out, torch.Tensor) or out.dtype is not torch.bfloat16 or out.shape[0] != T:
        return "out must be bf16 [T, HV, V]"
    bad_dev = _device_reason(q, {n: call.get(n) for n in (
        "k", "v", "a", "b", "A_log", "dt_bias", "checkpoint_state", "d_cache", "rawv_cache", "k_cache", "rawk_cache",
        "g_cache", "ssm_state_indices", "replay_indices", "query_start_loc", "write_pos", "cache_base", "is_flush", "out")})
    if bad_dev:
        return bad_dev
    if out.ndim == 3:
        if tuple(out.shape[1:]) != (hv, V) or out.stride(2) != 1 or out.stride(1) != V:
            return f"out layout {tuple(out.shape)} {out.stride()}"
    elif out.ndim != 2 or out.shape[1] != hv * V or out.stride(1) != 1:
        return f"out layout {tuple(out.shape)} {out.stride()}"
    return None


def _run_verify(call) -> torch.Tensor:
    """Launch the Replay-SSM verify kernel on a call that ``_verify_supported`` accepted."""
    _require_cuda(call["q"])
    ensure_ready(call["q"].device)
    q, st, out = call["q"], call["checkpoint_state"], call["out"]
    p = _C.GaGdnVerifyParams()
    p.q, p.k, p.v, p.a, p.b = (call[n].data_ptr() for n in ("q", "k", "v", "a", "b"))
    p.q_stride_tok, p.k_stride_tok, p.v_stride_tok = q.stride(0), call["k"].stride(0), call["v"].stride(0)
    p.a_stride_tok, p.b_stride_tok = call["a"].stride(0), call["b"].stride(0)
    p.A_log, p.dt_bias = call["A_log"].data_ptr(), call["dt_bias"].data_ptr()
    p.dt_bias_is_bf16 = int(call["dt_bias"].dtype is torch.bfloat16)
    p.checkpoint_state, p.state_is_bf16, p.state_stride_slot = st.data_ptr(), int(st.dtype is torch.bfloat16), st.stride(0)
    for field, name in (("d", "d_cache"), ("rawv", "rawv_cache"), ("k", "k_cache"), ("rawk", "rawk_cache"), ("g", "g_cache")):
        setattr(p, name, call[name].data_ptr())
        setattr(p, f"{field}_stride_slot", call[name].stride(0))
    si, ri = call["ssm_state_indices"], call["replay_indices"]
    p.ssm_state_indices, p.state_indices_is_i64 = si.data_ptr(), int(si.dtype is torch.int64)
    p.replay_indices, p.replay_indices_is_i64 = ri.data_ptr(), int(ri.dtype is torch.int64)
    p.query_start_loc = call["query_start_loc"].data_ptr()
    p.write_pos, p.cache_base, p.is_flush = (call[n].data_ptr() for n in ("write_pos", "cache_base", "is_flush"))
    p.out, p.o_stride_tok = out.data_ptr(), out.stride(0)
    p.batch = int(ri.numel())
    p.hv = st.shape[1]
    p.h = q.shape[1] if q.ndim == 3 else q.shape[-1] // K
    p.k_dim, p.v_dim, p.ring_len = K, V, int(call["max_cache_len"])
    p.scale = K**-0.5 if call.get("scale") is None else float(call["scale"])
    with torch.cuda.device(q.device):  # the library launches on the current device
        _C.check(_C.lib().ga_gdn_verify(ctypes.byref(p), torch.cuda.current_stream(q.device).cuda_stream), "ga_gdn_verify")
    return out


def gdn_replayssm_verify(**call) -> torch.Tensor:
    """The Replay-SSM verify step through the C ABI; raises ``dispatch.Declined`` with the reason when the call is
    outside what the kernel serves."""
    reason = _verify_supported(call)
    if reason is not None:
        raise dispatch.Declined(f"gdn_replayssm_verify: {reason}")
    return _run_verify(call)


def _replayssm_around(original, *args, **kwargs):
    """AROUND hook on SGLang's ``gdn_replayssm_spec_decode`` (``green_attention/gdn_recurrent.py:355-367``): serve the
    call when it is a production verify call, hand everything else to the stock function. No allocation and no
    host synchronisation, so it also runs while the target-verify CUDA graph is captured."""
    if kwargs and _on_green_sm100() and dispatch.enabled("gdn_verify"):
        reason = _verify_supported(kwargs)
        if reason is None:
            return _run_verify(kwargs)
        dispatch.log_fallback("gdn_verify", (reason,), kwargs)
    return original(*args, **kwargs)


dispatch.register("gdn_decode", _select_packed, _prewarm)
dispatch.register("gdn_decode", _select_split)
dispatch.register("gdn_verify", _select_spec)
