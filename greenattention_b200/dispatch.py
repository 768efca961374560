"""Op router of the ``green`` backend: which attention / GDN call runs on which B200 kernel.

Same surface as the reference router (``green_attention/dispatch.py:31-143``): the five ops, the selector
registry (``register`` / ``select`` / ``enabled`` / ``prewarm``), ``kvcache_op`` mapping ``max_seqlen_q`` to
an op, the once-per-signature decline log, the ``GREEN_ATTN_DISABLE`` switch, and ``with_kvcache`` wrapping
SGLang's ``flash_attn_with_kvcache``. A selector gets the call's keyword arguments and returns the callable
to launch or a string saying why it declines; it looks at shapes, dtypes and Python scalars only, so the
choice is the same at CUDA-graph capture and at replay.

Differences, all consequences of this being a single-target build with no alternative kernel path:

* ``extend`` covers every paged e4m3 call longer than ``MAX_VERIFY_Q`` query tokens (the reference only
  routed head_dim > 256 there because stock FA4 handled the rest on SM90).
* A paged e4m3 call that every selector declines is an error (``Declined``), not a silent hand-over, unless
  ``GREEN_ATTN_STRICT=0`` or the op is listed in ``GREEN_ATTN_DISABLE`` (the explicit A/B switch). Calls that
  are not paged e4m3 attention at all still go to the wrapped stock function untouched.
"""

from __future__ import annotations

import functools
import logging
import os
import threading
from collections import defaultdict
from typing import Any, Callable, Optional, Union

import torch

logger = logging.getLogger(__name__)

OPS = ("decode", "verify", "extend", "gdn_decode", "gdn_verify")
MAX_VERIFY_Q = 16

Selector = Callable[[dict], Union[Callable, str]]


class Declined(RuntimeError):
    """Every registered kernel declined a call this backend owns."""


def _parse_disabled(raw: str) -> frozenset:
    wanted = frozenset(part.strip() for part in raw.split(",") if part.strip())
    bad = sorted(wanted - frozenset(OPS))
    if bad:
        raise ValueError(f"GREEN_ATTN_DISABLE: unknown ops {bad}; valid: {OPS}")
    return wanted


DISABLED = _parse_disabled(os.environ.get("GREEN_ATTN_DISABLE", ""))
STRICT = os.environ.get("GREEN_ATTN_STRICT", "1") != "0"

_selectors: dict = defaultdict(list)
_prewarms: list = []
_seen: set = set()
_seen_lock = threading.Lock()


def register(op: str, selector: Selector, prewarm: Optional[Callable[[Any], None]] = None) -> None:
    """Add a kernel selector for ``op``; ``prewarm(backend)`` runs before CUDA-graph capture."""
    if op not in OPS:
        raise ValueError(f"unknown op {op!r}; valid: {OPS}")
    if selector not in _selectors[op]:
        _selectors[op].append(selector)
    if prewarm is not None and prewarm not in _prewarms:
        _prewarms.append(prewarm)


def prewarm(backend: Any) -> None:
    for fn in list(_prewarms):
        fn(backend)


def enabled(op: str) -> bool:
    return op not in DISABLED and len(_selectors[op]) > 0


def _describe(value: Any):
    if isinstance(value, torch.Tensor):
        return (str(value.dtype), tuple(value.shape[1:]))  # batch dimension left out
    if value is None or isinstance(value, (bool, int, float, str)):
        return value
    if isinstance(value, tuple) and all(isinstance(v, (int, float)) for v in value):
        return value
    return type(value).__name__


def _signature(kwargs: dict) -> tuple:
    return tuple((name, _describe(kwargs[name])) for name in sorted(kwargs))


def log_fallback(op: str, reasons: tuple, kwargs: dict) -> None:
    """One INFO line per distinct (op, reasons, argument signature)."""
    sig = _signature(kwargs)
    key = (op, tuple(reasons), sig)
    with _seen_lock:
        if key in _seen:
            return
        _seen.add(key)
    logger.info("green_attention: %s -> fallback (%s); signature=%s", op, "; ".join(reasons), sig)


def select(op: str, kwargs: dict) -> Optional[Callable]:
    """The kernel launcher for this call, or None when the op is off or every selector declined."""
    if op in DISABLED or not _selectors[op]:
        return None
    reasons = []
    for selector in _selectors[op]:
        verdict = selector(kwargs)
        if callable(verdict):
            return verdict
        reasons.append(str(verdict))
    log_fallback(op, tuple(reasons), kwargs)
    return None


def decline_reasons(op: str, kwargs: dict) -> tuple:
    return tuple(str(v) for v in (sel(kwargs) for sel in _selectors[op]) if not callable(v))


def kvcache_op(max_seqlen_q: Any) -> Optional[str]:
    """1 -> decode, 2..MAX_VERIFY_Q -> verify, anything else (symbolic lengths included) -> None."""
    if not isinstance(max_seqlen_q, int) or isinstance(max_seqlen_q, bool):
        return None
    if max_seqlen_q == 1:
        return "decode"
    if 2 <= max_seqlen_q <= MAX_VERIFY_Q:
        return "verify"
    return None


def owns(kwargs: dict) -> bool:
    """True for the calls this backend exists for: attention over a paged e4m3 KV cache."""
    kc = kwargs.get("k_cache")
    return (
        isinstance(kc, torch.Tensor)
        and kc.dtype == torch.float8_e4m3fn
        and kwargs.get("page_table") is not None
    )


def with_kvcache(fallback: Callable) -> Callable:
    """Wrap the stock ``flash_attn_with_kvcache``: paged e4m3 decode / verify / extend calls launch the
    B200 kernels; calls outside that scope reach ``fallback`` unchanged."""

    @functools.wraps(fallback)
    def flash_attn_with_kvcache(*args, **kwargs):
        mine = not args and owns(kwargs)
        op = kvcache_op(kwargs.get("max_seqlen_q"))
        if op is None and mine:
            op = "extend"
        if op is not None and args:
            log_fallback(op, ("positional arguments",), kwargs)
        elif op is not None:
            run = select(op, kwargs)
            if run is not None:
                return run(**kwargs)
            if mine and STRICT and op not in DISABLED and _selectors[op]:
                raise Declined(f"green_attention: {op} declined: " + "; ".join(decline_reasons(op, kwargs)))
        q, kc = kwargs.get("q"), kwargs.get("k_cache")
        if q is not None and kc is not None and kc.dtype == torch.float8_e4m3fn and q.dtype != kc.dtype:
            # the backend keeps decode queries in bf16 for the green kernels; the stock kernel wants the KV dtype
            kwargs["q"] = q.to(kc.dtype)
        return fallback(*args, **kwargs)

    return flash_attn_with_kvcache
