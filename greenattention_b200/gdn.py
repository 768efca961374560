"""GDN kernel wrapper installed into SGLang's ``GDNKernelDispatcher`` (reference: ``green_attention/gdn.py:57-110``).

An AROUND hook on ``GDNKernelDispatcher.__init__`` swaps the dispatcher's ``decode_kernel`` and
``verify_kernel`` for ``GreenGDNKernel`` objects. Each wraps the kernel SGLang picked: a call is served by a
green kernel when a selector accepts it and otherwise goes to the wrapped kernel with its capability flags
intact. ``extend`` always goes to the wrapped kernel. Only servers whose attention backend is ``green`` on an
sm_100 device are wrapped. SGLang is imported lazily so the module loads (and is tested) without it.
"""

from __future__ import annotations

import logging
import os

import torch

from greenattention_b200 import dispatch
from greenattention_b200 import gdn_recurrent  # noqa: F401  (registers the gdn selectors)

logger = logging.getLogger(__name__)

# Names this module expects SGLang to define (file under python/sglang/ -> symbols).
SGLANG_READS = {
    "srt/layers/attention/linear/kernels/kernel_backend.py": (
        "LinearAttnKernelBase", "uses_state_checkpoints", "supports_fused_chain_verify",
        "supports_strided_target_verify_qkv", "supports_track_state_snapshot", "decode", "extend", "target_verify",
    ),
    "srt/layers/attention/linear/gdn_backend.py": (
        "GDNKernelDispatcher", "__init__(decode_backend)", "decode_kernel", "verify_kernel", "packed_decode",
        "supports_packed_decode",
    ),
    "srt/runtime_context.py": ("attention_backends",),
}

TARGET = "sglang.srt.layers.attention.linear.gdn_backend.GDNKernelDispatcher.__init__"

_FLAGS = (
    "uses_state_checkpoints", "supports_fused_chain_verify", "supports_strided_target_verify_qkv",
    "supports_track_state_snapshot",
)


def _kernel_base():
    try:
        from sglang.srt.layers.attention.linear.kernels.kernel_backend import LinearAttnKernelBase

        return LinearAttnKernelBase
    except ImportError:
        return object


class GreenGDNKernel(_kernel_base()):
    def __init__(self, fallback):
        self.fallback = fallback
        for flag in _FLAGS:
            setattr(self, flag, getattr(fallback, flag, False))
        self.supports_packed_decode = getattr(fallback, "supports_packed_decode", False)

    def _green(self, op: str, call: dict):
        if not dispatch.enabled(op):
            return None
        return dispatch.select(op, call)

    def decode(self, q, k, v, a, b, **kwargs):
        call = dict(q=q, k=k, v=v, a=a, b=b, **kwargs)
        run = self._green("gdn_decode", call)
        return run(**call) if run is not None else self.fallback.decode(q, k, v, a, b, **kwargs)

    def packed_decode(self, mixed_qkv, a, b, **kwargs):
        call = dict(mixed_qkv=mixed_qkv, a=a, b=b, **kwargs)
        run = self._green("gdn_decode", call)
        return run(**call) if run is not None else self.fallback.packed_decode(mixed_qkv, a, b, **kwargs)

    def target_verify(self, A_log, dt_bias, q, k, v, a, b, **kwargs):
        call = dict(A_log=A_log, dt_bias=dt_bias, q=q, k=k, v=v, a=a, b=b, **kwargs)
        run = self._green("gdn_verify", call)
        if run is not None:
            return run(**call)
        return self.fallback.target_verify(A_log, dt_bias, q, k, v, a, b, **kwargs)

    def extend(self, q, k, v, g, beta, **kwargs):
        return self.fallback.extend(q, k, v, g, beta, **kwargs)


# Without an SGLang runtime context (a benchmark, a test, another host program calling the GDN front-end
# directly) nothing can say which attention backend the server runs; such callers declare themselves with
# ``set_standalone(True)`` or ``GREEN_ATTN_STANDALONE=1`` and only the device check remains.
_standalone = os.environ.get("GREEN_ATTN_STANDALONE", "0") == "1"


def set_standalone(on: bool = True) -> None:
    global _standalone
    _standalone = bool(on)


def _green_on_sm100() -> bool:
    if not torch.cuda.is_available() or torch.cuda.get_device_capability()[0] != 10:
        return False
    if _standalone:
        return True
    from sglang.srt.runtime_context import attention_backends

    return "green" in attention_backends()


def gdn_init_around(original, self, *args, **kwargs):
    original(self, *args, **kwargs)
    if not _green_on_sm100():
        return
    self.decode_kernel = GreenGDNKernel(self.decode_kernel)
    self.verify_kernel = GreenGDNKernel(self.verify_kernel)
    logger.info(
        "green_attention: GDN decode=%s verify=%s wrapped (green ops enabled: decode=%s verify=%s)",
        type(self.decode_kernel.fallback).__name__, type(self.verify_kernel.fallback).__name__,
        dispatch.enabled("gdn_decode"), dispatch.enabled("gdn_verify"),
    )
