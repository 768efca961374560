"""The ``green`` attention backend class (reference: ``green_attention/backend.py:39-56``): SGLang's
FlashAttention backend with its ``flash_attn_with_kvcache`` routed through ``dispatch`` so that paged e4m3
decode / verify / extend calls launch the B200 kernels. Decode keeps the query in bf16 (the kernel rounds it
to e4m3 itself). All kernels are loaded and their workspaces allocated in ``__init__``, before CUDA-graph
capture. Needs SGLang at import time, like the reference module.
"""

from __future__ import annotations

from sglang.srt.layers.attention.flashattention_backend import FlashAttentionBackend

from greenattention_b200 import attn_decode  # noqa: F401  (registers the decode/verify/extend kernels)
from greenattention_b200 import dispatch

SGLANG_READS = {
    "srt/layers/attention/flashattention_backend.py": (
        "FlashAttentionBackend", "__init__(fa_impl_ver)", "_init_flash_attention_functions",
        "flash_attn_with_kvcache", "prepare_paged_mha_query",
    ),
}


class GreenAttentionBackend(FlashAttentionBackend):
    def __init__(self, model_runner, **kwargs):
        super().__init__(model_runner, fa_impl_ver=4, **kwargs)
        dispatch.prewarm(self)

    def _init_flash_attention_functions(self, device_capability):
        super()._init_flash_attention_functions(device_capability)
        self.flash_attn_with_kvcache = dispatch.with_kvcache(self.flash_attn_with_kvcache)

    def prepare_paged_mha_query(self, q, q_rope, k_rope, layer, *, logical_batch_size, kv_head_num, is_prefill):
        kw = dict(logical_batch_size=logical_batch_size, kv_head_num=kv_head_num, is_prefill=is_prefill)
        if q_rope is not None or not dispatch.enabled("extend" if is_prefill else "decode"):
            return super().prepare_paged_mha_query(q, q_rope, k_rope, layer, **kw)
        # the stock logic on an empty slice yields the descales without casting q
        _, _, k_rope, k_descale, v_descale = super().prepare_paged_mha_query(q[:0], None, k_rope, layer, **kw)
        return q, None, k_rope, k_descale, v_descale
