"""SGLang plugin entry point (reference: ``green_attention/plugin.py:46-137``): registers the ``green``
attention backend, its CLI choices and the GDN kernel hook. Launch with ``--attention-backend green``.

The draft backend that goes with a green target depends on the speculative algorithm
(``EXPECTED_DRAFT_BACKENDS``); a mismatch only logs a warning. Everything from SGLang is imported inside
the functions, so importing this module needs no SGLang.
"""

from __future__ import annotations

import logging

logger = logging.getLogger(__name__)

BACKEND = "green"

SGLANG_READS = {
    "srt/plugins/hook_registry.py": ("HookRegistry", "HookType", "register", "AROUND"),
    "srt/layers/attention/attention_registry.py": ("register_attention_backend",),
    "srt/arg_groups/choices.py": (
        "add_attention_backend_choices", "add_chunked_prefix_cache_attention_backend",
        "add_deterministic_attention_backend_choices", "add_radix_supported_deterministic_attention_backend_choices",
    ),
    "srt/runtime_context.py": ("get_spec",),
    "srt/model_executor/model_runner.py": ("is_draft_worker",),
    "srt/arg_groups/fields/spec.py": ("speculative_algorithm", "speculative_draft_attention_backend"),
    "srt/arg_groups/resolution_hooks.py": ("register_resolution_hook", '"handle_model_specific_adjustments"'),
    "srt/arg_groups/model_hook.py": (
        "handle_model_specific_adjustments", "attention_backends_of", '"Gemma4ForConditionalGeneration"',
    ),
    "srt/arg_groups/model_override_base.py": ("model_config_of",),
}

# speculative algorithm -> draft attention backends that fit a green target (None = flag unset, the draft
# runner inherits the target's backend). Algorithms not listed expect fa4.
EXPECTED_DRAFT_BACKENDS = {"FROZEN_KV_MTP": (None, BACKEND, "triton")}
DEFAULT_DRAFT_BACKENDS = ("fa4",)


def _spec_backends():
    """(speculative algorithm, --speculative-draft-attention-backend); (None, None) without speculation."""
    from sglang.srt.runtime_context import get_spec

    spec = get_spec()
    if spec.speculative_algorithm is None:
        return None, None
    return spec.speculative_algorithm, spec.speculative_draft_attention_backend


def _create_green_backend(runner):
    from greenattention_b200.backend import GreenAttentionBackend

    algorithm, draft = _spec_backends()
    fits = EXPECTED_DRAFT_BACKENDS.get(algorithm, DEFAULT_DRAFT_BACKENDS)
    if runner.is_draft_worker:
        logger.info("green_attention: serving the %s draft", algorithm)
    elif draft is not None and draft not in fits:
        names = " or ".join("unset" if b is None else repr(b) for b in fits)
        logger.warning(
            "green_attention: target backend is green but the %s draft runs on %r; expected %s", algorithm, draft, names
        )
    return GreenAttentionBackend(runner)


# SGLang's Gemma-4 argument check compares the attention backend against a fixed list of names and offers no
# extension point. ``green`` is the FA4 backend class with other kernels behind it, so for that one check, and
# only for these architectures, it answers to the name "fa4" (reference: ``green_attention/plugin.py:84-114``).
GEMMA4_ARCHS = frozenset((
    "Gemma4ForConditionalGeneration", "Gemma4ForCausalLM", "Gemma4UnifiedForConditionalGeneration",
))


def _gemma4_accepts_green(server_args, previous) -> None:
    """Resolution hook around ``handle_model_specific_adjustments``: while the stock step runs,
    ``model_hook.attention_backends_of`` reports ``green`` as ``fa4`` for Gemma-4 models; the function is put
    back whatever the step does."""
    import sglang.srt.arg_groups.model_hook as model_hook
    from sglang.srt.arg_groups.model_override_base import model_config_of

    stock = model_hook.attention_backends_of

    def renamed(cfg):
        names = stock(cfg)
        arch = model_config_of(server_args).hf_config.architectures[0]
        if arch not in GEMMA4_ARCHS:
            return names
        return tuple("fa4" if n == BACKEND else n for n in names)

    model_hook.attention_backends_of = renamed
    try:
        previous(server_args)
    finally:
        model_hook.attention_backends_of = stock


def register() -> None:
    """Called by SGLang's plugin loader in every process before a model is built."""
    from sglang.srt.arg_groups.choices import (
        add_attention_backend_choices,
        add_chunked_prefix_cache_attention_backend,
        add_deterministic_attention_backend_choices,
        add_radix_supported_deterministic_attention_backend_choices,
    )
    from sglang.srt.arg_groups.resolution_hooks import register_resolution_hook
    from sglang.srt.layers.attention.attention_registry import register_attention_backend
    from sglang.srt.plugins.hook_registry import HookRegistry, HookType

    from greenattention_b200 import gdn, gdn_recurrent

    add_attention_backend_choices([BACKEND])
    add_chunked_prefix_cache_attention_backend(BACKEND)
    add_deterministic_attention_backend_choices([BACKEND])
    add_radix_supported_deterministic_attention_backend_choices([BACKEND])
    register_attention_backend(BACKEND)(_create_green_backend)
    HookRegistry.register(gdn.TARGET, gdn.gdn_init_around, HookType.AROUND)
    HookRegistry.register(gdn_recurrent.REPLAY_TARGET, gdn_recurrent._replayssm_around, HookType.AROUND)
    register_resolution_hook("handle_model_specific_adjustments")(_gemma4_accepts_green)
