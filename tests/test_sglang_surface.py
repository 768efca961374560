"""The SGLang-facing surface on the CPU, against stand-in ``sglang`` modules (SGLang is not installable here).

* ``plugin.register()`` registers the backend name, its CLI choices, the three hooks and the Gemma-4 shim
  (reference behaviour: ``green_attention/plugin.py:117-137``; test pattern: ``test/unit/test_plugin.py:12-22``);
* ``backend.GreenAttentionBackend`` wraps ``flash_attn_with_kvcache`` and leaves decode queries uncast
  (``green_attention/backend.py:39-56``);
* the static half of the reference's contract test (``test/unit/test_contract.py:94-99``): every name a module
  imports from ``sglang`` is declared in that module's ``SGLANG_READS``. The other half (SGLang really provides
  those names) needs an installed SGLang and is not runnable here.
"""

import ast
import importlib
import os
import sys
import types
from pathlib import Path

import pytest
import torch

PACKAGE = Path(__file__).resolve().parent.parent / "greenattention_b200"


def _module(monkeypatch, name, **attrs):
    mod = types.ModuleType(name)
    for k, v in attrs.items():
        setattr(mod, k, v)
    monkeypatch.setitem(sys.modules, name, mod)
    parent, _, leaf = name.rpartition(".")
    if parent:
        if parent not in sys.modules:
            _module(monkeypatch, parent)
        setattr(sys.modules[parent], leaf, mod)
    return mod


class _Recorder:
    def __init__(self):
        self.choices, self.backends, self.hooks, self.resolution = [], {}, [], {}


@pytest.fixture
def sglang_stub(monkeypatch):
    rec = _Recorder()

    class HookType:
        AROUND = "around"

    class HookRegistry:
        @staticmethod
        def register(target, fn, kind):
            rec.hooks.append((target, fn, kind))

    def register_attention_backend(name):
        def deco(fn):
            rec.backends[name] = fn
            return fn
        return deco

    def register_resolution_hook(step):
        def deco(fn):
            rec.resolution[step] = fn
            return fn
        return deco

    def adder(kind):
        return lambda names: rec.choices.append((kind, names))

    _module(monkeypatch, "sglang.srt.plugins.hook_registry", HookRegistry=HookRegistry, HookType=HookType)
    _module(monkeypatch, "sglang.srt.layers.attention.attention_registry",
            register_attention_backend=register_attention_backend)
    _module(monkeypatch, "sglang.srt.arg_groups.choices",
            add_attention_backend_choices=adder("attention"),
            add_chunked_prefix_cache_attention_backend=adder("chunked"),
            add_deterministic_attention_backend_choices=adder("deterministic"),
            add_radix_supported_deterministic_attention_backend_choices=adder("radix"))
    _module(monkeypatch, "sglang.srt.arg_groups.resolution_hooks", register_resolution_hook=register_resolution_hook)
    spec = types.SimpleNamespace(speculative_algorithm=None, speculative_draft_attention_backend=None)
    _module(monkeypatch, "sglang.srt.runtime_context", get_spec=lambda: spec, attention_backends=lambda: ("green",))

    class FlashAttentionBackend:
        def __init__(self, model_runner, fa_impl_ver=3, **kw):
            self.fa_impl_ver = fa_impl_ver
            self._init_flash_attention_functions((10, 0))

        def _init_flash_attention_functions(self, device_capability):
            self.flash_attn_with_kvcache = lambda *a, **k: "stock"

        def prepare_paged_mha_query(self, q, q_rope, k_rope, layer, *, logical_batch_size, kv_head_num, is_prefill):
            return q.to(torch.float8_e4m3fn), q_rope, k_rope, "kd", "vd"

    _module(monkeypatch, "sglang.srt.layers.attention.flashattention_backend", FlashAttentionBackend=FlashAttentionBackend)
    monkeypatch.delitem(sys.modules, "greenattention_b200.backend", raising=False)
    yield rec
    sys.modules.pop("greenattention_b200.backend", None)


def test_register_installs_backend_choices_and_hooks(sglang_stub):
    from greenattention_b200 import gdn, gdn_recurrent, plugin

    plugin.register()
    assert {k for k, _ in sglang_stub.choices} == {"attention", "chunked", "deterministic", "radix"}
    assert all(names in (["green"], "green") for _, names in sglang_stub.choices)
    assert set(sglang_stub.backends) == {"green"}
    targets = {t: fn for t, fn, kind in sglang_stub.hooks if kind == "around"}
    assert targets[gdn.TARGET] is gdn.gdn_init_around
    assert targets[gdn_recurrent.REPLAY_TARGET] is gdn_recurrent._replayssm_around
    assert sglang_stub.resolution["handle_model_specific_adjustments"] is plugin._gemma4_accepts_green


def test_backend_wraps_kvcache_and_keeps_decode_query_uncast(sglang_stub, monkeypatch):
    from greenattention_b200 import dispatch

    prewarmed = []
    monkeypatch.setattr(dispatch, "prewarm", lambda backend: prewarmed.append(backend))
    backend_mod = importlib.import_module("greenattention_b200.backend")
    b = backend_mod.GreenAttentionBackend(types.SimpleNamespace())
    assert b.fa_impl_ver == 4 and prewarmed == [b]
    # a call that is not paged e4m3 attention passes through to the stock function
    assert b.flash_attn_with_kvcache(q=torch.zeros(2, 8, 128, dtype=torch.bfloat16), max_seqlen_q=300) == "stock"
    assert b.flash_attn_with_kvcache.__wrapped__ is not None
    q = torch.ones(3, 8, 128, dtype=torch.bfloat16)
    layer = types.SimpleNamespace(head_dim=128)
    kw = dict(logical_batch_size=3, kv_head_num=2, is_prefill=False)
    q2, q_rope, _, kd, vd = b.prepare_paged_mha_query(q, None, None, layer, **kw)
    assert q2 is q and q_rope is None and (kd, vd) == ("kd", "vd")  # bf16 query kept, descales from the stock logic
    # with a rope part the stock logic owns the call
    q3, *_ = b.prepare_paged_mha_query(q, q, None, layer, **kw)
    assert q3.dtype == torch.float8_e4m3fn
    # an op that is switched off hands the query to the stock cast
    monkeypatch.setattr(dispatch, "enabled", lambda op: False)
    q4, *_ = b.prepare_paged_mha_query(q, None, None, layer, **kw)
    assert q4.dtype == torch.float8_e4m3fn


def test_created_backend_comes_from_the_registered_factory(sglang_stub, monkeypatch):
    from greenattention_b200 import dispatch, plugin

    monkeypatch.setattr(dispatch, "prewarm", lambda backend: None)
    plugin.register()
    made = sglang_stub.backends["green"](types.SimpleNamespace(is_draft_worker=False))
    assert type(made).__name__ == "GreenAttentionBackend"


@pytest.mark.parametrize("arch, expect", [
    ("Gemma4ForConditionalGeneration", ("fa4", "triton")),
    ("Gemma4ForCausalLM", ("fa4", "triton")),
    ("Qwen3NextForCausalLM", ("green", "triton")),
])
def test_gemma4_shim_renames_green_only_for_gemma4_and_restores(sglang_stub, monkeypatch, arch, expect):
    from greenattention_b200 import plugin

    stock = lambda cfg: ("green", "triton")  # noqa: E731
    hook = _module(monkeypatch, "sglang.srt.arg_groups.model_hook", attention_backends_of=stock)
    cfg = types.SimpleNamespace(hf_config=types.SimpleNamespace(architectures=[arch]))
    _module(monkeypatch, "sglang.srt.arg_groups.model_override_base", model_config_of=lambda args: cfg)
    seen = []

    def previous(server_args):
        seen.append(hook.attention_backends_of(None))

    plugin._gemma4_accepts_green("args", previous)
    assert seen == [expect]
    assert hook.attention_backends_of is stock

    def failing(server_args):
        raise RuntimeError("boom")

    with pytest.raises(RuntimeError):
        plugin._gemma4_accepts_green("args", failing)
    assert hook.attention_backends_of is stock


def test_gdn_hook_wraps_dispatcher_kernels_only_on_green(sglang_stub, monkeypatch):
    from greenattention_b200 import gdn

    class Disp:
        pass

    def original(self, *a, **k):
        self.decode_kernel, self.verify_kernel = "tri-decode", "tri-verify"

    d = Disp()
    monkeypatch.setattr(gdn, "_green_on_sm100", lambda: False)
    gdn.gdn_init_around(original, d)
    assert d.decode_kernel == "tri-decode"
    monkeypatch.setattr(gdn, "_green_on_sm100", lambda: True)
    gdn.gdn_init_around(original, d)
    assert isinstance(d.decode_kernel, gdn.GreenGDNKernel) and d.verify_kernel.fallback == "tri-verify"


def test_standalone_switch_replaces_the_runtime_context_question(monkeypatch):
    from greenattention_b200 import gdn

    monkeypatch.setattr(torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(torch.cuda, "get_device_capability", lambda *a: (10, 0))
    gdn.set_standalone(True)
    try:
        assert gdn._green_on_sm100() is True  # no sglang import attempted
        monkeypatch.setattr(torch.cuda, "get_device_capability", lambda *a: (9, 0))
        assert gdn._green_on_sm100() is False
    finally:
        gdn.set_standalone(False)


# ------------------------------------------------------------------ static contract: declared == imported


def _declared(tree):
    for node in tree.body:
        if isinstance(node, ast.Assign) and any(isinstance(t, ast.Name) and t.id == "SGLANG_READS" for t in node.targets):
            return ast.literal_eval(node.value)
    return {}


def _sglang_imports(tree):
    names = set()
    for node in ast.walk(tree):
        if isinstance(node, ast.ImportFrom) and (node.module or "").startswith("sglang."):
            names.update(a.asname or a.name for a in node.names)
        elif isinstance(node, ast.Import):
            for a in node.names:
                if a.name.startswith("sglang."):
                    names.add(a.name.rsplit(".", 1)[-1])
    return names


READERS = sorted(p for p in PACKAGE.glob("*.py") if "sglang" in p.read_text())


@pytest.mark.parametrize("path", READERS, ids=lambda p: p.name)
def test_every_sglang_import_is_declared(path):
    tree = ast.parse(path.read_text())
    imports = _sglang_imports(tree)
    declared_map = _declared(tree)
    if not imports and not declared_map:
        pytest.skip("mentions sglang only in prose")
    declared = {n for names in declared_map.values() for n in names}
    # a whole-module import (`import sglang.srt.x.model_hook as model_hook`) is declared by its file key
    files = {os.path.splitext(os.path.basename(k))[0] for k in declared_map}
    undeclared = {n for n in imports if n not in declared and n not in files}
    assert not undeclared, f"{path.name}: declare {sorted(undeclared)} in SGLANG_READS"
    for key, names in declared_map.items():
        assert key.endswith(".py") and names and all(isinstance(n, str) for n in names), key


def test_hook_targets_name_what_sglang_reads_declares():
    """The dotted hook targets end in a symbol that the module's ``SGLANG_READS`` lists under the matching file."""
    from greenattention_b200 import gdn, gdn_recurrent

    for mod, target in ((gdn, gdn.TARGET), (gdn_recurrent, gdn_recurrent.REPLAY_TARGET)):
        parts = target.split(".")
        assert parts[0] == "sglang"
        declared = {n.split("(")[0] for names in mod.SGLANG_READS.values() for n in names}
        assert parts[-1] in declared or parts[-2] in declared, target
        files = [k for k in mod.SGLANG_READS if any(k.endswith("/".join(parts[1:i]) + ".py") for i in range(2, len(parts) + 1))]
        assert files, f"{target}: no SGLANG_READS file key matches the dotted path"


def test_pyproject_registers_the_plugin_entry_point():
    text = (PACKAGE.parent / "pyproject.toml").read_text()
    assert '[project.entry-points."sglang.srt.plugins"]' in text
    assert 'green_attention = "greenattention_b200.plugin:register"' in text
    from greenattention_b200 import plugin

    assert callable(plugin.register)
