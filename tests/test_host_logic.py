"""Host-side logic on the CPU: op routing, decline rules, the split bound against the table taken from the
reference, plugin warnings, and that the C-ABI library loads and exports every declared symbol. Mirrors the
reference's CPU unit tests (``test/unit/test_dispatch.py``, ``test/unit/test_plugin.py``)."""

import importlib
import json
import logging
import os
import re
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLD = os.path.join(os.path.dirname(__file__), "golden", "host_tables.json")


@pytest.fixture
def dispatch(monkeypatch):
    def load(disable="", strict="1"):
        monkeypatch.setenv("GREEN_ATTN_DISABLE", disable)
        monkeypatch.setenv("GREEN_ATTN_STRICT", strict)
        import greenattention_b200.dispatch as module

        return importlib.reload(module)

    yield load
    monkeypatch.delenv("GREEN_ATTN_DISABLE", raising=False)
    monkeypatch.delenv("GREEN_ATTN_STRICT", raising=False)
    import greenattention_b200.dispatch as module

    importlib.reload(module)
    import greenattention_b200.attn_decode as ad
    import greenattention_b200.gdn_recurrent as gr

    importlib.reload(ad)
    importlib.reload(gr)


def _stock(**kwargs):
    return "stock"


def _call(wrapped, max_seqlen_q, dtype=torch.bfloat16):
    return wrapped(q=torch.zeros(2, 8, 128, dtype=dtype), max_seqlen_q=max_seqlen_q)


def test_ops_and_kvcache_op_match_reference_table(dispatch):
    d = dispatch()
    with open(GOLD) as f:
        table = json.load(f)
    assert list(d.OPS) == table["ops"] and d.MAX_VERIFY_Q == table["max_verify_q"]
    for arg, want in table["kvcache_op"]:
        assert d.kvcache_op(arg) == want, arg


def test_plan_splits_matches_reference_table():
    from greenattention_b200 import attn_decode

    with open(GOLD) as f:
        rows = json.load(f)["plan_splits"]
    for batch, ctx, sm, units, windowed, want in rows:
        assert attn_decode.plan_splits(batch, ctx, sm, units, windowed) == want


def test_decode_and_verify_route_by_query_length(dispatch):
    d = dispatch()
    d.register("decode", lambda kw: lambda **_: "decode")
    d.register("verify", lambda kw: lambda **_: "verify")
    wrapped = d.with_kvcache(_stock)
    assert _call(wrapped, 1) == "decode"
    assert _call(wrapped, 4) == "verify"
    # not a paged e4m3 call and not a decode/verify length: stays on the stock function
    assert _call(wrapped, d.MAX_VERIFY_Q + 1) == "stock"
    assert _call(wrapped, None) == "stock"


def test_long_paged_fp8_call_is_extend(dispatch):
    d = dispatch()
    d.register("extend", lambda kw: lambda **_: "extend")
    wrapped = d.with_kvcache(_stock)
    kc = torch.zeros(1, 16, 2, 128, dtype=torch.float8_e4m3fn)
    pt = torch.zeros(1, 1, dtype=torch.int32)
    for mq in (d.MAX_VERIFY_Q + 1, None):
        assert wrapped(q=torch.zeros(2, 8, 128), k_cache=kc, page_table=pt, max_seqlen_q=mq) == "extend"
    assert wrapped(q=torch.zeros(2, 8, 128), k_cache=kc.to(torch.bfloat16), page_table=pt, max_seqlen_q=40) == "stock"


def test_disable_env_forces_stock_per_op(dispatch):
    d = dispatch("decode")
    d.register("decode", lambda kw: lambda **_: "decode")
    d.register("verify", lambda kw: lambda **_: "verify")
    wrapped = d.with_kvcache(_stock)
    assert _call(wrapped, 1) == "stock"
    assert _call(wrapped, 4) == "verify"
    assert not d.enabled("decode") and d.enabled("verify")


def test_disable_env_rejects_unknown_op(dispatch):
    with pytest.raises(ValueError, match="unknown ops"):
        dispatch("decode,prefill")


def test_register_rejects_unknown_op(dispatch):
    with pytest.raises(ValueError, match="unknown op"):
        dispatch().register("prefill", lambda kw: "no")


def test_first_accepting_selector_wins(dispatch):
    d = dispatch()
    d.register("decode", lambda kw: "head_dim unsupported")
    d.register("decode", lambda kw: lambda **_: "second")
    assert _call(d.with_kvcache(_stock), 1) == "second"


def test_decline_logs_once_per_signature(dispatch, caplog):
    d = dispatch()
    d.register("decode", lambda kw: f"q.dtype={kw['q'].dtype}")
    wrapped = d.with_kvcache(_stock)
    with caplog.at_level(logging.INFO, logger=d.__name__):
        for _ in range(3):
            assert _call(wrapped, 1) == "stock"
        assert _call(wrapped, 1, torch.float16) == "stock"
    lines = [r.getMessage() for r in caplog.records if "fallback" in r.getMessage()]
    assert len(lines) == 2
    assert "q.dtype=torch.bfloat16" in lines[0] and "q.dtype=torch.float16" in lines[1]


def test_owned_call_that_is_declined_raises_in_strict_mode(dispatch):
    d = dispatch()
    d.register("decode", lambda kw: "declined for the test")
    wrapped = d.with_kvcache(_stock)
    kc = torch.zeros(1, 16, 2, 128, dtype=torch.float8_e4m3fn)
    pt = torch.zeros(1, 1, dtype=torch.int32)
    with pytest.raises(d.Declined, match="declined for the test"):
        wrapped(q=torch.zeros(2, 8, 128, dtype=torch.bfloat16), k_cache=kc, page_table=pt, max_seqlen_q=1)


def test_non_strict_mode_casts_bf16_query_for_the_stock_fp8_kernel(dispatch):
    d = dispatch(strict="0")
    d.register("decode", lambda kw: "declined")
    seen = {}
    wrapped = d.with_kvcache(lambda **kw: seen.setdefault("q", kw["q"]))
    kc = torch.zeros(1, 16, 2, 128, dtype=torch.float8_e4m3fn)
    pt = torch.zeros(1, 1, dtype=torch.int32)
    q = torch.full((2, 8, 128), 1.5, dtype=torch.bfloat16)
    wrapped(q=q, k_cache=kc, page_table=pt, max_seqlen_q=1)
    assert seen["q"].dtype == torch.float8_e4m3fn and seen["q"].float().eq(1.5).all()
    seen.clear()
    wrapped(q=q, k_cache=kc.to(torch.bfloat16), page_table=pt, max_seqlen_q=1)
    assert seen["q"] is q


def _cpu_case(**over):
    from greenattention_b200 import workloads as W

    kw = W.make_paged_case([300, 40], [4, 4], 16, q_heads=8, kv_heads=2, head_dim=128, seed=20)
    kw.update(over)
    return kw


@pytest.mark.parametrize(
    "mutate,needle",
    [
        (lambda kw: kw.update(softcap=30.0), "softcap"),
        (lambda kw: kw.update(window_size=(128, 5)), "window"),
        (lambda kw: kw.update(sinks=torch.zeros(8)), "sinks"),
        (lambda kw: kw.update(max_seqlen_q=17), "max_seqlen_q"),
        (lambda kw: kw.update(causal=False, max_seqlen_q=4), "non-causal"),
        (lambda kw: kw.update(k_cache=kw["k_cache"].float(), v_cache=kw["v_cache"].float()), "e4m3"),
        (lambda kw: kw.update(q=kw["q"][:, :3]), "q shape"),
        (lambda kw: kw.update(cu_seqlens_q=None), "paged"),
        (lambda kw: kw.update(k_cache=kw["k_cache"][:, :12], v_cache=kw["v_cache"][:, :12]), "power of two"),
        (lambda kw: kw.update(k_descale=torch.ones(3, 2)), "k_descale"),
        (lambda kw: kw.update(page_table=kw["page_table"].long()), "page_table"),
        (lambda kw: kw.update(out=torch.zeros(8, 8, 64, dtype=torch.bfloat16)), "out layout"),
    ],
)
def test_selector_declines_without_touching_a_gpu(mutate, needle):
    from greenattention_b200 import attn_decode

    kw = _cpu_case()
    mutate(kw)
    why = attn_decode.select(kw)
    assert isinstance(why, str) and needle in why, why


def test_valid_cpu_call_is_declined_only_for_not_being_prewarmed():
    from greenattention_b200 import attn_decode

    assert attn_decode.select(_cpu_case()) == "kernel not prewarmed for this device"
    assert attn_decode.select_extend(_cpu_case(max_seqlen_q=300)) == "kernel not prewarmed for this device"


@pytest.mark.parametrize("stray", ["cache_seqlens", "page_table", "cu_seqlens_q", "k_descale", "out"])
def test_tensor_on_another_device_than_q_is_declined(stray):
    """The C ABI takes raw addresses, so a length / index tensor left on the host while q is on a device must be
    declined by the selector, never launched. ``meta`` tensors stand in for the device here."""
    from greenattention_b200 import attn_decode
    from greenattention_b200 import workloads as W

    kw = W.make_paged_case([300, 40], [1, 1], 16, q_heads=8, kv_heads=2, head_dim=128, seed=21, descale="rand",
                           out_mode="given")
    moved = {k: (v.to("meta") if isinstance(v, torch.Tensor) and k != stray else v) for k, v in kw.items()}
    why = attn_decode.select(moved)
    assert isinstance(why, str) and why.startswith(f"{stray} is on cpu"), why


def test_gdn_selectors_decline_tensors_on_another_device(monkeypatch):
    from greenattention_b200 import gdn, gdn_recurrent
    from greenattention_b200 import workloads as W

    monkeypatch.setattr(gdn, "_green_on_sm100", lambda: True)
    c = W.make_gdn_case(2, 4, h=2, hv=4, seed=3)
    assert callable(gdn_recurrent._select_spec(c))
    moved = {k: (v.to("meta") if isinstance(v, torch.Tensor) and k != "cache_indices" else v) for k, v in c.items()}
    why = gdn_recurrent._select_spec(moved)
    assert isinstance(why, str) and "cache_indices is on cpu" in why, why
    rc = W.make_gdn_replay_case([4, 2], h=2, hv=4, ring_len=16)
    moved = {k: (v.to("meta") if isinstance(v, torch.Tensor) and k != "write_pos" else v) for k, v in rc.items()}
    why = gdn_recurrent._verify_supported(moved)
    assert isinstance(why, str) and "write_pos is on cpu" in why, why
    with pytest.raises(Exception, match="no CPU path|no CUDA"):
        gdn_recurrent._launch  # noqa: B018 - the launchers themselves refuse host tensors:
        gdn_recurrent._require_cuda(c["q"])


def test_no_cpu_path(monkeypatch):
    from greenattention_b200 import _C, attn_decode

    monkeypatch.setattr(torch.cuda, "is_available", lambda: False)
    with pytest.raises(_C.GreenAttentionError, match="no CPU path"):
        attn_decode.ensure_ready()


def test_library_loads_and_exports_every_declared_symbol():
    from greenattention_b200 import _C, build

    build.build()
    lib = _C.lib()
    with open(os.path.join(ROOT, "include", "green_attention.h")) as f:
        header = f.read()
    declared = set(re.findall(r"^\s*(?:int|size_t|const char\*)\s+(ga_\w+)\s*\(", header, flags=re.M))
    assert declared == set(_C.EXPORTS), declared ^ set(_C.EXPORTS)
    for name in declared:
        assert hasattr(lib, name), name
    assert lib.ga_abi_version() == _C.ABI_VERSION
    assert lib.ga_sm_count(0) == -1  # nothing initialised: no compute call is made here


def test_struct_layouts_match_the_header():
    """Field names and order of the ctypes mirrors follow the C structs."""
    from greenattention_b200 import _C

    with open(os.path.join(ROOT, "include", "green_attention.h")) as f:
        header = f.read()
    for cname, ctype in (("GaAttnParams", _C.GaAttnParams), ("GaMergeParams", _C.GaMergeParams),
                         ("GaGdnParams", _C.GaGdnParams), ("GaGdnVerifyParams", _C.GaGdnVerifyParams)):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cname, cname), header, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            parts = [x.strip() for x in decl.split(",")]
            names.append(re.split(r"[\s\*]+", parts[0])[-1])
            names.extend(x.lstrip("*").strip() for x in parts[1:])
        assert names == [n for n, _ in ctype._fields_], cname


@pytest.fixture
def create(monkeypatch):
    from greenattention_b200 import plugin

    backend = types.ModuleType("greenattention_b200.backend")
    backend.GreenAttentionBackend = lambda runner: "green"
    monkeypatch.setitem(sys.modules, "greenattention_b200.backend", backend)

    def run(algorithm, draft, is_draft=False):
        monkeypatch.setattr(plugin, "_spec_backends", lambda: (algorithm, draft))
        return plugin._create_green_backend(types.SimpleNamespace(is_draft_worker=is_draft))

    return run


@pytest.mark.parametrize(
    "algorithm, draft, warns",
    [
        (None, None, False),
        ("FROZEN_KV_MTP", None, False),
        ("FROZEN_KV_MTP", "green", False),
        ("FROZEN_KV_MTP", "triton", False),
        ("FROZEN_KV_MTP", "fa4", True),
        ("DFLASH", "fa4", False),
        ("DFLASH", None, False),
        ("DFLASH", "flashinfer", True),
        ("DFLASH", "green", True),
    ],
)
def test_target_warns_on_unexpected_draft_backend(create, caplog, algorithm, draft, warns):
    from greenattention_b200 import plugin

    with caplog.at_level(logging.WARNING, logger=plugin.__name__):
        assert create(algorithm, draft) == "green"
    assert any("draft runs on" in r.message for r in caplog.records) == warns


def test_gdn_wrapper_delegates_when_no_selector_accepts(monkeypatch):
    from greenattention_b200 import gdn

    monkeypatch.setattr(gdn, "_green_on_sm100", lambda: False)

    class Stock:
        uses_state_checkpoints = True
        supports_fused_chain_verify = False
        supports_strided_target_verify_qkv = True
        supports_track_state_snapshot = False
        supports_packed_decode = True

        def decode(self, q, k, v, a, b, **kw):
            return "stock-decode"

        def packed_decode(self, mixed_qkv, a, b, **kw):
            return "stock-packed"

        def target_verify(self, A_log, dt_bias, q, k, v, a, b, **kw):
            return "stock-verify"

        def extend(self, q, k, v, g, beta, **kw):
            return "stock-extend"

    w = gdn.GreenGDNKernel(Stock())
    assert w.uses_state_checkpoints and w.supports_packed_decode and not w.supports_fused_chain_verify
    t = torch.zeros(1)
    assert w.decode(t, t, t, t, t) == "stock-decode"
    assert w.packed_decode(t, t, t) == "stock-packed"
    assert w.target_verify(t, t, t, t, t, t, t) == "stock-verify"
    assert w.extend(t, t, t, t, t) == "stock-extend"
