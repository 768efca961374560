"""Gated-DeltaNet recurrent kernel on the GPU, through the plugin front-end and the C ABI, against the CPU
oracle and the golden fixtures. Cases follow the reference's GDN op tests
(``op_test/sm90/test_gdn_recurrent.py:52-125,233-258``): packed and split decode, fp32 and bf16 state, PAD rows,
strided gate inputs, determinism, CUDA-graph replay equal to eager bit for bit, back-to-back calls; plus the
accepted-prefix commit of the speculative form.

Tolerance (the stated parity bar): outputs and fp32 states within 1e-3 relative (outputs are compared in fp32
against the fp32 oracle, normalised by the largest reference magnitude; states by relative Frobenius norm
<= 1e-5 as the reference's tests do); accept-prefix / PAD bookkeeping bit-exact.
"""

import os

import numpy as np
import pytest
import torch

from greenattention_b200 import workloads as W
from tests.golden import cases

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(autouse=True)
def _force_gate(monkeypatch):
    import greenattention_b200.gdn as gdn_mod
    from greenattention_b200 import gdn_recurrent

    monkeypatch.setattr(gdn_mod, "_green_on_sm100", lambda: True)
    gdn_recurrent.ensure_ready()


def to_cuda(c):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}


def oracle_spec(c, accept="given", **opts):
    from oracle import gdn_oracle

    st = c["ssm_states"].clone()
    acc = c["accept_lens"] if accept == "given" else None
    out = gdn_oracle.recurrent_spec(c["q"], c["k"], c["v"], c["a"], c["b"], c["A_log"], c["dt_bias"], st,
                                    c["cache_indices"], acc, scale=c["scale"], **opts)
    return out, st


def run_spec(c, out_dtype=torch.float32):
    from greenattention_b200 import gdn_recurrent

    g = to_cuda(c)
    out = gdn_recurrent.gdn_spec_decode(
        q=g["q"], k=g["k"], v=g["v"], a=g["a"], b=g["b"], A_log=g["A_log"], dt_bias=g["dt_bias"],
        ssm_states=g["ssm_states"], cache_indices=g["cache_indices"], accept_lens=g["accept_lens"],
        scale=g["scale"], out_dtype=out_dtype,
    )
    torch.cuda.synchronize()
    return out.float().cpu(), g["ssm_states"].float().cpu(), g


def assert_close(out, ref, st, ref_st, out_rel=1e-3, st_rel=1e-5):
    oerr = (out - ref).abs().max().item() / max(ref.abs().max().item(), 1e-12)
    assert oerr <= out_rel, f"out rel err {oerr}"
    rel = ((st - ref_st).norm() / ref_st.norm()).item()
    assert rel <= st_rel, f"state rel err {rel}"


@pytest.mark.parametrize("name", sorted(cases.GDN_CASES))
def test_golden_fixture(name):
    c = cases.gdn_case(name)
    gold = np.load(os.path.join(GOLD, f"gdn_{name}.npz"))
    out, st, _ = run_spec(c)
    idx = c["cache_indices"].long()
    assert_close(out, torch.from_numpy(gold["out"]), st[idx], torch.from_numpy(gold["state"]))


@pytest.mark.parametrize("tokens", [1, 2, 3, 4, 5, 8])
@pytest.mark.parametrize("hv,h", [(32, 16), (48, 16), (8, 8)])
def test_spec_vs_oracle(tokens, hv, h):
    c = W.make_gdn_case(9, tokens, h=h, hv=hv, seed=tokens * 10 + hv, gate_params="rand", normalise_qk=False,
                        state_std=0.1, pad_rows=(2,))
    ref, ref_st = oracle_spec(c)
    before = c["ssm_states"].clone()
    out, st, _ = run_spec(c)
    assert_close(out, ref, st, ref_st)
    idx = c["cache_indices"].long()
    acc = c["accept_lens"].tolist()
    for n in range(9):  # bookkeeping is bit-exact: nothing accepted or PAD -> untouched slot
        if idx[n] >= 0 and acc[n] == 0:
            assert torch.equal(st[idx[n]], before[idx[n]])
    untouched = sorted(set(range(before.shape[0])) - {int(i) for i in idx if i >= 0})
    assert torch.equal(st[untouched], before[untouched])
    assert out[2].abs().max().item() == 0.0


def test_spec_bf16_output_and_config_shape():
    c = W.make_gdn_case(16, 4, h=16, hv=32, seed=77)
    ref, ref_st = oracle_spec(c)
    out, st, _ = run_spec(c, out_dtype=torch.bfloat16)
    assert (out - ref).abs().max().item() <= 2 ** -8 * ref.abs().max().item() + 1e-6
    assert ((st - ref_st).norm() / ref_st.norm()).item() <= 1e-5


@pytest.mark.parametrize("sd", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("B", [1, 8, 51])
def test_packed_decode(sd, B):
    from greenattention_b200 import gdn_recurrent
    from oracle import gdn_oracle

    H, HV, K, V = 16, 48, 128, 128
    g = torch.Generator().manual_seed(B)
    mixed = torch.randn((B, 2 * H * K + HV * V), generator=g).to(torch.bfloat16)
    ba = torch.randn((B, 2 * HV), generator=g).to(torch.bfloat16)
    a, b = ba[:, :HV], ba[:, HV:]  # strided gate views
    A_log = torch.log(torch.rand(HV, generator=g) * 16 + 1e-3)
    dt_bias = torch.randn(HV, generator=g)
    state = (torch.randn((B + 3, HV, V, K), generator=g) * 0.1).to(sd)
    idx = torch.randperm(B + 3, generator=g)[:B].to(torch.int32)
    if B > 4:
        idx[0] = -1
    q, k, v = torch.split(mixed, [H * K, H * K, HV * V], dim=-1)
    ref_state = state.clone()
    ref = gdn_oracle.recurrent_spec(q.view(B, 1, H, K), k.view(B, 1, H, K), v.view(B, 1, HV, V), a.unsqueeze(1),
                                    b.unsqueeze(1), A_log, dt_bias, ref_state, idx, None, round_beta_bf16=True)
    call = dict(mixed_qkv=mixed.cuda(), a=ba.cuda()[:, :HV], b=ba.cuda()[:, HV:], A_log=A_log.cuda(),
                dt_bias=dt_bias.cuda(), scale=K ** -0.5, ssm_states=state.cuda(), cache_indices=idx.cuda(),
                num_v_heads=HV, head_v_dim=V)
    run = gdn_recurrent._select_packed(call)
    assert callable(run), run
    out = run(**call)
    torch.cuda.synchronize()
    assert out.shape == (1, B, HV, V) and out.dtype == torch.bfloat16
    err = (out.float().cpu()[0] - ref[:, 0]).abs().max().item()
    assert err <= (1e-3 if sd is torch.float32 else 2e-3), err
    rel = ((call["ssm_states"].float().cpu() - ref_state.float()).norm() / ref_state.float().norm()).item()
    assert rel <= (1e-5 if sd is torch.float32 else 1e-2), rel
    if B > 4:
        assert out[0, 0].abs().max().item() == 0.0
        untouched = sorted(set(range(B + 3)) - {int(i) for i in idx if i >= 0})
        assert torch.equal(call["ssm_states"].cpu()[untouched], state[untouched])


def test_split_decode_pad_and_length_semantics():
    from greenattention_b200 import gdn_recurrent
    from oracle import gdn_oracle

    H, HV, K, V, B = 16, 32, 128, 128, 6
    c = W.make_gdn_case(B, 1, h=H, hv=HV, seed=31, gate_params="rand", normalise_qk=False, state_std=0.1, pad_rows=(1,))
    ref_state = c["ssm_states"].clone()
    ref = gdn_oracle.recurrent_spec(c["q"], c["k"], c["v"], c["a"], c["b"], c["A_log"], c["dt_bias"], ref_state,
                                    c["cache_indices"], None, pad_reads_zero=True)
    g = to_cuda(c)
    qsl = torch.arange(B + 1, dtype=torch.int32)
    qsl[-1] += 1  # the last request claims two tokens: zero output, untouched state
    call = dict(q=g["q"].view(1, B, H, K), k=g["k"].view(1, B, H, K), v=g["v"].view(1, B, HV, V),
                a=g["a"].view(B, HV), b=g["b"].view(B, HV), A_log=g["A_log"], dt_bias=g["dt_bias"],
                ssm_states=g["ssm_states"], cache_indices=g["cache_indices"], query_start_loc=qsl.cuda())
    run = gdn_recurrent._select_split(call)
    assert callable(run), run
    out = run(**call).float().cpu()[0]
    assert (out[:B - 1] - ref[:B - 1, 0]).abs().max().item() <= 1e-3
    assert out[1].abs().max().item() > 0  # PAD row still produces output from a zero state
    assert out[B - 1].abs().max().item() == 0.0
    st = g["ssm_states"].cpu()
    last = int(c["cache_indices"][B - 1])
    assert torch.equal(st[last], c["ssm_states"][last])
    keep = [int(i) for n, i in enumerate(c["cache_indices"].tolist()) if i >= 0 and n != B - 1]
    assert ((st[keep] - ref_state[keep]).norm() / ref_state[keep].norm()).item() <= 1e-5


def test_deterministic_and_graph_replay_equals_eager():
    from greenattention_b200 import gdn_recurrent

    base = to_cuda(W.make_gdn_case(32, 4, h=16, hv=32, seed=5))
    kw = {n: base[n] for n in ("q", "k", "v", "a", "b", "A_log", "dt_bias", "cache_indices", "accept_lens", "scale")}
    s1, s2, s3 = (base["ssm_states"].clone() for _ in range(3))
    o1 = gdn_recurrent.gdn_spec_decode(ssm_states=s1, **kw)
    o2 = gdn_recurrent.gdn_spec_decode(ssm_states=s2, **kw)
    assert torch.equal(o1, o2) and torch.equal(s1, s2)
    out = torch.empty_like(o1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        gdn_recurrent.gdn_spec_decode(ssm_states=s3.clone(), out=out, **kw)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gdn_recurrent.gdn_spec_decode(ssm_states=s3, out=out, **kw)
    for _ in range(3):
        s3.copy_(base["ssm_states"])
        graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, o1) and torch.equal(s3, s1)


def test_back_to_back_calls():
    from greenattention_b200 import gdn_recurrent

    variants = [to_cuda(W.make_gdn_case(b, t, h=16, hv=32, seed=90 + i))
                for i, (b, t) in enumerate([(8, 4), (3, 1), (17, 2)])]
    refs = []
    for c in variants:
        ref, ref_st = oracle_spec({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in c.items()})
        refs.append((ref, ref_st, c["ssm_states"].clone()))
    for it in range(60):
        c, (ref, ref_st, start) = variants[it % 3], refs[it % 3]
        c["ssm_states"].copy_(start)
        out = gdn_recurrent.gdn_spec_decode(
            q=c["q"], k=c["k"], v=c["v"], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
            ssm_states=c["ssm_states"], cache_indices=c["cache_indices"], accept_lens=c["accept_lens"],
            out_dtype=torch.float32)
        assert_close(out.cpu(), ref, c["ssm_states"].cpu(), ref_st)


def test_declines():
    from greenattention_b200 import gdn_recurrent

    c = to_cuda(W.make_gdn_case(4, 4, h=16, hv=32, seed=6))
    base = dict(q=c["q"], k=c["k"], v=c["v"], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
                ssm_states=c["ssm_states"], cache_indices=c["cache_indices"], accept_lens=c["accept_lens"])
    for mutate, needle in (
        (lambda kw: kw.update(q=kw["q"].float()), "dtype"),
        (lambda kw: kw.update(ssm_states=kw["ssm_states"][:, :, :64]), "state shape"),
        (lambda kw: kw.update(accept_lens=kw["accept_lens"].long()), "accept_lens"),
        (lambda kw: kw.update(A_log=kw["A_log"][:5]), "A_log"),
    ):
        kw = dict(base)
        mutate(kw)
        why = gdn_recurrent._select_spec(kw)
        assert isinstance(why, str) and needle in why, why
