"""The CPU oracle against the golden fixtures (outputs of the reference's own torch oracle, and of the
third-party naive GDN recurrence), and the seeded generators against the recorded input digests."""

import json
import os

import numpy as np
import pytest
import torch

from oracle import attn_oracle, gdn_oracle
from tests.golden import cases

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


@pytest.mark.parametrize("name", sorted(cases.ATTN_CASES))
def test_attention_oracle_matches_reference_outputs(name):
    kw = cases.ATTN_CASES[name]()
    gold = load("attn_" + name)
    assert cases.digest(kw) == str(gold["digest"]), "seeded generator drifted from the fixture inputs"
    out, lse = attn_oracle.paged_attention(kw)
    ref_out, ref_lse = torch.from_numpy(gold["out"]), torch.from_numpy(gold["lse"])
    assert out.shape == ref_out.shape and lse.shape == ref_lse.shape
    assert torch.equal(torch.isfinite(lse), torch.isfinite(ref_lse))
    assert (out - ref_out).abs().max().item() <= 2e-5
    fin = torch.isfinite(ref_lse)
    assert (lse[fin] - ref_lse[fin]).abs().max().item() <= 2e-5


def test_merge_of_range_partials_equals_whole():
    kw = cases.ATTN_CASES["saturation"]()
    one = {k: (v[:1] if isinstance(v, torch.Tensor) and k in ("q", "page_table", "cache_seqlens", "k_descale",
                                                                 "v_descale") else v) for k, v in kw.items()}
    one["cu_seqlens_q"] = kw["cu_seqlens_q"][:2]
    L = int(one["cache_seqlens"][0])
    whole, whole_lse = attn_oracle.paged_attention(one)
    parts = attn_oracle.kv_range_partials(one, [(0, 400), (400, 401), (401, 1100), (1100, L), (L, L + 50)])
    o, lse = attn_oracle.merge_partials(*parts)
    assert (o - whole[0]).abs().max().item() <= 1e-5
    assert (lse - whole_lse[:, 0]).abs().max().item() <= 1e-5


def test_merge_all_empty_is_zero_and_minus_inf():
    o, lse = attn_oracle.merge_partials(torch.randn(3, 4, 8), torch.full((3, 4), -float("inf")))
    assert torch.count_nonzero(o) == 0 and torch.isinf(lse).all() and (lse < 0).all()


@pytest.mark.parametrize("name", sorted(cases.GDN_CASES))
def test_gdn_oracle_matches_independent_recurrence(name):
    c = cases.gdn_case(name)
    gold = load("gdn_" + name)
    assert cases.digest(c) == str(gold["digest"])
    before = c["ssm_states"].clone()
    out = gdn_oracle.recurrent_spec(
        c["q"], c["k"], c["v"], c["a"], c["b"], c["A_log"], c["dt_bias"], c["ssm_states"], c["cache_indices"],
        c["accept_lens"], scale=c["scale"],
    )
    ref = torch.from_numpy(gold["out"])
    assert (out - ref).abs().max().item() <= 1e-3 * ref.abs().max().item()
    idx = c["cache_indices"].long()
    st = c["ssm_states"][idx]
    ref_st = torch.from_numpy(gold["state"])
    rel = ((st - ref_st).norm() / ref_st.norm()).item()
    assert rel <= 1e-5, rel
    # accepted-prefix bookkeeping is bit-exact: accept 0 leaves the slot untouched, unreferenced slots too
    acc = c["accept_lens"].tolist()
    for n, a in enumerate(acc):
        if a == 0:
            assert torch.equal(c["ssm_states"][idx[n]], before[idx[n]])
    untouched = sorted(set(range(before.shape[0])) - set(idx.tolist()))
    assert torch.equal(c["ssm_states"][untouched], before[untouched])


def test_gdn_pad_semantics():
    c = cases.gdn_case("spec4")
    c["cache_indices"][1] = -1
    before = c["ssm_states"].clone()
    args = (c["q"], c["k"], c["v"], c["a"], c["b"], c["A_log"], c["dt_bias"])
    st = c["ssm_states"].clone()
    out = gdn_oracle.recurrent_spec(*args, st, c["cache_indices"], None, scale=c["scale"])
    assert torch.count_nonzero(out[1]) == 0
    st2 = before.clone()
    out2 = gdn_oracle.recurrent_spec(*args, st2, c["cache_indices"], None, scale=c["scale"], pad_reads_zero=True)
    assert torch.count_nonzero(out2[1]) > 0
    assert torch.equal(st, st2)


def test_host_tables_fixture_is_well_formed():
    with open(os.path.join(GOLD, "host_tables.json")) as f:
        t = json.load(f)
    assert t["ops"] == ["decode", "verify", "extend", "gdn_decode", "gdn_verify"] and t["max_verify_q"] == 16
    assert len(t["plan_splits"]) == 1152


def test_extract_requests_gives_the_same_attention_as_the_whole_call():
    """``workloads.extract_requests`` (the sampler the full-size GPU tests and the bench use to check part of a
    call on the host) must not change what the oracle computes for the requests it keeps."""
    from greenattention_b200 import workloads as W
    from oracle import attn_oracle

    kw = W.make_paged_case([300, 0, 41, 1000, 64], [2, 2, 1, 3, 2], 16, q_heads=8, kv_heads=2, head_dim=128, seed=44,
                           descale="rand", window=(200, 0), kv_stack=True, q_strided=True)
    whole, lse = attn_oracle.paged_attention(kw)
    pick = [3, 0, 4]
    sub = W.extract_requests(kw, pick)
    part, lse_part = attn_oracle.paged_attention(sub)
    rows = W.request_rows(kw, pick)
    assert torch.equal(part, whole[rows])
    assert torch.equal(lse_part, lse[:, rows])
    assert sub["k_cache"].shape[0] == 63 + 19 + 4  # only the pages those requests own
