"""Replay-SSM verify: the oracle against the contract's closed form, and the host-side selector. No GPU.

The oracle (``oracle/gdn_oracle.replay_verify``) folds the ring history into the state and runs the ordinary
chained recurrence; the closed form (``replay_verify_closed_form``) evaluates ``T = (I + A)^-1``, ``D = R T^T``,
``O = e^G hw_q + D F`` with the history as a correction of ``hw_q`` / ``hw_k``, exactly as the reference documents
its kernels (``docs/gdn-contract.md:111-124``). Both must give the same outputs.
"""

import copy

import pytest
import torch

from greenattention_b200 import workloads as W


@pytest.mark.parametrize("ring_len", [16, 32])
@pytest.mark.parametrize("seed", [1, 2])
def test_oracle_matches_the_closed_form(ring_len, seed):
    from oracle import gdn_oracle

    c = W.make_gdn_replay_case([4, 2, 0, 3, 4, 1, 4], h=2, hv=6, ring_len=ring_len, pad_rows=(1,), flush_rows=(3,),
                               seed=seed)
    c2 = copy.deepcopy(c)
    seq = gdn_oracle.replay_verify(c)
    closed = gdn_oracle.replay_verify_closed_form(c2)
    live = ~torch.isnan(seq)
    assert torch.equal(torch.isnan(closed), ~live)
    assert (seq[live] - closed[live]).abs().max().item() <= 1e-12 * max(1.0, seq[live].abs().max().item())
    assert seq[c["query_start_loc"][1]:c["query_start_loc"][2]].abs().max().item() == 0.0  # PAD rows


def test_oracle_with_empty_ring_is_the_plain_chained_recurrence():
    from oracle import gdn_oracle

    spec = [4, 4, 4]
    c = W.make_gdn_replay_case(spec, h=2, hv=4, ring_len=16, write_pos=[0, 0, 0], seed=3)
    out = gdn_oracle.replay_verify(copy.deepcopy(c), dtype=torch.float32)
    B, T = len(spec), 4
    st = c["checkpoint_state"].clone()
    ref = gdn_oracle.recurrent_spec(
        c["q"].view(B, T, 2, 128), c["k"].view(B, T, 2, 128), c["v"].view(B, T, 4, 128), c["a"].view(B, T, 4),
        c["b"].view(B, T, 4), c["A_log"], c["dt_bias"], st, c["ssm_state_indices"],
        torch.zeros(B, dtype=torch.int32), scale=c["scale"])
    assert (out.view(B, T, 4, 128) - ref).abs().max().item() <= 1e-5
    assert torch.equal(st, c["checkpoint_state"])


def test_oracle_ring_writes_follow_the_cursor():
    from oracle import gdn_oracle

    L = 16
    c = W.make_gdn_replay_case([4, 4, 3], h=2, hv=4, ring_len=L, write_pos=[14, 16, 0], cache_base=[15, 3, 7], seed=4)
    before = copy.deepcopy(c)
    gdn_oracle.replay_verify(c)
    for name in ("d_cache", "rawv_cache", "k_cache", "rawk_cache", "g_cache"):
        changed = c[name].float() != before[name].float()
        pos = changed.any(dim=1) if name == "g_cache" else changed.any(dim=3).any(dim=1)  # [ring, L]
        # slot 0: 14 entries from position 15 -> tokens 0, 1 land at (15+14)&15 = 13 and 14; tokens 2, 3 are dropped
        assert set(torch.nonzero(pos[0]).flatten().tolist()) <= {13, 14}
        assert not pos[1].any()               # full ring: nothing written
        assert set(torch.nonzero(pos[2]).flatten().tolist()) <= {7, 8, 9}
    assert torch.equal(c["checkpoint_state"], before["checkpoint_state"])
    for name in ("write_pos", "cache_base", "is_flush"):
        assert torch.equal(c[name], before[name])


@pytest.mark.parametrize(
    "mutate, needle",
    [
        (lambda c: c.update(launch_mode="decode"), "launch_mode"),
        (lambda c: c.update(beta_cache=torch.zeros(1)), "beta_cache"),
        (lambda c: c.update(max_cache_len=8), "max_cache_len"),
        (lambda c: c.update(use_qk_l2norm_in_kernel=False), "l2norm"),
        (lambda c: c.update(null_block_id=0), "null_block_id"),
        (lambda c: c.update(max_spec_len=5), "max_spec_len"),
        (lambda c: c.update(q=c["q"].float()), "q dtype"),
        (lambda c: c.update(scale=0.5), "scale"),
        (lambda c: c.update(rawv_cache=None), "rawv_cache"),
        (lambda c: c.update(is_flush=c["is_flush"].to(torch.int32)), "is_flush"),
        (lambda c: c.update(out=c["out"].float()), "out"),
        (lambda c: c.update(checkpoint_state=c["checkpoint_state"].double()), "state dtype"),
    ],
)
def test_selector_declines_what_the_kernel_does_not_serve(mutate, needle):
    from greenattention_b200 import gdn_recurrent

    c = W.make_gdn_replay_case([4, 2], h=2, hv=4, ring_len=16)
    assert gdn_recurrent._verify_supported(c) is None
    mutate(c)
    reason = gdn_recurrent._verify_supported(c)
    assert isinstance(reason, str) and needle in reason, reason


def test_flat_layout_and_int64_indices_are_accepted():
    from greenattention_b200 import gdn_recurrent

    c = W.make_gdn_replay_case([4, 2, 1], h=2, hv=6, ring_len=32, flat=True, idx_dtype=torch.int64)
    assert gdn_recurrent._verify_supported(c) is None


def test_hook_hands_other_calls_to_the_stock_function(monkeypatch):
    from greenattention_b200 import gdn_recurrent

    monkeypatch.setattr(gdn_recurrent, "_on_green_sm100", lambda: True)
    c = W.make_gdn_replay_case([4], h=2, hv=4, ring_len=16)
    c["launch_mode"] = "decode"
    assert gdn_recurrent._replayssm_around(lambda *a, **k: "stock", **c) == "stock"
