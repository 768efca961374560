"""Replay-SSM verify on the GPU, through ``gdn_recurrent.gdn_replayssm_verify`` and the C ABI, against the CPU oracle.

Cases follow what the reference's contract pins for this call (``docs/gdn-contract.md:83-132``; its GPU tests,
``op_test/sm90/test_gdn_recurrent.py:128-258``, compare with SGLang's Triton kernel, which is not available here):
ragged spec lens 0..4, PAD rows, rows under flush, ring lengths 16 / 32, empty / partly full / full rings with
wrap-around, 2 or 3 value heads per key head, fp32 and bf16 checkpoint, flattened q/k/v/out, int64 indices,
determinism, and that nothing but ``out`` and the ring rows at the cursor is written.

Tolerance: bf16 outputs within 2^-8 relative + 1e-3 of the largest reference magnitude of the fp64 oracle (bf16
rounding of the output plus fp32 accumulation); the ring rows as (high + residual) within 1e-3 of the largest
magnitude (2e-2 with a bf16 checkpoint); gates within 1e-6; everything that must stay untouched bit-identical.
"""

import copy

import pytest
import torch

from greenattention_b200 import workloads as W

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _force_gate(monkeypatch):
    import greenattention_b200.gdn as gdn_mod
    from greenattention_b200 import gdn_recurrent

    monkeypatch.setattr(gdn_mod, "_green_on_sm100", lambda: True)
    gdn_recurrent.ensure_ready()


def to_cuda(c):
    return {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in c.items()}


def run_and_check(c, state_tol=1e-3):
    from greenattention_b200 import gdn_recurrent
    from oracle import gdn_oracle

    before = copy.deepcopy(c)
    g = to_cuda(copy.deepcopy(c))
    out = gdn_recurrent.gdn_replayssm_verify(**g)
    torch.cuda.synchronize()
    assert out.data_ptr() == g["out"].data_ptr()
    ref_call = copy.deepcopy(c)
    ref = gdn_oracle.replay_verify(ref_call).float()
    T = ref.shape[0]
    got = out.float().cpu().reshape(T, -1, 128)
    flushed = torch.isnan(ref)
    # rows of flushed requests keep what the caller put there
    assert torch.equal(got[flushed], before["out"].float().reshape(T, -1, 128)[flushed])
    live = ~flushed
    if live.any():
        scale = max(ref[live].abs().max().item(), 1e-6)
        err = (got[live] - ref[live]).abs()
        bound = ref[live].abs() * 2.0**-8 + state_tol * scale
        assert (err <= bound).all(), f"out err {err.max().item()} vs scale {scale}"
    # ring: rows the oracle wrote, compared as high + residual; every other ring entry bit-identical
    for hi_name, lo_name in (("d_cache", "rawv_cache"), ("k_cache", "rawk_cache")):
        want_hi, want_lo = ref_call[hi_name].float(), ref_call[lo_name].float()
        got_hi, got_lo = g[hi_name].float().cpu(), g[lo_name].float().cpu()
        written = ((want_hi != before[hi_name].float()) | (want_lo != before[lo_name].float())).any(dim=3).any(dim=1)
        want, have = want_hi + want_lo, got_hi + got_lo
        mask = written[:, None, :, None].expand_as(want)
        if mask.any():
            mag = max(want[mask].abs().max().item(), 1e-6)
            assert (have[mask] - want[mask]).abs().max().item() <= state_tol * mag, hi_name
            # the high part is the bf16 rounding of the value: allow one bf16 step where the fp32 value sits on a tie
            assert (got_hi[mask] - want_hi[mask]).abs().max().item() <= 2.0**-7 * mag + state_tol * mag
        assert torch.equal(got_hi[~mask], before[hi_name].float()[~mask]), f"{hi_name} touched outside the cursor"
        assert torch.equal(got_lo[~mask], before[lo_name].float()[~mask]), f"{lo_name} touched outside the cursor"
    gw = ref_call["g_cache"] != before["g_cache"]
    gg = g["g_cache"].cpu()
    if gw.any():
        assert (gg[gw] - ref_call["g_cache"][gw]).abs().max().item() <= 1e-6
    assert torch.equal(gg[~gw], before["g_cache"][~gw])
    for name in ("checkpoint_state", "write_pos", "cache_base", "is_flush", "q", "k", "v"):
        assert torch.equal(g[name].cpu(), before[name]), f"{name} modified"
    return got


@pytest.mark.parametrize("ring_len", [16, 32])
@pytest.mark.parametrize("heads", [(16, 32), (16, 48), (4, 4)])
def test_ragged_batch_with_pad_and_flush(ring_len, heads):
    h, hv = heads
    spec = [4, 2, 0, 3, 4, 1, 4, 4, 2, 3]
    run_and_check(W.make_gdn_replay_case(spec, h=h, hv=hv, ring_len=ring_len, pad_rows=(1, 6), flush_rows=(4,),
                                         seed=10 + ring_len + hv))


@pytest.mark.parametrize("write_pos", [0, 1, 13, 14, 15, 16])
def test_ring_cursor_positions(write_pos):
    """Empty ring, one entry, room for 3 / 2 / 1 of 4 new tokens, full ring; the base wraps around the end."""
    L = 16
    run_and_check(W.make_gdn_replay_case([4, 4, 3, 1], h=4, hv=8, ring_len=L, write_pos=[write_pos] * 4,
                                         cache_base=[0, 15, 9, 3], seed=30 + write_pos))


def test_empty_ring_equals_the_committing_kernel():
    """With no history the outputs are those of the chained step that commits nothing."""
    from greenattention_b200 import gdn_recurrent

    B, T, h, hv = 6, 4, 4, 8
    c = W.make_gdn_replay_case([T] * B, h=h, hv=hv, ring_len=16, write_pos=[0] * B, seed=41)
    got = run_and_check(c)
    g = to_cuda(c)
    out = gdn_recurrent.gdn_spec_decode(
        q=g["q"].view(B, T, h, 128), k=g["k"].view(B, T, h, 128), v=g["v"].view(B, T, hv, 128),
        a=g["a"].view(B, T, hv), b=g["b"].view(B, T, hv), A_log=g["A_log"], dt_bias=g["dt_bias"],
        ssm_states=g["checkpoint_state"].clone(), cache_indices=g["ssm_state_indices"],
        accept_lens=torch.zeros(B, dtype=torch.int32, device="cuda"), scale=g["scale"], out_dtype=torch.bfloat16)
    torch.cuda.synchronize()
    assert torch.equal(out.float().cpu().view(B * T, hv, 128), got)


def test_bf16_checkpoint_flat_layout_and_int64_indices():
    c = W.make_gdn_replay_case([4, 3, 4, 2], h=4, hv=12, ring_len=32, state_dtype=torch.bfloat16, flat=True,
                               idx_dtype=torch.int64, seed=51)
    run_and_check(c, state_tol=2e-3)


def test_bf16_dt_bias():
    c = W.make_gdn_replay_case([4, 4], h=4, hv=8, ring_len=32, seed=52)
    c["dt_bias"] = c["dt_bias"].to(torch.bfloat16)
    run_and_check(c)


def test_deterministic_and_back_to_back():
    from greenattention_b200 import gdn_recurrent

    c = W.make_gdn_replay_case([4, 2, 3, 4, 4, 1], h=16, hv=32, ring_len=32, seed=61)
    outs = []
    for _ in range(3):
        g = to_cuda(copy.deepcopy(c))
        outs.append((gdn_recurrent.gdn_replayssm_verify(**g).clone(), g["d_cache"].clone(), g["k_cache"].clone()))
    torch.cuda.synchronize()
    for o, d, k in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(d, outs[0][1]) and torch.equal(k, outs[0][2])


def test_cuda_graph_replay_equals_eager():
    from greenattention_b200 import gdn_recurrent

    c = W.make_gdn_replay_case([4, 4, 2, 3], h=16, hv=32, ring_len=32, seed=71)
    eager = to_cuda(copy.deepcopy(c))
    gdn_recurrent.gdn_replayssm_verify(**eager)
    g = to_cuda(copy.deepcopy(c))
    gdn_recurrent.gdn_replayssm_verify(**to_cuda(copy.deepcopy(c)))  # warm-up outside capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        gdn_recurrent.gdn_replayssm_verify(**g)
    for name in ("d_cache", "rawv_cache", "k_cache", "rawk_cache", "g_cache", "out"):
        g[name].copy_(c[name].cuda().reshape(g[name].shape))
    graph.replay()
    torch.cuda.synchronize()
    for name in ("out", "d_cache", "rawv_cache", "k_cache", "rawk_cache", "g_cache"):
        assert torch.equal(g[name], eager[name]), name
