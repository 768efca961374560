"""``ga_attn_decode_noalloc`` (the decode entry point for hosts that cannot supply a workspace) against
``ga_attn_decode`` on the same inputs, through the C ABI.

Where the two entry points launch the same kernels (head_dim 128 with at most 8 rows per kv head) only the
scratch differs (a fixed array inside the library versus the caller's workspace), so their outputs must agree
to the bit. For the other shapes the workspace entry point takes the tcgen05 kernel while this one keeps the
warp-level kernel: two implementations of the same math, which must agree far inside the tolerance. Different
calls are made in a row because the built-in array keeps the previous call's contents: a stale split plan or
partial slot would show up in the next one. The file is named to be collected last.
"""

import ctypes

import pytest
import torch

from greenattention_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _both(kw):
    from greenattention_b200 import attn_decode

    run = attn_decode.select(kw)
    assert callable(run), run
    ref_out, ref_lse = run(**kw)
    out, lse = attn_decode.decode_noalloc(**kw)
    torch.cuda.synchronize()
    return (out, lse), (ref_out, ref_lse)


def test_noalloc_matches_workspace_entry_point_twice_in_a_row():
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    attn_decode.ensure_ready()
    first = W.make_paged_case([20000, 137, 0, 4097, 64, 9000], [1] * 6, 16, q_heads=16, kv_heads=2, head_dim=128,
                              seed=301, descale="rand", extra_pages=4)
    second = W.make_paged_case([3, 700, 31000], [2, 2, 2], 64, q_heads=16, kv_heads=2, head_dim=128, seed=302,
                               window=(511, 0))
    # head_dim 256 takes other kernel instances (GQA 2 decode: the 8-row one; GQA 6 x 2 tokens: the 16-row one)
    third = W.make_paged_case([9000, 1, 300, 0, 2500], [1] * 5, 64, q_heads=4, kv_heads=2, head_dim=256, seed=305,
                              descale="rand", window=(1023, 0))
    fourth = W.make_paged_case([5000, 70], [2, 2], 16, q_heads=12, kv_heads=2, head_dim=256, seed=306)
    dev = torch.device("cuda", torch.cuda.current_device())
    for kw_cpu in (first, second, third, fourth):
        kw = W.case_to(kw_cpu, "cuda")
        (out, lse), (ref_out, ref_lse) = _both(kw)
        rows = kw["max_seqlen_q"] * (kw["q"].shape[1] // kw["k_cache"].shape[2])
        if kw["q"].shape[2] == 128 and rows <= 8:
            assert torch.equal(out, ref_out)
            assert torch.equal(lse, ref_lse)
        else:
            diff = (out.float() - ref_out.float()).abs()
            assert (diff <= 5e-3 + 1e-2 * ref_out.float().abs()).all()  # a bf16 step of the larger outputs at most
            fin = torch.isfinite(ref_lse)
            assert torch.equal(torch.isfinite(lse), fin)
            assert (lse[fin] - ref_lse[fin]).abs().max().item() <= 2e-3
        # the status word of the built-in array is readable after the call (and says the call was clean)
        assert attn_decode.workspace_status(dev, builtin=True) == 0
        ref_o, _ = attn_oracle.paged_attention(kw_cpu)
        assert ((out.float().cpu() - ref_o).abs() <= 2e-2 + 2e-2 * ref_o.abs()).all()


def test_noalloc_status_word_reports_a_bad_call_until_the_next_call_clears_it():
    from greenattention_b200 import attn_decode

    attn_decode.ensure_ready()
    dev = torch.device("cuda", torch.cuda.current_device())
    kw = W.case_to(W.make_paged_case([200, 64], [1, 1], 64, q_heads=8, kv_heads=2, head_dim=128, seed=307, pt_pad=0), "cuda")
    good_lens = kw["cache_seqlens"].clone()
    kw["cache_seqlens"] = torch.tensor([kw["page_table"].shape[1] * 64 + 1, 64], dtype=torch.int32, device="cuda")
    attn_decode.decode_noalloc(**kw)
    assert attn_decode.workspace_status(dev, builtin=True) == 5  # length beyond the page-table row: cut and recorded
    kw["cache_seqlens"] = good_lens
    attn_decode.decode_noalloc(**kw)
    assert attn_decode.workspace_status(dev, builtin=True) == 0


def test_noalloc_rejects_calls_beyond_its_scratch():
    from greenattention_b200 import _C, attn_decode

    attn_decode.ensure_ready()
    big_rows = W.case_to(W.make_paged_case([300, 40], [4, 4], 16, q_heads=16, kv_heads=2, head_dim=128, seed=303), "cuda")
    with pytest.raises(_C.GreenAttentionError, match="exceeds the built-in scratch"):
        attn_decode.decode_noalloc(**big_rows)
    lens = [8] * 1025
    big_batch = W.case_to(W.make_paged_case(lens, [1] * 1025, 16, q_heads=4, kv_heads=2, head_dim=128, seed=304), "cuda")
    with pytest.raises(_C.GreenAttentionError, match="exceeds the built-in scratch"):
        attn_decode.decode_noalloc(**big_batch)
    assert isinstance(ctypes.sizeof(_C.GaAttnParams), int)
