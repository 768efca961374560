"""``ga_attn_decode_noalloc`` (the decode entry point for hosts that cannot supply a workspace) against
``ga_attn_decode`` on the same inputs, through the C ABI.

The two entry points launch the same kernels; only the scratch differs (a fixed array inside the library
versus the caller's workspace), so their outputs must agree to the bit. Two different calls are made in a
row because the built-in array keeps the previous call's contents: a stale split plan or partial slot would
show up in the second one. The file is named to be collected last.
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
    for kw_cpu in (first, second):
        kw = W.case_to(kw_cpu, "cuda")
        (out, lse), (ref_out, ref_lse) = _both(kw)
        assert torch.equal(out, ref_out)
        assert torch.equal(lse, ref_lse)
        ref_o, _ = attn_oracle.paged_attention(kw_cpu)
        assert ((out.float().cpu() - ref_o).abs() <= 2e-2 + 2e-2 * ref_o.abs()).all()


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
