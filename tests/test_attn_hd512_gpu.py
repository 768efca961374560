"""head_dim 512 decode (four 128-byte slabs per head; the reference's Gemma-4 global shape, instance (512, 8) of
``green_attention/attn_decode.py:58-62``) on the GPU against the CPU oracle, through the plugin front-end and the C ABI.

Built here: the decode step (one query token, GQA <= 8, i.e. at most 8 rows per kv head) on the per-head split-KV
kernel. Not built: more query tokens per request and extend at this head dim; the selectors decline them with a reason.
The matrix is the decode part of the reference's op tests (``op_test/sm90/test_attn_decode_fp8.py:219-365``).

Tolerance: the same as every other shape (bf16 output within atol 2e-2 + rtol 2e-2, LSE within 5e-3). The reference
allows its own head_dim 512 kernel the rounding floor of an e4m3 P (``test_attn_decode_fp8.py:178-192``); this kernel's
P carries a residual term (about 2^-8 relative), so it does not need that allowance.
"""

import pytest
import torch

from greenattention_b200 import dispatch
from greenattention_b200 import workloads as W
from tests.test_attn_gpu import check, compare, run

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn

G8 = dict(q_heads=32, kv_heads=4, head_dim=512)  # Gemma-4 global attention
G4 = dict(q_heads=8, kv_heads=2, head_dim=512)
G1 = dict(q_heads=3, kv_heads=3, head_dim=512)
LENS = [1, 2, 63, 64, 65, 127, 129, 1000, 4097]


@pytest.fixture(scope="module", autouse=True)
def _ready():
    from greenattention_b200 import attn_decode

    attn_decode.ensure_ready()
    yield
    assert attn_decode.workspace_status(torch.device("cuda", torch.cuda.current_device())) == 0


@pytest.mark.parametrize("inst", [G8, G4, G1], ids=["gqa8", "gqa4", "mha"])
@pytest.mark.parametrize("page", [16, 64, 128])
@pytest.mark.parametrize("q_dtype", [FP8, torch.bfloat16])
def test_ragged_lengths(inst, page, q_dtype):
    check(W.make_paged_case(LENS, [1] * len(LENS), page, q_dtype=q_dtype, seed=page + inst["kv_heads"], descale="rand", **inst))


def test_pages_below_the_tma_box():
    check(W.make_paged_case([1, 5, 40, 333], [1] * 4, 4, seed=3, descale="rand", **G8))


def test_empty_sequences_and_whole_batch_empty():
    check(W.make_paged_case([0, 17, 0, 300], [1, 1, 1, 1], 64, seed=6, **G8))
    check(W.make_paged_case([0, 0, 0], [1, 1, 1], 64, seed=6, **G8))


@pytest.mark.parametrize("batch", [1, 3])
def test_long_context_is_cut_into_many_slices(batch):
    lens = [40000 - 7777 * i for i in range(batch)]
    check(W.make_paged_case(lens, [1] * batch, 64, seed=11, extra_pages=8, descale="rand", kv_std=0.5, **G8))


def test_production_like_batch():
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1, 6000, (40,), generator=g).tolist()
    lens[7], lens[20] = 0, 1
    check(W.make_paged_case(lens, [1] * 40, 64, seed=21, descale="rand", descale_range=(0.5, 2.0), kv_std=0.5, **G8))


@pytest.mark.parametrize("L", [1, 1023, 1024, 1025, 1089, 5000])
def test_window_edges(L):
    check(W.make_paged_case([L, 7, 3000], [1, 1, 1], 64, seed=L % 97, window=(1023, 0), **G8))


@pytest.mark.parametrize("descale", ["none", "scalar", "rand"])
def test_descale_forms(descale):
    check(W.make_paged_case([500, 129, 2000], [1, 1, 1], 64, descale=descale, seed=8, **G8))


def test_fp8_saturation_range():
    kw = W.make_paged_case([1500, 333, 64], [1, 1, 1], 64, kv_std=150.0, seed=9, **G4)
    kw["k_descale"] = torch.full((3, 2), 1 / 150.0)
    kw["v_descale"] = torch.full((3, 2), 1 / 150.0)
    check(kw)


def test_peaked_softmax_short_rows():
    check(W.make_paged_case([3, 9, 40, 70], [1, 1, 1, 1], 64, seed=41, q_std=2.0, kv_std=2.0, **G8), lse_tol=1e-2)


@pytest.mark.parametrize("out_mode", ["given", "strided"])
def test_out_argument_and_strided_views(out_mode):
    check(W.make_paged_case([700, 129, 33], [1, 1, 1], 64, out_mode=out_mode, q_strided=True, kv_stack=True, seed=12, **G8))


def test_no_lse():
    check(W.make_paged_case([700, 129], [1, 1], 64, return_lse=False, seed=15, **G8))


def test_deterministic():
    kw = W.case_to(W.make_paged_case([4000, 129, 900, 20000], [1] * 4, 64, seed=16, **G8), "cuda")
    a, la = run(kw)
    b, lb = run(kw)
    assert torch.equal(a, b) and torch.equal(la, lb)


def test_cuda_graph_replay_with_changed_lengths():
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    lens = [2048 + 37 * i for i in range(8)]
    kw_cpu = W.make_paged_case(lens, [1] * 8, 64, seed=25, extra_pages=4, pt_pad=16, **G8)
    kw = W.case_to(kw_cpu, "cuda")
    fn = attn_decode.select(kw)
    assert callable(fn)
    fn(**kw)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            static_out = fn(**kw)
    for shrink in (5, 700, 2047):
        new_lens = [max(0, L - shrink - 3 * i) for i, L in enumerate(lens)]
        kw["cache_seqlens"].copy_(torch.tensor(new_lens, dtype=torch.int32))
        kw_cpu["cache_seqlens"] = torch.tensor(new_lens, dtype=torch.int32)
        graph.replay()
        torch.cuda.synchronize()
        ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
        compare(static_out[0], static_out[1], ref_o, ref_lse)


def test_what_is_not_built_is_declined_with_a_reason():
    from greenattention_b200 import attn_decode

    two_tokens = W.case_to(W.make_paged_case([700, 129], [2, 2], 64, seed=16, **G8), "cuda")  # 16 rows per kv head
    why = attn_decode.select(two_tokens)
    assert isinstance(why, str) and "at most 8 rows" in why
    assert callable(attn_decode.select(W.case_to(W.make_paged_case([700, 129], [2, 2], 64, seed=16, **G4), "cuda")))  # 8 rows
    ext = W.case_to(W.make_paged_case([700], [300], 64, seed=17, **G8), "cuda")
    why = attn_decode.select_extend(ext)
    assert isinstance(why, str) and "no extend kernel for head_dim 512" in why
    one = W.case_to(W.make_paged_case([700, 129], [1, 1], 64, seed=18, **G8), "cuda")
    with pytest.raises(dispatch.Declined):
        attn_decode.decode_noalloc(**one)
