"""The all-heads decode kernel (``attn_wide_kernel``: one query token, head_dim 128, 4..8 kv heads, pages of at
least 16 tokens, every TMA box holding all kv heads of a token run; two boxes per tile on 16-token pages) on the GPU against the CPU oracle, through the
plugin front-end and the C ABI. The matrix is the decode part of the reference's op tests
(``op_test/sm90/test_attn_decode_fp8.py:219-365``) on the shapes this kernel takes; everything else stays on the
per-head kernel, which ``tests/test_attn_gpu.py`` covers.

Tolerance: bf16 output within atol 2e-2 + rtol 2e-2 of the oracle, LSE within 5e-3, empty rows exactly zero / -inf.
"""

import pytest
import torch

from greenattention_b200 import workloads as W
from tests.test_attn_gpu import check, compare, run

pytestmark = pytest.mark.gpu
FP8 = torch.float8_e4m3fn

KVH8_G8 = dict(q_heads=64, kv_heads=8, head_dim=128)  # the production shape
KVH8_G4 = dict(q_heads=32, kv_heads=8, head_dim=128)
KVH4_G8 = dict(q_heads=32, kv_heads=4, head_dim=128)
KVH6_G2 = dict(q_heads=12, kv_heads=6, head_dim=128)  # neither count a power of two
KVH5_G1 = dict(q_heads=5, kv_heads=5, head_dim=128)   # MHA, odd head count
LENS = [1, 2, 31, 32, 33, 63, 64, 65, 127, 1000, 4097]


@pytest.fixture(scope="module", autouse=True)
def _ready():
    from greenattention_b200 import attn_decode

    attn_decode.ensure_ready()
    yield
    assert attn_decode.workspace_status(torch.device("cuda", torch.cuda.current_device())) == 0


@pytest.mark.parametrize("inst", [KVH8_G8, KVH8_G4, KVH4_G8, KVH6_G2, KVH5_G1], ids=["kvh8g8", "kvh8g4", "kvh4g8", "kvh6g2", "kvh5g1"])
@pytest.mark.parametrize("page", [16, 32, 64, 128])
@pytest.mark.parametrize("q_dtype", [FP8, torch.bfloat16])
def test_ragged_lengths(inst, page, q_dtype):
    check(W.make_paged_case(LENS, [1] * len(LENS), page, q_dtype=q_dtype, seed=page + inst["kv_heads"], descale="rand", **inst))


@pytest.mark.parametrize("L", [1, 15, 16, 17, 31, 32, 33, 47, 48, 49, 4736, 65536])
def test_sixteen_token_pages_around_box_and_tile_ends(L):
    """Two 16-token boxes per 32-token tile; a sequence that ends inside the first box leaves the second one out, and
    the page-table row is padded with an id outside the pool right behind the last page in use."""
    kw = W.make_paged_case([L, 40, 3], [1, 1, 1], 16, seed=L % 97, extra_pages=8, descale="rand", **KVH8_G8)
    pt = kw["page_table"]
    used = -(-L // 16)
    if used < pt.shape[1]:
        pt[0, used:] = -1  # padding must never be looked at
    check(kw)
    check(W.make_paged_case([L, 5000], [1, 1], 16, seed=L % 89, window=(1023, 0), **KVH4_G8))


def test_empty_sequences_and_whole_batch_empty():
    check(W.make_paged_case([0, 17, 0, 300], [1, 1, 1, 1], 64, seed=6, **KVH8_G8))
    check(W.make_paged_case([0, 0, 0], [1, 1, 1], 64, seed=6, **KVH8_G8))  # zeros and -inf everywhere


@pytest.mark.parametrize("batch", [1, 2, 5])
def test_long_context_is_cut_into_many_slices(batch):
    """A few long requests: every CTA gets a slice of the same request and the combine kernel merges dozens of
    partials per kv head."""
    lens = [60000 - 7777 * i for i in range(batch)]
    check(W.make_paged_case(lens, [1] * batch, 64, seed=11, extra_pages=8, descale="rand", kv_std=0.5, **KVH8_G8))


@pytest.mark.parametrize("L", [31, 32, 33, 4736, 4737, 9472, 9473, 65536, 100003])
def test_slice_boundary_lengths(L):
    """Lengths around multiples of the tile (32 tokens) and of 148 tiles (one tile per CTA, two, ...)."""
    check(W.make_paged_case([L], [1], 32, seed=L % 97, extra_pages=8, **KVH4_G8))
    check(W.make_paged_case([L, 5, 40], [1, 1, 1], 64, seed=L % 89, extra_pages=8, **KVH8_G4))


def test_ragged_production_like_batch():
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(1, 9000, (48,), generator=g).tolist()
    lens[7], lens[20] = 0, 1
    check(W.make_paged_case(lens, [1] * 48, 64, seed=21, descale="rand", descale_range=(0.5, 2.0), kv_std=0.5, **KVH8_G8))


@pytest.mark.parametrize("L", [1, 2, 1023, 1024, 1025, 1056, 1057, 2048, 5000, 16384])
def test_window_edges(L):
    check(W.make_paged_case([L, 7, 3000], [1, 1, 1], 64, seed=L % 97, window=(1023, 0), **KVH8_G8))


def test_window_shorter_than_a_tile():
    check(W.make_paged_case([700, 33, 5000], [1, 1, 1], 32, seed=31, window=(9, 0), **KVH4_G8))
    check(W.make_paged_case([700, 33, 5000], [1, 1, 1], 64, seed=32, window=(0, 0), **KVH8_G4))  # only the key itself


@pytest.mark.parametrize("descale", ["none", "scalar", "rand"])
def test_descale_forms(descale):
    check(W.make_paged_case([500, 129, 2000], [1, 1, 1], 64, descale=descale, seed=8, **KVH8_G8))


def test_fp8_saturation_range():
    kw = W.make_paged_case([1500, 333, 64], [1, 1, 1], 64, kv_std=150.0, seed=9, **KVH8_G4)
    kw["k_descale"] = torch.full((3, 8), 1 / 150.0)
    kw["v_descale"] = torch.full((3, 8), 1 / 150.0)
    check(kw)


def test_peaked_softmax_short_rows():
    """Rows that rest on a handful of keys: the two-term e4m3 split of P must hold the tolerance."""
    kw = W.make_paged_case([3, 9, 40, 70], [1, 1, 1, 1], 32, seed=41, q_std=4.0, kv_std=2.0, **KVH8_G8)
    check(kw, lse_tol=1e-2)


@pytest.mark.parametrize("out_mode", ["given", "strided"])
def test_out_argument_and_strided_views(out_mode):
    check(W.make_paged_case([700, 129, 33], [1, 1, 1], 64, out_mode=out_mode, q_strided=True, kv_stack=True, seed=12, **KVH8_G8))


def test_no_lse():
    check(W.make_paged_case([700, 129], [1, 1], 64, return_lse=False, seed=15, **KVH8_G8))


def test_query_token_counts_other_than_one_keep_the_per_head_kernel():
    """Two query tokens x GQA 8 = 16 rows: not this kernel's shape, served by the 16-row per-head instance."""
    check(W.make_paged_case([700, 129, 33], [2, 2, 2], 64, seed=16, **KVH8_G8))
    check(W.make_paged_case([700, 129, 33], [2, 2, 2], 64, seed=17, **KVH8_G4))  # 8 rows from 2 tokens x GQA 4: wide


def test_deterministic():
    kw = W.case_to(W.make_paged_case([4000, 129, 900, 30000], [1] * 4, 64, seed=16, **KVH8_G8), "cuda")
    a, la = run(kw)
    b, lb = run(kw)
    assert torch.equal(a, b) and torch.equal(la, lb)


@pytest.mark.parametrize("batch", [1, 8, 32])
def test_cuda_graph_replay_with_changed_lengths(batch):
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    lens = [2048 + 37 * i for i in range(batch)]
    kw_cpu = W.make_paged_case(lens, [1] * batch, 64, seed=17 + batch, extra_pages=4, pt_pad=16, **KVH8_G8)
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


def test_fp32_partial_output_for_the_kv_sharded_path():
    """``decode_partial`` (normalised fp32 O + natural-log LSE, what a KV-range shard sends) also runs here."""
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    kw_cpu = W.make_paged_case([20000], [1], 64, seed=51, descale="rand", kv_std=0.5, **KVH8_G8)
    kw = W.case_to(kw_cpu, "cuda")
    o, lse = attn_decode.decode_partial(**kw)
    torch.cuda.synchronize()
    ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
    assert o.dtype == torch.float32
    assert ((o.cpu() - ref_o).abs() <= 2e-2 + 2e-2 * ref_o.abs()).all()
    assert (lse.cpu() - ref_lse).abs().max().item() <= 5e-3


def test_agrees_with_the_per_head_kernel_on_the_same_call(monkeypatch):
    """Two different gathers of the same bytes: the results agree far inside the tolerance (not bitwise: the tiles
    are 32 instead of 64 tokens, so the running max is updated at other points)."""
    from greenattention_b200 import attn_decode

    kw = W.case_to(W.make_paged_case([5000, 64, 33, 12000], [1] * 4, 64, seed=61, descale="rand", kv_std=0.5, **KVH8_G8), "cuda")
    wide, lse_w = run(kw)
    narrow, lse_n = attn_decode.decode_noalloc(**kw)  # the entry point without a workspace keeps the per-head kernel
    torch.cuda.synchronize()
    assert (wide.float() - narrow.float()).abs().max().item() <= 5e-3
    assert (lse_w - lse_n).abs().max().item() <= 1e-3
