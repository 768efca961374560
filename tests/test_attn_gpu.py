"""FP8 paged attention on the GPU, through the plugin front-end and the C ABI, against the CPU oracle and the
golden fixtures. The matrix follows the reference's op tests (``op_test/sm90/test_attn_decode_fp8.py:219-434``,
``op_test/sm90/test_attn_extend_fp8.py:36-138``) on the shapes this build serves (head_dim 128 / 256).

Tolerance (the stated parity bar): bf16 output within atol 2e-2 + rtol 2e-2 of the oracle, LSE within 5e-3
(1e-2 for the peaked case), finite/-inf LSE pattern identical, empty rows exactly zero.
"""

import os

import numpy as np
import pytest
import torch

from greenattention_b200 import workloads as W
from tests.golden import cases

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn
ATOL = RTOL = 2e-2
GOLD = os.path.join(os.path.dirname(__file__), "golden")

HD128 = dict(q_heads=8, kv_heads=2, head_dim=128)     # GQA 4
HD128_G8 = dict(q_heads=16, kv_heads=2, head_dim=128)  # GQA 8
HD256 = dict(q_heads=4, kv_heads=2, head_dim=256)     # GQA 2
HD256_G6 = dict(q_heads=12, kv_heads=2, head_dim=256)  # GQA 6: a group size that is not a power of two
LENS = [1, 2, 127, 128, 129, 255, 1000, 4097]


@pytest.fixture(scope="module", autouse=True)
def _ready():
    from greenattention_b200 import attn_decode

    attn_decode.ensure_ready()
    yield
    assert attn_decode.workspace_status(torch.device("cuda", torch.cuda.current_device())) == 0


def run(kw, select=None):
    from greenattention_b200 import attn_decode

    fn = (select or attn_decode.select)(kw)
    assert callable(fn), f"declined: {fn}"
    return fn(**kw)


def compare(out, lse, ref_o, ref_lse, lse_tol=5e-3):
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == tuple(ref_o.shape)
    o = out.float().cpu()
    assert not torch.isnan(o).any()
    err = (o - ref_o).abs()
    bound = ATOL + RTOL * ref_o.abs()
    worst = (err - bound).max().item()
    assert worst <= 0, f"out exceeds atol/rtol by {worst}, max abs err {err.max().item()}"
    if lse is not None:
        l = lse.cpu()
        assert l.shape == ref_lse.shape and l.dtype == torch.float32
        fin = torch.isfinite(ref_lse)
        assert torch.equal(torch.isfinite(l), fin)
        assert torch.equal(l[~fin], ref_lse[~fin])
        if fin.any():
            lerr = (l[fin] - ref_lse[fin]).abs().max().item()
            assert lerr <= lse_tol, f"lse err {lerr}"
        dead_rows = (~fin).T  # [total_q, QH]
        assert o[dead_rows].abs().max().item() == 0.0 if dead_rows.any() else True
    return err.max().item()


def check(kw_cpu, select=None, lse_tol=5e-3):
    from oracle import attn_oracle

    kw = W.case_to(kw_cpu, "cuda")
    res = run(kw, select)
    out, lse = res if kw["return_softmax_lse"] else (res, None)
    if "out" in kw:
        assert out.data_ptr() == kw["out"].data_ptr(), "out= not honoured"
    ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
    return compare(out, lse, ref_o, ref_lse, lse_tol)


def check_extend(kw_cpu, **opts):
    from greenattention_b200 import attn_decode

    return check(kw_cpu, select=attn_decode.select_extend, **opts)


# ------------------------------------------------------------------ golden fixtures (reference's own oracle output)


@pytest.mark.parametrize("name", sorted(cases.ATTN_CASES))
def test_golden_fixture(name):
    from greenattention_b200 import attn_decode

    kw_cpu = cases.ATTN_CASES[name]()
    gold = np.load(os.path.join(GOLD, f"attn_{name}.npz"))
    kw = W.case_to(kw_cpu, "cuda")
    sel = attn_decode.select if kw["max_seqlen_q"] * (kw["q"].shape[1] // kw["k_cache"].shape[2]) <= 128 and \
        kw["max_seqlen_q"] <= 16 else attn_decode.select_extend
    out, lse = run(kw, sel)
    compare(out, lse, torch.from_numpy(gold["out"]), torch.from_numpy(gold["lse"]),
            lse_tol=1e-2 if name == "peaked" else 5e-3)


@pytest.mark.parametrize("name", ["c1", "verify_ragged", "window_hd256", "empty_rows"])
def test_golden_fixture_through_extend_kernel(name):
    from greenattention_b200 import attn_decode

    kw_cpu = cases.ATTN_CASES[name]()
    gold = np.load(os.path.join(GOLD, f"attn_{name}.npz"))
    out, lse = run(W.case_to(kw_cpu, "cuda"), attn_decode.select_extend)
    compare(out, lse, torch.from_numpy(gold["out"]), torch.from_numpy(gold["lse"]))


# ------------------------------------------------------------------ decode / verify matrix


@pytest.mark.parametrize("page", [1, 16, 64])
@pytest.mark.parametrize("qlen", [1, 2, 4, 7, 10])
@pytest.mark.parametrize("q_dtype", [FP8, torch.bfloat16])
def test_ragged_lengths(page, qlen, q_dtype):
    lens = [max(L, qlen) for L in LENS]
    check(W.make_paged_case(lens, [qlen] * len(lens), page, q_dtype=q_dtype, seed=page + qlen, descale="rand", **HD128))


@pytest.mark.parametrize("page", [1, 16, 128])
@pytest.mark.parametrize("qlen", [1, 5, 16])
def test_ragged_lengths_hd256(page, qlen):
    lens = [max(L, qlen) for L in LENS]
    check(W.make_paged_case(lens, [qlen] * len(lens), page, seed=7 * page + qlen, descale="rand", **HD256))


@pytest.mark.parametrize("qlen", [1, 2, 5, 16])
def test_gqa8_rows(qlen):
    lens = [max(L, qlen) for L in LENS]
    check(W.make_paged_case(lens, [qlen] * len(lens), 64, seed=50 + qlen, descale="rand", **HD128_G8))


@pytest.mark.parametrize("qlen", [1, 2, 3, 5, 16])
def test_gqa6_hd256_rows(qlen):
    """head_dim 256 with 6 query heads per kv head, one of the reference's instance shapes
    (``green_attention/attn_decode.py:58-68``): rows per kv head 6 .. 96, over every row-count instance."""
    lens = [max(L, qlen) for L in LENS]
    check(W.make_paged_case(lens, [qlen] * len(lens), 64, seed=80 + qlen, descale="rand", **HD256_G6))


def test_gqa6_hd256_extend():
    """128 rows do not divide by 6: a query block is 21 tokens x 6 heads, two rows of the tile stay empty."""
    lens = [700, 129, 2048, 33, 21, 22]
    qlens = [700, 64, 333, 5, 21, 22]
    check_extend(W.make_paged_case(lens, qlens, 64, seed=86, descale="rand", **HD256_G6))
    check_extend(W.make_paged_case(lens, qlens, 16, seed=87, window=(1023, 0), **HD256_G6))


@pytest.mark.parametrize("page", [1, 16])
def test_ragged_query_lengths(page):
    check(W.make_paged_case([5, 300, 129, 40, 2048, 12, 700, 10], [1, 4, 2, 10, 3, 1, 6, 4], page, seed=3,
                            descale="rand", **HD128))


@pytest.mark.parametrize("batch", [1, 2, 5])
@pytest.mark.parametrize("qlen", [1, 4])
def test_long_context_split_kv(batch, qlen):
    lens = [20000 - 777 * i for i in range(batch)]
    check(W.make_paged_case(lens, [qlen] * batch, 16, seed=11, extra_pages=8, descale="rand", **HD128))


def test_empty_sequence():
    check(W.make_paged_case([0, 17, 0, 300], [1, 1, 1, 1], 16, seed=6, **HD128))
    check(W.make_paged_case([0, 0], [4, 4], 16, seed=6, **HD128))  # all rows empty: zeros and -inf


@pytest.mark.parametrize("qlen", [1, 4])
def test_dynamic_splits_ragged_batch(qlen):
    lens = [40000, 3, 256, 257, 1024, 9000, 128 * 7 + 5, 16384]
    check(W.make_paged_case(lens, [qlen] * len(lens), 16, seed=40 + qlen, extra_pages=8, **HD128))


@pytest.mark.parametrize("L", [255, 256, 257, 511, 512, 513, 2048, 2049, 65536, 100003])
def test_dynamic_splits_boundary_lengths(L):
    check(W.make_paged_case([L], [1], 16, seed=L % 97, extra_pages=8, **HD128))
    check(W.make_paged_case([L, 5], [4, 4], 16, seed=L % 89, extra_pages=8, **HD128))


@pytest.mark.parametrize("descale", ["none", "scalar", "rand"])
def test_descale_forms(descale):
    check(W.make_paged_case([500, 129, 2000], [4, 4, 4], 16, descale=descale, seed=8, **HD128))


@pytest.mark.parametrize("inst", [HD128, HD256])
def test_fp8_saturation_range(inst):
    kw = W.make_paged_case([1500, 333, 64], [1, 1, 1], 16, kv_std=150.0, seed=9, **inst)
    kw["k_descale"] = torch.full((3, 2), 1 / 150.0)
    kw["v_descale"] = torch.full((3, 2), 1 / 150.0)
    check(kw)


def test_peaked_softmax():
    check(cases.ATTN_CASES["peaked"](), lse_tol=1e-2)


@pytest.mark.parametrize("out_mode", ["given", "strided"])
def test_out_argument(out_mode):
    check(W.make_paged_case([700, 129, 33], [4, 4, 4], 16, out_mode=out_mode, seed=12, **HD128))


def test_strided_q_and_stacked_kv():
    check(W.make_paged_case([700, 129, 33], [1, 1, 1], 16, q_strided=True, kv_stack=True, seed=13, **HD128))
    check(W.make_paged_case([700, 129, 33], [4, 4, 4], 1, q_strided=True, kv_stack=True, seed=14, **HD128))


def test_no_lse():
    check(W.make_paged_case([700, 129], [4, 4], 16, return_lse=False, seed=15, **HD128))


def test_deterministic():
    kw = W.case_to(W.make_paged_case([4000, 129, 900, 30000], [4, 4, 4, 4], 16, seed=16, **HD128), "cuda")
    a, la = run(kw)
    b, lb = run(kw)
    assert torch.equal(a, b) and torch.equal(la, lb)


@pytest.mark.parametrize("batch", [1, 8, 32])
@pytest.mark.parametrize("qlen", [1, 4])
def test_cuda_graph_capture_replay(batch, qlen):
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    lens = [2048 + 37 * i for i in range(batch)]
    kw_cpu = W.make_paged_case(lens, [qlen] * batch, 16, seed=17 + batch, extra_pages=4, pt_pad=64, **HD128)
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
        new_lens = [max(qlen, L - shrink - 3 * i) for i, L in enumerate(lens)]
        kw["cache_seqlens"].copy_(torch.tensor(new_lens, dtype=torch.int32))
        kw_cpu["cache_seqlens"] = torch.tensor(new_lens, dtype=torch.int32)
        graph.replay()
        torch.cuda.synchronize()
        ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
        compare(static_out[0], static_out[1], ref_o, ref_lse)


def test_graph_replay_changing_split_plan():
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    batch, qlen = 4, 4
    kw_cpu = W.make_paged_case([30000] * batch, [qlen] * batch, 16, seed=44, extra_pages=4, pt_pad=16, **HD128)
    kw = W.case_to(kw_cpu, "cuda")
    fn = attn_decode.select(kw)
    fn(**kw)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            static_out = fn(**kw)
    for new_lens in ([30000, 20000, 9000, 5000], [qlen, 10, 700, 30000], [0, 0, 0, 0], [12345, 4, 4, 29999]):
        kw["cache_seqlens"].copy_(torch.tensor(new_lens, dtype=torch.int32))
        kw_cpu["cache_seqlens"] = torch.tensor(new_lens, dtype=torch.int32)
        graph.replay()
        torch.cuda.synchronize()
        ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
        compare(static_out[0], static_out[1], ref_o, ref_lse)


@pytest.mark.parametrize("inst,qlen", [(HD128, 5), (HD256, 16), (HD128_G8, 3)])
def test_verify_large_batch(inst, qlen):
    # enough (request, kv head) pairs to fill every SM: verify then runs one tcgen05 CTA per pair
    g = torch.Generator().manual_seed(qlen)
    lens = torch.randint(qlen, 700, (96,), generator=g).tolist()
    lens[3], lens[40] = qlen, 0
    check(W.make_paged_case(lens, [qlen] * 96, 64, seed=70 + qlen, descale="rand", kv_std=0.5, **inst))
    check(W.make_paged_case(lens, [qlen] * 96, 16, seed=71 + qlen, window=(127, 0), **inst))


# ------------------------------------------------------------------ sliding window


@pytest.mark.parametrize("L", [1, 2, 1023, 1024, 1025, 1026, 1027, 1152, 2048, 5000, 16384])
def test_window_edges(L):
    check(W.make_paged_case([L], [1], 16, seed=L % 97, window=(1023, 0), **HD256))
    check(W.make_paged_case([L, 7], [4, 4], 16, seed=L % 89 + 1, window=(1023, 0), **HD256))


def test_window_qlen_row_bounds():
    lens = [3000, 4096, 4097]
    check(W.make_paged_case(lens, [16] * 3, 16, seed=61, window=(1023, 0), **HD256))
    check(W.make_paged_case(lens, [2, 5, 16], 64, seed=62, window=(1023, 0), **HD256))


@pytest.mark.parametrize("batch", [1, 3])
def test_window_split_kv(batch):
    lens = [20000 - 777 * i for i in range(batch)]
    check(W.make_paged_case(lens, [4] * batch, 16, seed=71 + batch, extra_pages=8, window=(1023, 0), **HD256))


# ------------------------------------------------------------------ extend


@pytest.mark.parametrize("page", [1, 16, 64])
@pytest.mark.parametrize("q_dtype", [FP8, torch.bfloat16])
def test_extend_prefix_and_ragged(page, q_dtype):
    lens = [700, 129, 2048, 33, 32, 1, 300]
    qlens = [700, 64, 333, 5, 32, 1, 299]
    check_extend(W.make_paged_case(lens, qlens, page, q_dtype=q_dtype, seed=page, descale="rand", **HD128))


@pytest.mark.parametrize("qlen", [31, 32, 33, 63, 64, 65, 127, 128, 129])
def test_extend_query_block_boundaries(qlen):
    lens = [qlen + p for p in (0, 3, 130, 1000)]
    check_extend(W.make_paged_case(lens, [qlen] * len(lens), 16, seed=qlen, **HD256))


def test_extend_empty_queries_and_sequences():
    check_extend(W.make_paged_case([300, 0, 50, 17], [5, 0, 50, 0], 16, seed=3, **HD128))


def test_extend_long_prefill_and_window():
    check_extend(W.make_paged_case([4500, 37], [3000, 37], 64, seed=4, extra_pages=4, kv_std=0.5, **HD256))
    check_extend(W.make_paged_case([4500, 37], [3000, 37], 64, seed=5, extra_pages=4, window=(1023, 0), **HD256))


@pytest.mark.parametrize("out_mode", ["none", "given", "strided"])
@pytest.mark.parametrize("ret_lse", [True, False])
def test_extend_out_and_lse(out_mode, ret_lse):
    check_extend(W.make_paged_case([700, 129, 33], [300, 129, 9], 16, out_mode=out_mode, return_lse=ret_lse, seed=6,
                                   **HD128))


def test_extend_graph_replay_over_different_query_splits():
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    batch, total = 4, 256
    kw_cpu = W.make_paged_case([3000] * batch, [total // batch] * batch, 16, seed=10, extra_pages=4, pt_pad=8, **HD128)
    kw = W.case_to(kw_cpu, "cuda")
    fn = attn_decode.select_extend(kw)
    assert callable(fn)
    fn(**kw)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            static_out = fn(**kw)
    for qlens, new_lens in (
        ([64, 64, 64, 64], [3000, 900, 64, 2000]),
        ([1, 250, 3, 2], [1, 2999, 3, 1000]),
        ([0, 0, 256, 0], [0, 7, 256, 0]),
        ([31, 33, 64, 128], [31, 700, 64, 3000]),
    ):
        cu = torch.zeros(batch + 1, dtype=torch.int32)
        cu[1:] = torch.tensor(qlens, dtype=torch.int32).cumsum(0)
        kw["cu_seqlens_q"].copy_(cu)
        kw["cache_seqlens"].copy_(torch.tensor(new_lens, dtype=torch.int32))
        kw_cpu["cu_seqlens_q"], kw_cpu["cache_seqlens"] = cu, torch.tensor(new_lens, dtype=torch.int32)
        graph.replay()
        torch.cuda.synchronize()
        ref_o, ref_lse = attn_oracle.paged_attention(kw_cpu)
        compare(static_out[0], static_out[1], ref_o, ref_lse)


# ------------------------------------------------------------------ routing and declines on real tensors


def test_dispatch_routes_by_query_length():
    from greenattention_b200 import dispatch
    from oracle import attn_oracle

    def stock(**kw):
        raise AssertionError("went to the stock kernel")

    wrapped = dispatch.with_kvcache(stock)
    for qlen in (1, 5, 40):
        kw_cpu = W.make_paged_case([400, 2 * qlen + 1], [qlen, qlen], 16, seed=13, return_lse=False, **HD128)
        out = wrapped(**W.case_to(kw_cpu, "cuda"))
        ref_o, _ = attn_oracle.paged_attention(kw_cpu)
        compare(out, None, ref_o, None)


@pytest.mark.parametrize(
    "mutate,needle",
    [
        (lambda kw: kw.update(softcap=30.0), "softcap"),
        (lambda kw: kw.update(window_size=(128, 5)), "window"),
        (lambda kw: kw.update(sinks=torch.zeros(8, device="cuda")), "sinks"),
        (lambda kw: kw.update(max_seqlen_q=17), "max_seqlen_q"),
        (lambda kw: kw.update(causal=False, max_seqlen_q=4), "non-causal"),
        (lambda kw: kw.update(k_cache=kw["k_cache"].to(torch.bfloat16), v_cache=kw["v_cache"].to(torch.bfloat16)), "e4m3"),
        (lambda kw: kw.update(q=kw["q"][:, :3]), "q shape"),
        (lambda kw: kw.update(cu_seqlens_q=None), "paged"),
        (lambda kw: kw.update(k_cache=kw["k_cache"][:, :12], v_cache=kw["v_cache"][:, :12]), "power of two"),
    ],
)
def test_declines_out_of_scope(mutate, needle):
    from greenattention_b200 import attn_decode

    kw = W.case_to(W.make_paged_case([300, 40], [4, 4], 16, seed=20, **HD128), "cuda")
    mutate(kw)
    why = attn_decode.select(kw)
    assert isinstance(why, str) and needle in why, why


def test_ganged_verify_route_in_a_fresh_process():
    """``GREEN_ATTN_GANG=1`` (read once per process) makes the tcgen05 verify route run in gangs of kv_heads CTAs on
    slices of whole requests; the combine kernel then looks the partial slots up by (gang, kv head). Same bar."""
    import subprocess
    import sys

    code = (
        "import torch, sys; sys.path.insert(0, '.');"
        "from greenattention_b200 import attn_decode, workloads as W;"
        "from oracle import attn_oracle;"
        "attn_decode.ensure_ready();"
        "cases=[W.make_paged_case([9000, 300, 5, 40000, 0, 777], [5]*6, 64, q_heads=16, kv_heads=4, head_dim=128, seed=5, descale='rand', kv_std=0.5),"
        " W.make_paged_case([3000]*40, [16]*40, 64, q_heads=16, kv_heads=2, head_dim=256, seed=6, window=(511, 0))];\n"
        "for c in cases:\n"
        "    kw = W.case_to(c, 'cuda'); out, lse = attn_decode.select(kw)(**kw); torch.cuda.synchronize()\n"
        "    ref, ref_lse = attn_oracle.paged_attention(c)\n"
        "    assert ((out.float().cpu() - ref).abs() <= 2e-2 + 2e-2 * ref.abs()).all()\n"
        "    fin = torch.isfinite(ref_lse); assert (lse.cpu()[fin] - ref_lse[fin]).abs().max() <= 5e-3\n"
        "assert attn_decode.workspace_status(torch.device('cuda', 0)) == 0; print('ganged ok')"
    )
    env = dict(os.environ, GREEN_ATTN_GANG="1")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "ganged ok" in res.stdout, res.stderr[-2000:]


def test_warp_level_route_of_the_shapes_the_tcgen05_kernel_takes_by_default():
    """``GREEN_ATTN_TC_MIN_ROWS_128 / _256 = 17`` (read once per process) keep head_dim 256 decode and 9 - 16 rows at
    head_dim 128 on the warp-level instances: still product code (it is what pools with tiny pages, unaligned rows and
    the no-workspace entry point run for these shapes). Same bar."""
    import subprocess
    import sys

    code = (
        "import torch, sys; sys.path.insert(0, '.');"
        "from greenattention_b200 import attn_decode, workloads as W;"
        "from oracle import attn_oracle;"
        "attn_decode.ensure_ready();"
        "cases=[W.make_paged_case([9000, 300, 5, 40000, 0, 777], [1]*6, 64, q_heads=12, kv_heads=2, head_dim=256, seed=7, descale='rand', kv_std=0.5),"
        " W.make_paged_case([3000, 64, 12000], [2]*3, 64, q_heads=16, kv_heads=2, head_dim=128, seed=8, window=(511, 0)),"
        " W.make_paged_case([700, 129, 5000], [3]*3, 16, q_heads=8, kv_heads=2, head_dim=256, seed=9)];\n"
        "for c in cases:\n"
        "    kw = W.case_to(c, 'cuda'); out, lse = attn_decode.select(kw)(**kw); torch.cuda.synchronize()\n"
        "    ref, ref_lse = attn_oracle.paged_attention(c)\n"
        "    assert ((out.float().cpu() - ref).abs() <= 2e-2 + 2e-2 * ref.abs()).all()\n"
        "    fin = torch.isfinite(ref_lse); assert (lse.cpu()[fin] - ref_lse[fin]).abs().max() <= 5e-3\n"
        "assert attn_decode.workspace_status(torch.device('cuda', 0)) == 0; print('warp-level ok')"
    )
    env = dict(os.environ, GREEN_ATTN_TC_MIN_ROWS_128="17", GREEN_ATTN_TC_MIN_ROWS_256="17")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, "-c", code], cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "warp-level ok" in res.stdout, res.stderr[-2000:]
