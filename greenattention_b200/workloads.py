"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference measures on no public dataset: its tests and benches draw seeded random paged caches
(``op_test/sm90/test_attn_decode_fp8.py:40-102``, ``op_test/sm90/gdn_common.py:30-151``). These
builders produce the same kind of input (random page permutation with pages no request owns,
padded page-table rows, e4m3 K/V, per-(request, kv head) descales, strided variants) for the five
named configurations, on any device, from a ``torch.Generator`` seeded by the caller.
"""

from __future__ import annotations

import math

import torch

FP8 = torch.float8_e4m3fn


def _gen(seed: int, device) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(int(seed))
    return g


def _e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-448.0, 448.0).to(FP8)


def _fill_e4m3(dst: torch.Tensor, std: float, gen, chunk_pages: int = 4096) -> None:
    """Fill an e4m3 pool page-chunk by page-chunk so a multi-GB pool never needs an fp32 twin."""
    n = dst.shape[0]
    for p0 in range(0, n, chunk_pages):
        p1 = min(n, p0 + chunk_pages)
        blk = torch.randn((p1 - p0,) + tuple(dst.shape[1:]), generator=gen, device=dst.device) * std
        dst[p0:p1] = _e4m3(blk)


def make_paged_case(
    lens, qlens, page, *, q_heads, kv_heads, head_dim, seed=0, device="cpu", q_dtype=torch.bfloat16,
    kv_std=1.0, q_std=1.0, descale="none", descale_range=(0.5, 1.0), window=(-1, -1), kv_stack=False,
    q_strided=False, out_mode="none", extra_pages=2, pt_pad=1, return_lse=True, softmax_scale=None,
):
    """A random paged FP8 cache plus queries, as keyword arguments of ``flash_attn_with_kvcache``.

    ``descale``: "none" | "scalar" (one value expanded with strides (0, 0)) | "rand" (per request
    and kv head, uniform in ``descale_range``). ``kv_stack``: K and V are interleaved views of one
    pool. ``q_strided`` / ``out_mode="strided"``: last-dim-contiguous views of wider buffers.
    """
    dev = torch.device(device)
    g = _gen(seed, dev)
    B = len(lens)
    pages_per = [max(1, -(-int(L) // page)) for L in lens]
    n_pages = sum(pages_per) + extra_pages
    perm = torch.randperm(n_pages, generator=g, device=dev).to(torch.int32)
    max_p = max(pages_per) + pt_pad
    pt = torch.zeros((B, max_p), dtype=torch.int32, device=dev)
    pos = 0
    for b, npg in enumerate(pages_per):
        pt[b, :npg] = perm[pos:pos + npg]
        pos += npg
    shape = (n_pages, page, kv_heads, head_dim)
    if kv_stack:
        buf = torch.empty((n_pages, 2, page, kv_heads, head_dim), dtype=FP8, device=dev)
        kc, vc = buf[:, 0], buf[:, 1]
    else:
        kc = torch.empty(shape, dtype=FP8, device=dev)
        vc = torch.empty(shape, dtype=FP8, device=dev)
    _fill_e4m3(kc, kv_std, g)
    _fill_e4m3(vc, kv_std, g)
    lo, hi = descale_range
    if descale == "rand":
        kd = (torch.rand((B, kv_heads), generator=g, device=dev) * (hi - lo) + lo).float()
        vd = (torch.rand((B, kv_heads), generator=g, device=dev) * (hi - lo) + lo).float()
    elif descale == "scalar":
        kd = torch.tensor([0.37], device=dev).expand(B, kv_heads)
        vd = torch.tensor([0.61], device=dev).expand(B, kv_heads)
    else:
        kd = vd = None
    total_q = int(sum(qlens))
    qf = torch.randn((total_q, q_heads, head_dim), generator=g, device=dev) * q_std
    qv = _e4m3(qf) if q_dtype == FP8 else qf.to(q_dtype)
    if q_strided:
        qbuf = torch.zeros((total_q, q_heads, 2 * head_dim), dtype=q_dtype, device=dev)
        qbuf[..., :head_dim] = qv
        q = qbuf[..., :head_dim]
    else:
        q = qv
    cu = torch.zeros(B + 1, dtype=torch.int32, device=dev)
    cu[1:] = torch.tensor(list(qlens), dtype=torch.int32, device=dev).cumsum(0)
    kw = dict(
        q=q, k_cache=kc, v_cache=vc, page_table=pt,
        cache_seqlens=torch.tensor(list(lens), dtype=torch.int32, device=dev),
        cu_seqlens_q=cu, max_seqlen_q=int(max(qlens)) if len(qlens) else 0,
        softmax_scale=head_dim**-0.5 if softmax_scale is None else softmax_scale, causal=True,
        window_size=tuple(window), softcap=0.0, return_softmax_lse=return_lse, num_splits=0,
    )
    if kd is not None:
        kw["k_descale"], kw["v_descale"] = kd, vd
    if out_mode == "given":
        kw["out"] = torch.full((total_q, q_heads, head_dim), float("nan"), dtype=torch.bfloat16, device=dev)
    elif out_mode == "strided":
        ob = torch.full((total_q, q_heads, 2 * head_dim), float("nan"), dtype=torch.bfloat16, device=dev)
        kw["out"] = ob[..., :head_dim]
    return kw


def case_to(kw: dict, device) -> dict:
    """Copy every tensor of a case to ``device`` keeping strides of strided views (K/V stacking)."""
    out = {}
    kc, vc = kw.get("k_cache"), kw.get("v_cache")
    stacked = (
        kc is not None and vc is not None and kc.untyped_storage().data_ptr() == vc.untyped_storage().data_ptr()
    )
    for name, val in kw.items():
        if not isinstance(val, torch.Tensor):
            out[name] = val
        elif stacked and name in ("k_cache", "v_cache"):
            continue
        elif val.dim() >= 1 and val.stride(-1) == 1 and not val.is_contiguous() and 0 not in val.stride():
            wide = torch.empty_strided(val.shape, val.stride(), dtype=val.dtype, device=device)
            wide.copy_(val)
            out[name] = wide
        elif 0 in val.stride():
            base = val.flatten()[:1].clone().to(device)
            out[name] = base.expand(val.shape)
        else:
            out[name] = val.to(device)
    if stacked:
        n_pages, page, kvh, hd = kc.shape
        buf = torch.empty((n_pages, 2, page, kvh, hd), dtype=kc.dtype, device=device)
        buf[:, 0].copy_(kc)
        buf[:, 1].copy_(vc)
        out["k_cache"], out["v_cache"] = buf[:, 0], buf[:, 1]
    return out


def extract_requests(kw: dict, requests, device="cpu") -> dict:
    """The sub-call that holds only ``requests`` (indices into the batch) of a paged call, on ``device``, with a
    compacted page pool: the pages those requests own are gathered in page-table order and renumbered 0, 1, ...,
    so a multi-GB pool resident on a GPU can be checked request by request on the host without copying all of
    it. Token order, page contents, queries and descales are untouched, so attention over the sub-call equals
    rows ``cu[r]:cu[r+1]`` of attention over the whole call."""
    kc, vc, pt = kw["k_cache"], kw["v_cache"], kw["page_table"]
    page = kc.shape[1]
    lens = kw["cache_seqlens"].tolist()
    cu = kw["cu_seqlens_q"].tolist()
    requests = [int(r) for r in requests]
    ids, rows_q, new_pt_rows, qlens = [], [], [], []
    n_new = 0
    for r in requests:
        npg = max(1, -(-int(lens[r]) // page))
        ids.append(pt[r, :npg].long())
        new_pt_rows.append(torch.arange(n_new, n_new + npg, dtype=torch.int32))
        n_new += npg
        rows_q.append(torch.arange(cu[r], cu[r + 1]))
        qlens.append(cu[r + 1] - cu[r])
    ids = torch.cat(ids).to(kc.device)
    max_p = max(t.numel() for t in new_pt_rows) + 1
    new_pt = torch.zeros((len(requests), max_p), dtype=torch.int32)
    for i, t in enumerate(new_pt_rows):
        new_pt[i, : t.numel()] = t
    rows_q = torch.cat(rows_q) if rows_q else torch.zeros(0, dtype=torch.long)
    new_cu = torch.zeros(len(requests) + 1, dtype=torch.int32)
    new_cu[1:] = torch.tensor(qlens, dtype=torch.int32).cumsum(0)
    sub = {k: v for k, v in kw.items() if not isinstance(v, torch.Tensor)}
    sub.update(
        q=kw["q"][rows_q.to(kw["q"].device)].to(device),
        k_cache=kc[ids].to(device), v_cache=vc[ids].to(device),
        page_table=new_pt.to(device),
        cache_seqlens=torch.tensor([int(lens[r]) for r in requests], dtype=torch.int32, device=device),
        cu_seqlens_q=new_cu.to(device), max_seqlen_q=int(max(qlens)) if qlens else 0,
    )
    for name in ("k_descale", "v_descale"):
        t = kw.get(name)
        if t is not None:
            sub[name] = (t[torch.tensor(requests, device=t.device)] if t.shape[0] > 1 else t).to(device).contiguous()
    sub.pop("out", None)
    return sub


def request_rows(kw: dict, requests) -> torch.Tensor:
    """Row indices (dim 0 of q / out) of ``requests``, in the order ``extract_requests`` lays them out."""
    cu = kw["cu_seqlens_q"].tolist()
    return torch.cat([torch.arange(cu[int(r)], cu[int(r) + 1]) for r in requests])


# ------------------------------------------------------------------ the named configurations


def c1_cpu_decode(device="cpu", seed=1):
    """Batch 4, 8 query / 2 kv heads, head_dim 128, contexts [137, 512, 64, 300], page 16, 256-page pool."""
    lens = [137, 512, 64, 300]
    used = sum(-(-L // 16) for L in lens)
    return make_paged_case(
        lens, [1] * 4, 16, q_heads=8, kv_heads=2, head_dim=128, seed=seed, device=device,
        kv_std=1.0, descale="none", extra_pages=256 - used,
    )


def c2_production_decode(device="cuda", seed=2, batch=128, ctx_lo=1024, ctx_hi=32768, lens=None):
    """Batch 128, 64 query / 8 kv heads, head_dim 128, page 64, contexts uniform in [1k, 32k],
    K/V N(0, 0.5) in e4m3 with descales U(0.5, 2)."""
    if lens is None:
        g = _gen(seed, "cpu")
        lens = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g).tolist()
    return make_paged_case(
        lens, [1] * len(lens), 64, q_heads=64, kv_heads=8, head_dim=128, seed=seed, device=device,
        kv_std=0.5, descale="rand", descale_range=(0.5, 2.0), extra_pages=8, return_lse=False,
    )


def c3_spec_verify(device="cuda", seed=3, batch=64, prefix=8192, q_len=5):
    """Batch 64, 5 query tokens (1 accepted + 4 draft, causal inside the chain), 32 query / 8 kv heads,
    head_dim 128, page 64; the 5 new tokens are already in the cache so ``cache_seqlens = prefix + 5``."""
    return make_paged_case(
        [prefix + q_len] * batch, [q_len] * batch, 64, q_heads=32, kv_heads=8, head_dim=128, seed=seed,
        device=device, kv_std=0.5, descale="none", extra_pages=8, return_lse=False,
    )


def c4_extend(device="cuda", seed=4, batch=8, prefix=16384, q_len=2048, window=None):
    """Batch 8, 2048 new tokens on a 16k cached prefix, 16 query / 8 kv heads, head_dim 256, page 64;
    ``window`` None = full attention, 1024 = sliding layer (passed as ``window_size=(1023, 0)``)."""
    ws = (-1, -1) if window is None else (int(window) - 1, 0)
    return make_paged_case(
        [prefix + q_len] * batch, [q_len] * batch, 64, q_heads=16, kv_heads=8, head_dim=256, seed=seed,
        device=device, kv_std=0.5, descale="none", extra_pages=8, return_lse=False, window=ws,
    )


def make_gdn_case(
    batch, tokens, *, h=16, hv=32, k=128, v=128, slots=None, seed=5, device="cpu", state_std=0.02,
    state_dtype=torch.float32, pad_rows=(), accept="rand", normalise_qk=True, gate_params="zero",
):
    """Inputs of one speculative GDN step: ``tokens`` chained draft tokens per request.

    q, k ``[B, T, H, K]`` bf16 (L2-normalised when ``normalise_qk``), v ``[B, T, HV, V]`` bf16 N(0,1),
    raw gates a, b ``[B, T, HV]`` bf16 N(0,1). ``gate_params="zero"`` sets ``A_log = dt_bias = 0`` so that
    ``g = -softplus(a)`` and ``beta = sigmoid(b)``; "rand" draws them like the reference's tests
    (``op_test/sm90/gdn_common.py:47-48``). ``accept``: "rand" (uniform 0..T) | "all" | a list.
    """
    dev = torch.device(device)
    g = _gen(seed, dev)
    B, T = batch, tokens
    slots = B + 8 if slots is None else slots
    q = torch.randn((B, T, h, k), generator=g, device=dev)
    kk = torch.randn((B, T, h, k), generator=g, device=dev)
    if normalise_qk:
        q = q / q.norm(dim=-1, keepdim=True)
        kk = kk / kk.norm(dim=-1, keepdim=True)
    vv = torch.randn((B, T, hv, v), generator=g, device=dev)
    a = torch.randn((B, T, hv), generator=g, device=dev)
    b = torch.randn((B, T, hv), generator=g, device=dev)
    if gate_params == "zero":
        A_log = torch.zeros(hv, device=dev)
        dt_bias = torch.zeros(hv, device=dev)
    else:
        A_log = torch.log(torch.rand(hv, generator=g, device=dev) * 16 + 1e-3)
        dt_bias = torch.randn(hv, generator=g, device=dev)
    state = (torch.randn((slots, hv, v, k), generator=g, device=dev) * state_std).to(state_dtype)
    idx = torch.randperm(slots, generator=g, device=dev)[:B].to(torch.int32)
    for r in pad_rows:
        idx[r] = -1
    if accept == "rand":
        acc = torch.randint(0, T + 1, (B,), generator=g, device=dev, dtype=torch.int32)
    elif accept == "all":
        acc = torch.full((B,), T, dtype=torch.int32, device=dev)
    else:
        acc = torch.tensor(list(accept), dtype=torch.int32, device=dev)
    return dict(
        q=q.to(torch.bfloat16), k=kk.to(torch.bfloat16), v=vv.to(torch.bfloat16),
        a=a.to(torch.bfloat16), b=b.to(torch.bfloat16), A_log=A_log.float(), dt_bias=dt_bias.float(),
        ssm_states=state, cache_indices=idx, accept_lens=acc, scale=k**-0.5,
    )


def make_gdn_replay_case(
    spec_lens, *, h=16, hv=32, ring_len=32, write_pos=None, cache_base=None, pad_rows=(), flush_rows=(), seed=6,
    device="cpu", state_dtype=torch.float32, state_std=0.02, flat=False, idx_dtype=torch.int32,
):
    """Keyword arguments of one Replay-SSM verify call (``gdn_replayssm_spec_decode``, ``launch_mode="verify"``;
    layouts of ``docs/gdn-contract.md:83-95`` in the reference): ``spec_lens[n]`` in 0..4 draft tokens per request,
    ring slot n for request n with ``write_pos[n]`` committed entries starting at physical position
    ``cache_base[n]`` (random when None), history deltas N(0, 0.05), history keys L2-normalised, history gates in
    (-1, 0). ``flat``: q/k/v/out given as ``[T, heads * dim]``."""
    dev = torch.device(device)
    g = _gen(seed, dev)
    B, T, L = len(spec_lens), int(sum(spec_lens)), ring_len
    k, v = 128, 128
    ring = B
    qsl = torch.tensor([0] + list(torch.tensor(list(spec_lens)).cumsum(0).tolist()), dtype=torch.int32, device=dev)

    def unit(*shape):
        x = torch.randn(shape, generator=g, device=dev)
        return x / x.norm(dim=-1, keepdim=True)

    wp = torch.randint(0, L + 1, (ring + 1,), generator=g, device=dev) if write_pos is None else \
        torch.tensor(list(write_pos) + [0], device=dev)
    cb = torch.randint(0, L, (ring + 1,), generator=g, device=dev) if cache_base is None else \
        torch.tensor(list(cache_base) + [0], device=dev)
    slots = B + 4
    sidx = torch.randperm(slots, generator=g, device=dev)[:B]
    for r in pad_rows:
        sidx[r] = -1
    fl = torch.zeros(ring + 1, dtype=torch.int8, device=dev)
    for r in flush_rows:
        fl[r] = 1
    q, kk = unit(max(T, 1), h, k)[:T], unit(max(T, 1), h, k)[:T]
    vv = torch.randn((T, hv, v), generator=g, device=dev)
    call = dict(
        q=q.to(torch.bfloat16), k=kk.to(torch.bfloat16), v=vv.to(torch.bfloat16),
        a=torch.randn((T, hv), generator=g, device=dev).to(torch.bfloat16),
        b=torch.randn((T, hv), generator=g, device=dev).to(torch.bfloat16),
        A_log=torch.log(torch.rand(hv, generator=g, device=dev) * 2 + 0.1),
        dt_bias=torch.randn(hv, generator=g, device=dev) * 0.5,
        checkpoint_state=(torch.randn((slots, hv, v, k), generator=g, device=dev) * state_std).to(state_dtype),
        d_cache=(torch.randn((ring, hv, L, v), generator=g, device=dev) * 0.05).to(torch.bfloat16),
        rawv_cache=torch.zeros((ring, hv, L, v), dtype=torch.bfloat16, device=dev),
        k_cache=unit(ring, h, L, k).to(torch.bfloat16),
        rawk_cache=torch.zeros((ring, h, L, k), dtype=torch.bfloat16, device=dev),
        g_cache=-torch.rand((ring, hv, L), generator=g, device=dev),
        beta_cache=None,
        out=torch.full((T, hv, v), 7.0, dtype=torch.bfloat16, device=dev),
        query_start_loc=qsl, ssm_state_indices=sidx.to(idx_dtype),
        replay_indices=torch.arange(B, device=dev).to(idx_dtype),
        write_pos=wp.to(torch.int32), cache_base=cb.to(torch.int32), is_flush=fl,
        launch_mode="verify", null_block_id=-1, scale=k**-0.5, use_qk_l2norm_in_kernel=True,
        max_spec_len=4, max_cache_len=L,
    )
    if flat:
        for name in ("q", "k", "v", "out"):
            call[name] = call[name].reshape(T, -1)
    return call


def gdn_replay_bytes(call: dict) -> int:
    """Algorithmic bytes of one Replay-SSM verify call: the checkpoint tile of every live (request, value head)
    read once, plus the history rows read and the ring rows / outputs written."""
    st = call["checkpoint_state"]
    hv, L = st.shape[1], call["d_cache"].shape[2]
    h = call["k_cache"].shape[1]
    qsl = call["query_start_loc"].tolist()
    total = 0
    for n, (si, ri) in enumerate(zip(call["ssm_state_indices"].tolist(), call["replay_indices"].tolist())):
        nt = min(qsl[n + 1] - qsl[n], 4)
        if nt <= 0 or si < 0 or int(call["is_flush"][ri]) != 0:
            continue
        W = min(max(int(call["write_pos"][ri]), 0), L)
        total += hv * 128 * 128 * st.element_size()
        total += W * (hv * (128 * 2 + 4) + h * 128 * 2)
        total += nt * (hv * 128 * 2 * 3 + h * 128 * 2 * 2)
    return total


def c5_gdn_spec(device="cuda", seed=5, batch=256, tokens=4):
    """Batch 256, 16 qk / 32 v heads, d_k = d_v = 128, fp32 state N(0, 0.02), 4 draft tokens,
    accepted-prefix lengths uniform in 0..4."""
    return make_gdn_case(batch, tokens, h=16, hv=32, seed=seed, device=device, slots=batch)


def attn_kv_bytes(kw: dict) -> int:
    """Algorithmic K+V bytes one call must read: ``sum(visible tokens) * 2 * kv_heads * head_dim``
    (the byte model of ``bench/bench_attn_decode.py:126,155-156``), window-limited where one is set."""
    kc = kw["k_cache"]
    kvh, hd = kc.shape[2], kc.shape[3]
    lens = kw["cache_seqlens"].tolist()
    cu = kw["cu_seqlens_q"].tolist()
    wl = kw.get("window_size", (-1, -1))[0]
    tok = 0
    for b, L in enumerate(lens):
        ql = cu[b + 1] - cu[b]
        if L <= 0 or ql <= 0:
            continue
        lo = 0 if wl is None or wl < 0 else max(0, L - ql - wl)
        tok += L - lo
    return tok * 2 * kvh * hd


def attn_flops(kw: dict) -> float:
    """4 * QH * HD * (query, key) pairs (``bench/bench_attn_extend.py:104``)."""
    q, kc = kw["q"], kw["k_cache"]
    qh, hd = q.shape[1], kc.shape[3]
    lens = kw["cache_seqlens"].tolist()
    cu = kw["cu_seqlens_q"].tolist()
    wl = kw.get("window_size", (-1, -1))[0]
    pairs = 0
    for b, L in enumerate(lens):
        ql = cu[b + 1] - cu[b]
        for t in range(ql):
            p = L - ql + t
            if p < 0:
                continue
            lo = 0 if wl is None or wl < 0 else max(0, p - wl)
            pairs += p + 1 - lo
    return 4.0 * qh * hd * pairs


def gdn_bytes(case: dict) -> int:
    """State read for every live request + state write for every request that commits at least one
    token + activations (``bench/bench_gdn.py:79-83`` extended by the commit rule)."""
    st = case["ssm_states"]
    tile = st.shape[1] * st.shape[2] * st.shape[3] * st.element_size()
    live = int((case["cache_indices"] >= 0).sum())
    commits = int(((case["accept_lens"] > 0) & (case["cache_indices"] >= 0)).sum())
    act = sum(case[n].numel() * case[n].element_size() for n in ("q", "k", "v", "a", "b"))
    out = case["v"].numel() * 2
    return tile * (live + commits) + act + out


__all__ = [n for n in dir() if not n.startswith("_") and n not in ("math", "torch", "annotations")]
