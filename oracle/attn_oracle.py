"""CPU oracle for FP8 (e4m3) paged-KV attention. TEST INFRASTRUCTURE ONLY.

This file is a checker: it is imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``. The product path never imports it.

It restates, in plain torch fp32 on the CPU, the attention semantics the reference pins in its
own shape-generic test oracle (``op_test/sm90/test_attn_decode_fp8.py:105-149``):

* a bf16 query is first rounded to e4m3 (round-to-nearest-even, saturating at +-448) because the
  kernels multiply Q and K as FP8 (``test_attn_decode_fp8.py:108``; device side
  ``csrc/sm90/attn_decode_fp8/kernel.cuh:489-496``);
* K and V pages are dequantised exactly and multiplied by the per-(request, kv head) descale
  (``test_attn_decode_fp8.py:130-131``);
* token ``n`` of request ``b`` lives in page ``page_table[b, n // page]`` at row ``n % page``
  (``test_attn_decode_fp8.py:125-128``; device side ``kernel.cuh:160-195``);
* query ``t`` of a ``ql``-token request sits at absolute position ``L - ql + t`` and attends keys
  ``<=`` that position, and with a left window ``W`` only keys ``>= position - W``
  (``test_attn_decode_fp8.py:134-137``);
* the result is ``softmax(scale * q k^T) v`` in fp32 and the natural-log LSE, laid out
  ``out [total_q, q_heads, head_dim]`` and ``lse [q_heads, total_q]``
  (``test_attn_decode_fp8.py:138-148``); rows without any visible key give 0 and -inf
  (``kernel.cuh:621-624``).

Parity pin: ``tests/golden/attn_*.npz`` hold outputs of the reference's own ``reference()``
function, produced by ``tests/golden/make_golden.py`` in a container where the reference tree
was importable; ``tests/test_oracle_golden.py`` checks this restatement against them.
"""

from __future__ import annotations

import math

import torch

FP8 = torch.float8_e4m3fn
E4M3_MAX = 448.0


def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    """Saturating round-to-nearest-even to e4m3 (``test_attn_decode_fp8.py:36-37``)."""
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(FP8)


def token_slots(page_table_row: torch.Tensor, n_tokens: int, page: int):
    """(page id, row in page) of tokens 0..n_tokens-1 of one request: the bit-exact bookkeeping
    every kernel must reproduce (``kernel.cuh:160-195``: ``n >> page_shift``, ``n & page_mask``)."""
    n = torch.arange(n_tokens)
    return page_table_row[n // page].long(), n % page


def window_left_of(kw: dict) -> int:
    ws = kw.get("window_size", (-1, -1))
    if ws is None:
        return -1
    wl = ws[0]
    return -1 if wl is None else int(wl)


def paged_attention(kw: dict, q_as_e4m3: bool = True):
    """fp32 attention over the dequantised paged cache.

    ``kw`` uses the ``flash_attn_with_kvcache`` keyword names the reference's selectors read
    (``green_attention/attn_decode.py:152-258``): q, k_cache, v_cache, page_table, cache_seqlens,
    cu_seqlens_q, softmax_scale, window_size, k_descale, v_descale.
    Returns ``(out fp32 [total_q, QH, HD], lse fp32 [QH, total_q])``.
    """
    q = kw["q"]
    if q.dtype != FP8 and q_as_e4m3:
        q = to_e4m3(q)
    q = q.float()
    kc, vc, pt = kw["k_cache"], kw["v_cache"], kw["page_table"]
    lens = [int(x) for x in kw["cache_seqlens"].tolist()]
    cu = [int(x) for x in kw["cu_seqlens_q"].tolist()]
    page, kvh, hd = kc.shape[1], kc.shape[2], kc.shape[3]
    total_q, qh, _ = q.shape
    gqa = qh // kvh
    scale = kw.get("softmax_scale")
    scale = hd**-0.5 if scale is None else float(scale)
    wl = window_left_of(kw)
    kd, vd = kw.get("k_descale"), kw.get("v_descale")

    out = torch.zeros((total_q, qh, hd), dtype=torch.float32)
    lse = torch.full((qh, total_q), -math.inf, dtype=torch.float32)
    for b, L in enumerate(lens):
        q0, q1 = cu[b], cu[b + 1]
        ql = q1 - q0
        if L <= 0 or ql <= 0:
            continue
        pages, rows = token_slots(pt[b], L, page)
        k_tok = kc[pages, rows].float()  # [L, KVH, HD]
        v_tok = vc[pages, rows].float()
        cols = torch.arange(L)
        pos = L - ql + torch.arange(ql)
        visible = cols[None, :] <= pos[:, None]
        if wl >= 0:
            visible &= cols[None, :] >= (pos[:, None] - wl)
        for h in range(kvh):
            ks = k_tok[:, h] * (float(kd[b if kd.shape[0] > 1 else 0, h]) if kd is not None else 1.0)
            vs = v_tok[:, h] * (float(vd[b if vd.shape[0] > 1 else 0, h]) if vd is not None else 1.0)
            qq = q[q0:q1, h * gqa:(h + 1) * gqa]  # [ql, G, HD]
            s = torch.matmul(qq.reshape(ql * gqa, hd), ks.T).reshape(ql, gqa, L) * scale
            s = s.masked_fill(~visible[:, None, :], -math.inf)
            m = s.amax(-1, keepdim=True)
            live = torch.isfinite(m)
            m_safe = torch.where(live, m, torch.zeros_like(m))
            e = torch.exp(s - m_safe)
            den = e.sum(-1, keepdim=True)
            p = torch.where(live, e / den.clamp_min(1e-38), torch.zeros_like(e))
            o = torch.matmul(p.reshape(ql * gqa, L), vs).reshape(ql, gqa, hd)
            out[q0:q1, h * gqa:(h + 1) * gqa] = o
            row_lse = torch.where(live, m_safe + den.log(), torch.full_like(m, -math.inf))
            lse[h * gqa:(h + 1) * gqa, q0:q1] = row_lse.squeeze(-1).T
    return out, lse


def merge_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor):
    """LSE-weighted merge of normalised partial outputs (``kernel.cuh:665-749``).

    ``o_parts [S, rows, HD]`` are per-split softmax-normalised outputs, ``lse_parts [S, rows]`` the
    natural-log LSE of each split (-inf for a split that saw no key). Returns ``(o [rows, HD],
    lse [rows])``; rows no split saw give 0 / -inf (``kernel.cuh:712-717``).
    """
    o_parts = o_parts.float()
    lse_parts = lse_parts.float()
    m = lse_parts.amax(0)
    live = torch.isfinite(m)
    m_safe = torch.where(live, m, torch.zeros_like(m))
    w = torch.exp(lse_parts - m_safe[None])
    w = torch.where(torch.isfinite(lse_parts), w, torch.zeros_like(w))
    den = w.sum(0)
    o = (w[..., None] * o_parts).sum(0) / den.clamp_min(1e-38)[..., None]
    o = torch.where(live[..., None], o, torch.zeros_like(o))
    lse = torch.where(live, m_safe + den.log(), torch.full_like(m, -math.inf))
    return o, lse


def kv_range_partials(kw: dict, ranges):
    """Attention of a single-request decode call restricted to each ``[lo, hi)`` key range, as the
    KV-range-sharded long-context path computes it on each GPU. Returns (o_parts [S, QH, HD],
    lse_parts [S, QH]) whose ``merge_partials`` equals ``paged_attention`` of the whole range."""
    assert kw["cache_seqlens"].numel() == 1 and kw["q"].shape[0] == 1
    L = int(kw["cache_seqlens"][0])
    kc, vc, pt = kw["k_cache"], kw["v_cache"], kw["page_table"]
    page, kvh, hd = kc.shape[1], kc.shape[2], kc.shape[3]
    q = kw["q"]
    q = (to_e4m3(q) if q.dtype != FP8 else q).float()[0]  # [QH, HD]
    qh = q.shape[0]
    gqa = qh // kvh
    scale = kw.get("softmax_scale")
    scale = hd**-0.5 if scale is None else float(scale)
    kd, vd = kw.get("k_descale"), kw.get("v_descale")
    pages, rows = token_slots(pt[0], L, page)
    o_parts, l_parts = [], []
    for lo, hi in ranges:
        hi = min(hi, L)
        o = torch.zeros((qh, hd))
        l = torch.full((qh,), -math.inf)
        if hi > lo:
            k_tok = kc[pages[lo:hi], rows[lo:hi]].float()
            v_tok = vc[pages[lo:hi], rows[lo:hi]].float()
            for h in range(kvh):
                ks = k_tok[:, h] * (float(kd[0, h]) if kd is not None else 1.0)
                vs = v_tok[:, h] * (float(vd[0, h]) if vd is not None else 1.0)
                s = q[h * gqa:(h + 1) * gqa] @ ks.T * scale
                m = s.amax(-1, keepdim=True)
                e = torch.exp(s - m)
                den = e.sum(-1, keepdim=True)
                o[h * gqa:(h + 1) * gqa] = (e / den) @ vs
                l[h * gqa:(h + 1) * gqa] = (m + den.log()).squeeze(-1)
        o_parts.append(o)
        l_parts.append(l)
    return torch.stack(o_parts), torch.stack(l_parts)
