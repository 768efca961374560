"""CPU oracle for the Gated-DeltaNet recurrent update. TEST INFRASTRUCTURE ONLY.

Imported by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of ``bench.py``;
never by the product path.

PARITY UNPINNED by reference fixtures: the reference ships no torch implementation and no golden
vectors for this op (its GPU tests compare against SGLang's Triton kernels, which are not part of
the reference tree). This file restates the per-token math of ``docs/gdn-contract.md:25-37``:

    x    = a + dt_bias
    g    = -exp(A_log) * softplus(x)          softplus threshold 20 (``gdn_recurrent/kernel.cuh:45-49``)
    beta = sigmoid(b)                          rounded to bf16 in the packed call form (``kernel.cuh:259``)
    q'   = q / sqrt(sum q^2 + 1e-6) * scale    (``kernel.cuh:245-246``)
    k'   = k / sqrt(sum k^2 + 1e-6)
    S    = exp(g) * S ;  u = beta * (v - S k') ;  S = S + u (x) k' ;  o = S q'

with the state laid out ``[slots, HV, V, K]`` (K contiguous) and key head ``h = hv // (HV // H)``,
plus the edge semantics of ``docs/gdn-contract.md:61-67`` (PAD slot handling) and the
accepted-prefix commit the speculative path adds: after ``T`` chained tokens the stored state
becomes the state after exactly ``accept_len[n]`` tokens (0 leaves it bit-identical) while outputs
are produced for all ``T`` tokens. What pins it instead of reference fixtures:
``tests/golden/gdn_*.npz`` hold outputs of the independent third-party implementation
``fla.ops.gated_delta_rule.naive.naive_recurrent_gated_delta_rule`` (flash-linear-attention 0.5.1)
on the same seeded inputs, written by ``tests/golden/make_golden.py``.
"""

from __future__ import annotations

import torch


def gate(a, b, A_log, dt_bias, round_beta_bf16: bool = False, dtype=torch.float32):
    """(g, beta) from the raw gate inputs; ``a, b [..., HV]``, ``A_log, dt_bias [HV]``."""
    x = a.to(dtype) + dt_bias.to(dtype)
    sp = torch.where(x <= 20.0, torch.log1p(torch.exp(torch.clamp(x, max=20.0))), x)
    g = -torch.exp(A_log.to(dtype)) * sp
    beta = torch.sigmoid(b.to(dtype))
    if round_beta_bf16:
        beta = beta.to(torch.bfloat16).to(dtype)
    return g, beta


def l2norm(x, dtype=torch.float32):
    x = x.to(dtype)
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-6)


def recurrent_spec(
    q, k, v, a, b, A_log, dt_bias, state, cache_indices, accept_len=None, *,
    scale=None, l2norm_qk=True, round_beta_bf16=False, pad_reads_zero=False, dtype=torch.float32,
):
    """``T`` chained GDN tokens per request with accepted-prefix commit.

    q, k ``[B, T, H, K]``; v ``[B, T, HV, V]``; a, b ``[B, T, HV]``; state ``[slots, HV, V, K]``
    (modified in place); cache_indices ``[B]`` (``< 0`` = PAD); accept_len ``[B]`` in ``0..T``
    (None = commit all T, the plain decode behaviour).
    PAD rows: ``pad_reads_zero=False`` (packed decode form) gives a zero output row and leaves
    every state untouched; ``True`` (split decode form) computes from a zero state without
    storing it (``docs/gdn-contract.md:61-67``).
    Returns ``out fp32 [B, T, HV, V]``.
    """
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    grp = HV // H
    scale = K**-0.5 if scale is None else float(scale)
    g, beta = gate(a, b, A_log, dt_bias, round_beta_bf16, dtype)
    qn = (l2norm(q, dtype) if l2norm_qk else q.to(dtype)) * scale
    kn = l2norm(k, dtype) if l2norm_qk else k.to(dtype)
    qn = qn.repeat_interleave(grp, dim=2)  # [B, T, HV, K]
    kn = kn.repeat_interleave(grp, dim=2)
    out = torch.zeros((B, T, HV, V), dtype=dtype)
    idx = [int(i) for i in cache_indices.tolist()]
    acc = [T] * B if accept_len is None else [int(x) for x in accept_len.tolist()]
    for n in range(B):
        pad = idx[n] < 0
        if pad and not pad_reads_zero:
            continue
        S = torch.zeros((HV, V, K), dtype=dtype) if pad else state[idx[n]].to(dtype).clone()
        for t in range(T):
            if t == acc[n] and not pad:
                state[idx[n]] = S.to(state.dtype)
            S = S * torch.exp(g[n, t])[:, None, None]
            u = beta[n, t][:, None] * (v[n, t].to(dtype) - torch.einsum("hvk,hk->hv", S, kn[n, t]))
            S = S + u[:, :, None] * kn[n, t][:, None, :]
            out[n, t] = torch.einsum("hvk,hk->hv", S, qn[n, t])
        if acc[n] >= T and not pad:
            state[idx[n]] = S.to(state.dtype)
    return out.float()


def replay_verify(call: dict, *, dtype=torch.float64):
    """Replay-SSM speculative verify: up to 4 chained GDN tokens per request computed against a read-only
    checkpoint state plus the ring of deltas committed since that checkpoint, without writing the state.

    Restates ``docs/gdn-contract.md:83-124`` (arguments, reads / writes, row handling, math) and the write rules
    of ``green_attention/csrc/sm90/gdn_recurrent/verify.cuh:228-234,317-323,651-655,765-775``.

    ``call`` holds the keyword arguments of the production call: ``q, k [T, H, K]``, ``v [T, HV, V]``,
    ``a, b [T, HV]`` bf16, ``A_log, dt_bias [HV]``, ``checkpoint_state [slots, HV, V, K]`` (read only),
    ``d_cache, rawv_cache [ring, HV, L, V]`` bf16, ``k_cache, rawk_cache [ring, H, L, K]`` bf16,
    ``g_cache [ring, HV, L]`` fp32, ``query_start_loc [B+1]``, ``ssm_state_indices [B]`` (``< 0`` = PAD),
    ``replay_indices [B]``, ``write_pos, cache_base [ring+1]`` int32, ``is_flush [ring+1]`` int8, ``scale``.

    Per request n with ring slot r, ``W = clamp(write_pos[r], 0, L)`` committed history entries at physical
    positions ``(cache_base[r] + c) & (L-1)``: the effective state is
    ``S = exp(sum g_hist) S0 + sum_c exp(sum_{i>c} g_hist_i) d_c k_c^T`` (bf16 high parts of d and k only), on
    which the ordinary chained recurrence of :func:`recurrent_spec` runs for ``spec_len`` tokens. Written:
    ``out[bos+j]``; for ``write_pos + j < L`` the delta ``u_j`` as a (high, residual) bf16 pair into ``d_cache`` /
    ``rawv_cache``, ``g_j`` into ``g_cache``, and ``k'_j`` as a (high, residual) pair into ``k_cache`` /
    ``rawk_cache`` at ``(cache_base + write_pos + j) & (L-1)``. PAD rows: zero output, nothing else; rows whose
    ring slot is being flushed: nothing at all.
    Ring tensors are modified in place; returns ``out`` as ``[T, HV, V]`` in ``dtype``, rows of flushed
    requests NaN so that a test cannot compare them by accident.
    """
    H, HV, L = call["k_cache"].shape[1], call["d_cache"].shape[1], call["d_cache"].shape[2]
    K, V = call["k_cache"].shape[3], call["d_cache"].shape[3]
    T_all = call["q"].shape[0]
    q, k, v = call["q"].reshape(T_all, H, K), call["k"].reshape(T_all, H, K), call["v"].reshape(T_all, HV, V)
    grp = HV // H
    scale = K**-0.5 if call.get("scale") is None else float(call["scale"])
    g_all, beta_all = gate(call["a"], call["b"], call["A_log"], call["dt_bias"], False, dtype)
    qn_all = l2norm(q, dtype) * scale
    kn_all = l2norm(k, dtype)
    qsl = [int(x) for x in call["query_start_loc"].tolist()]
    sidx = [int(x) for x in call["ssm_state_indices"].tolist()]
    ridx = [int(x) for x in call["replay_indices"].tolist()]
    out = torch.zeros((T_all, HV, V), dtype=dtype)
    for n in range(len(sidx)):
        bos, nt = qsl[n], min(qsl[n + 1] - qsl[n], 4)
        if nt <= 0:
            continue
        r = ridx[n]
        if sidx[n] < 0:
            continue  # zero rows
        if int(call["is_flush"][r]) != 0:
            out[bos:bos + nt] = float("nan")
            continue
        base, wp = int(call["cache_base"][r]), int(call["write_pos"][r])
        W = min(max(wp, 0), L)
        S = call["checkpoint_state"][sidx[n]].to(dtype).clone()  # [HV, V, K]
        for c in range(W):
            ph = (base + c) & (L - 1)
            gh = call["g_cache"][r, :, ph].to(dtype)                       # [HV]
            dh = call["d_cache"][r, :, ph].to(dtype)                       # [HV, V]
            kh = call["k_cache"][r, :, ph].to(dtype).repeat_interleave(grp, dim=0)  # [HV, K]
            S = S * torch.exp(gh)[:, None, None] + dh[:, :, None] * kh[:, None, :]
        for j in range(nt):
            t = bos + j
            kn = kn_all[t].repeat_interleave(grp, dim=0)                   # [HV, K]
            qn = qn_all[t].repeat_interleave(grp, dim=0)
            S = S * torch.exp(g_all[t])[:, None, None]
            u = beta_all[t][:, None] * (v[t].to(dtype) - torch.einsum("hvk,hk->hv", S, kn))
            S = S + u[:, :, None] * kn[:, None, :]
            out[t] = torch.einsum("hvk,hk->hv", S, qn)
            if wp + j < L:
                ph = (base + W + j) & (L - 1)
                uf = u.float()
                hi = uf.to(torch.bfloat16)
                call["d_cache"][r, :, ph] = hi
                call["rawv_cache"][r, :, ph] = (uf - hi.float()).to(torch.bfloat16)
                call["g_cache"][r, :, ph] = g_all[t].float()
                kf = kn_all[t].float()
                khi = kf.to(torch.bfloat16)
                call["k_cache"][r, :, ph] = khi
                call["rawk_cache"][r, :, ph] = (kf - khi.float()).to(torch.bfloat16)
    return out


def replay_verify_closed_form(call: dict, *, dtype=torch.float64):
    """The same outputs from the closed form the reference's kernels evaluate (``docs/gdn-contract.md:111-124``):
    ``T = (I + A)^-1``, ``D = R T^T``, ``O = e^G hw_q + D F`` with the history folded into ``hw_q`` / ``hw_k``.
    No ring writes; used by the tests to check :func:`replay_verify` against the contract's own formulas."""
    H, HV, L = call["k_cache"].shape[1], call["d_cache"].shape[1], call["d_cache"].shape[2]
    K, V = call["k_cache"].shape[3], call["d_cache"].shape[3]
    T_all = call["q"].shape[0]
    q, k, v = call["q"].reshape(T_all, H, K), call["k"].reshape(T_all, H, K), call["v"].reshape(T_all, HV, V)
    grp = HV // H
    scale = K**-0.5 if call.get("scale") is None else float(call["scale"])
    g_all, beta_all = gate(call["a"], call["b"], call["A_log"], call["dt_bias"], False, dtype)
    qn_all = (l2norm(q, dtype) * scale).repeat_interleave(grp, dim=1)  # [T, HV, K]
    kn_all = l2norm(k, dtype).repeat_interleave(grp, dim=1)
    qsl = [int(x) for x in call["query_start_loc"].tolist()]
    out = torch.zeros((T_all, HV, V), dtype=dtype)
    for n, (si, r) in enumerate(zip(call["ssm_state_indices"].tolist(), call["replay_indices"].tolist())):
        bos, nt = qsl[n], min(qsl[n + 1] - qsl[n], 4)
        if nt <= 0 or si < 0:
            continue
        if int(call["is_flush"][r]) != 0:
            out[bos:bos + nt] = float("nan")
            continue
        base, W = int(call["cache_base"][r]), min(max(int(call["write_pos"][r]), 0), L)
        S0 = call["checkpoint_state"][si].to(dtype)
        kq, kk = kn_all[bos:bos + nt], kn_all[bos:bos + nt]
        qq = qn_all[bos:bos + nt]
        hw_q = torch.einsum("hvk,jhk->hvj", S0, qq)
        hw_k = torch.einsum("hvk,jhk->hvj", S0, kk)
        if W > 0:
            ph = [(base + c) & (L - 1) for c in range(W)]
            gh = call["g_cache"][r][:, ph].to(dtype)                                   # [HV, W]
            dh = call["d_cache"][r][:, ph].to(dtype)                                   # [HV, W, V]
            kh = call["k_cache"][r][:, ph].to(dtype).repeat_interleave(grp, dim=0)     # [HV, W, K]
            pre = torch.cumsum(gh, dim=1)
            total = pre[:, -1]
            decay = torch.exp(total[:, None] - pre)                                    # [HV, W]
            for hw, x in ((hw_q, qq), (hw_k, kk)):
                sc = torch.einsum("hck,jhk->hcj", kh, x)                               # khist_c . x'_j
                hw.mul_(torch.exp(total)[:, None, None]).add_(torch.einsum("hcv,hc,hcj->hvj", dh, decay, sc))
        g = g_all[bos:bos + nt].T                                                      # [HV, nt]
        beta = beta_all[bos:bos + nt].T
        G = torch.cumsum(g, dim=1)
        gram_kk = torch.einsum("ihk,jhk->hij", kk, kk)
        gram_kq = torch.einsum("ihk,jhk->hij", kk, qq)
        ii, jj = torch.meshgrid(torch.arange(nt), torch.arange(nt), indexing="ij")
        decay_ij = torch.exp(G[:, :, None] - G[:, None, :])                            # exp(G_i - G_j)
        A = (ii > jj)[None] * beta[:, :, None] * decay_ij * gram_kk
        Tm = torch.linalg.inv(torch.eye(nt, dtype=dtype)[None] + A)
        R = beta[:, None, :] * (v[bos:bos + nt].to(dtype).permute(1, 2, 0) - torch.exp(G)[:, None, :] * hw_k)
        D = torch.einsum("hvj,hij->hvi", R, Tm)
        F = (ii <= jj)[None] * torch.exp(G[:, None, :] - G[:, :, None]) * gram_kq      # exp(G_j - G_i) kq[i,j]
        O = torch.exp(G)[:, None, :] * hw_q + torch.einsum("hvi,hij->hvj", D, F)
        out[bos:bos + nt] = O.permute(2, 0, 1)
    return out
