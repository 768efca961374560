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
