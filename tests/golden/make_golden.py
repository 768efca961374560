"""Generate the golden fixtures in this directory. Run once, where the reference tree is importable:

    python tests/golden/make_golden.py --reference /path/to/GreenAttention

Attention: every case of ``cases.ATTN_CASES`` is run through the reference's own shape-generic oracle
``reference()`` (``op_test/sm90/test_attn_decode_fp8.py:105-149``) on CPU tensors; outputs and the LSE go
to ``attn_<case>.npz`` with the sha256 of the inputs. Host bookkeeping: the reference's ``plan_splits``
(``green_attention/attn_decode.py:123-134``) and ``kvcache_op`` (``green_attention/dispatch.py:109-116``)
are tabulated into ``host_tables.json``.

GDN: the reference has no CPU implementation of the recurrence, so ``gdn_<case>.npz`` holds the output of
the third-party ``fla.ops.gated_delta_rule.naive.naive_recurrent_gated_delta_rule`` (flash-linear-attention
0.5.1, shipped in the image) called token-prefix by token-prefix to obtain the state after each request's accepted prefix (stored for the referenced slots only).
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import warnings

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests.golden import cases  # noqa: E402


def attention(ref_root: str, only=None) -> None:
    sys.path[:0] = [ref_root, os.path.join(ref_root, "op_test", "sm90")]
    import test_attn_decode_fp8 as ref_tests  # the reference's test module (holds its torch oracle)

    for name, build in cases.ATTN_CASES.items():
        if only and name not in only:
            continue
        kw = build()
        out, lse = ref_tests.reference(kw)
        np.savez_compressed(
            os.path.join(HERE, f"attn_{name}.npz"),
            out=out.numpy().astype(np.float32), lse=lse.numpy().astype(np.float32),
            digest=np.array(cases.digest(kw)),
        )
        print(f"attn_{name}: out {tuple(out.shape)} |out|max {out.abs().max():.4f}")


def host_tables(ref_root: str) -> None:
    sys.path[:0] = [ref_root]
    from green_attention import attn_decode as ref_attn
    from green_attention import dispatch as ref_dispatch

    plan = []
    for batch in (1, 2, 4, 5, 8, 32, 51, 128, 1024):
        for ctx in (1, 255, 256, 257, 4096, 20000, 32768, 1 << 20):
            for sm in (132, 148):
                for units in (2, 4, 8, 16):
                    for windowed in (False, True):
                        plan.append([batch, ctx, sm, units, windowed,
                                     ref_attn.plan_splits(batch, ctx, sm, units, windowed)])
    ops = [[mq, ref_dispatch.kvcache_op(mq)] for mq in (None, 0, 1, 2, 5, 16, 17, 2048, "x", 1.0)]
    with open(os.path.join(HERE, "host_tables.json"), "w") as f:
        json.dump({"plan_splits": plan, "kvcache_op": ops, "max_verify_q": ref_dispatch.MAX_VERIFY_Q,
                   "ops": list(ref_dispatch.OPS)}, f)
    print(f"host_tables: {len(plan)} plan_splits rows, {len(ops)} kvcache_op rows")


def gdn() -> None:
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        from fla.ops.gated_delta_rule.naive import naive_recurrent_gated_delta_rule as fla_naive

    for name in cases.GDN_CASES:
        c = cases.gdn_case(name)
        B, T, H, K = c["q"].shape
        HV = c["v"].shape[2]
        grp = HV // H
        x = c["a"].float() + c["dt_bias"].float()
        sp = torch.where(x <= 20.0, torch.log1p(torch.exp(x.clamp(max=20.0))), x)
        g = -torch.exp(c["A_log"].float()) * sp
        beta = torch.sigmoid(c["b"].float())
        q = c["q"].float()
        k = c["k"].float()
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6)
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        q = q.repeat_interleave(grp, dim=2)
        k = k.repeat_interleave(grp, dim=2)
        idx = c["cache_indices"].long()
        s0 = c["ssm_states"][idx].float().transpose(-1, -2).contiguous()  # fla keeps [B, H, K, V]
        out, _ = fla_naive(q, k, c["v"].float(), beta, g, scale=c["scale"], initial_state=s0,
                           output_final_state=True)
        final = c["ssm_states"].float().clone()
        acc = c["accept_lens"].tolist()
        for n in range(B):
            if acc[n] == 0:
                continue
            _, st = fla_naive(q[n:n + 1, :acc[n]], k[n:n + 1, :acc[n]], c["v"][n:n + 1, :acc[n]].float(),
                              beta[n:n + 1, :acc[n]], g[n:n + 1, :acc[n]], scale=c["scale"],
                              initial_state=s0[n:n + 1], output_final_state=True)
            final[idx[n]] = st[0].transpose(-1, -2)
        np.savez_compressed(
            os.path.join(HERE, f"gdn_{name}.npz"),
            out=out.numpy().astype(np.float32), state=final[idx].numpy().astype(np.float32),
            digest=np.array(cases.digest(c)),
        )
        print(f"gdn_{name}: out {tuple(out.shape)} |out|max {out.abs().max():.4f}")


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the GreenAttention source tree")
    ap.add_argument("--only", nargs="*", help="attention cases to (re)generate; everything when absent")
    args = ap.parse_args()
    torch.manual_seed(0)
    attention(args.reference, args.only)
    if not args.only:
        host_tables(args.reference)
        gdn()
