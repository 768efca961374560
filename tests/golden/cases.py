"""The seeded cases behind the golden fixtures: shared by ``make_golden.py`` (which runs the
reference on them) and by the tests (which run the oracle and the CUDA path on them)."""

from __future__ import annotations

import hashlib

import torch

from greenattention_b200 import workloads as W

FP8 = torch.float8_e4m3fn


def _c1():
    return W.c1_cpu_decode("cpu")


def _verify_ragged():
    return W.make_paged_case(
        [5, 300, 129, 40, 2048, 12, 700, 10], [1, 4, 2, 10, 3, 1, 6, 4], 16,
        q_heads=32, kv_heads=8, head_dim=128, seed=103, descale="rand",
    )


def _window_hd256():
    return W.make_paged_case(
        [1, 2, 63, 64, 65, 100, 129, 1000], [1, 2, 4, 1, 5, 16, 3, 2], 16,
        q_heads=4, kv_heads=2, head_dim=256, seed=104, descale="scalar", window=(37, 0),
    )


def _empty_rows():
    return W.make_paged_case(
        [0, 17, 0, 300], [1, 1, 2, 1], 16, q_heads=8, kv_heads=2, head_dim=128, seed=105, descale="none",
    )


def _page1_fp8q():
    return W.make_paged_case(
        [1, 2, 127, 128, 129, 255], [1, 2, 4, 4, 4, 4], 1, q_heads=8, kv_heads=2, head_dim=128, seed=106,
        descale="rand", q_dtype=FP8, kv_stack=True, q_strided=True,
    )


def _extend_hd256():
    return W.make_paged_case(
        [200, 129, 96, 33, 1], [150, 64, 17, 5, 1], 64, q_heads=2, kv_heads=1, head_dim=256, seed=107,
        descale="rand", kv_std=0.5,
    )


def _extend_window_hd128():
    return W.make_paged_case(
        [300, 160, 50], [120, 160, 7], 16, q_heads=4, kv_heads=2, head_dim=128, seed=108, descale="none",
        window=(63, 0),
    )


def _saturation():
    kw = W.make_paged_case(
        [1500, 333, 64], [1, 1, 1], 16, q_heads=8, kv_heads=2, head_dim=128, seed=109, kv_std=150.0,
    )
    kw["k_descale"] = torch.full((3, 2), 1 / 150.0)
    kw["v_descale"] = torch.full((3, 2), 1 / 150.0)
    return kw


def _peaked():
    return W.make_paged_case(
        [3000, 1024], [4, 4], 16, q_heads=8, kv_heads=2, head_dim=128, seed=110, kv_std=3.0,
        descale="none",
    )


def _decode_hd512():
    # the reference's (512, 8) instance: Gemma-4 global attention, one query token
    return W.make_paged_case([1, 63, 300, 1025, 2500], [1] * 5, 64, q_heads=32, kv_heads=4, head_dim=512, seed=110,
                             descale="rand", q_dtype=torch.bfloat16)


ATTN_CASES = {
    "c1": _c1,
    "verify_ragged": _verify_ragged,
    "window_hd256": _window_hd256,
    "empty_rows": _empty_rows,
    "page1_fp8q": _page1_fp8q,
    "extend_hd256": _extend_hd256,
    "extend_window_hd128": _extend_window_hd128,
    "saturation": _saturation,
    "peaked": _peaked,
    "decode_hd512": _decode_hd512,
}

GDN_CASES = {
    "spec4": dict(batch=5, tokens=4, h=1, hv=2, slots=6, seed=201, accept=[0, 1, 2, 3, 4]),
    "decode1": dict(batch=3, tokens=1, h=1, hv=3, slots=4, seed=202, accept="all", gate_params="rand",
                    normalise_qk=False, state_std=0.1),
    "spec4_rand_gates": dict(batch=3, tokens=4, h=2, hv=4, slots=4, seed=203, accept=[4, 2, 3],
                             gate_params="rand", normalise_qk=False, state_std=0.1),
}


def gdn_case(name: str):
    return W.make_gdn_case(device="cpu", **GDN_CASES[name])


def digest(case: dict) -> str:
    """sha256 over the bytes of every tensor of a case (name order): pins the seeded generator."""
    h = hashlib.sha256()
    for name in sorted(case):
        val = case[name]
        if isinstance(val, torch.Tensor):
            t = val.contiguous()
            if t.dtype in (FP8, torch.bfloat16):
                t = t.view(torch.uint8 if t.dtype == FP8 else torch.int16)
            h.update(name.encode())
            h.update(t.numpy().tobytes())
    return h.hexdigest()
