"""Benchmark of the hot path: FP8 (e4m3) paged-KV attention and the Gated-DeltaNet speculative step on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl green|reference]

The headline line is the production decode configuration (batch 128 per GPU, 64 query / 8 kv heads, head_dim 128,
page 64, contexts uniform in [1k, 32k]); a step is one decode call over the whole batch. ``value`` is KV bytes
attended per second (algorithmic bytes ``sum(ctx) * 2 * kv_heads * head_dim`` over the device time of the K timed
steps), inputs resident in HBM; ``e2e`` is the same quantity through the plugin call (``dispatch.with_kvcache``)
with the step's inputs (query, page table, lengths) copied from pinned host memory and the output copied back
every step; the KV pool is the serving cache and stays resident, as it does in the server. With N > 1 every rank
owns its own 128 requests and KV pool (requests are partitioned, no collective on the data path): weak scaling.

The same line carries, each measured in this run with CUDA events and the L2 flushed before every call:
``attn`` (speculative verify, extend with full and sliding-window attention, each with its own roofline block and
an oracle check of a sample of what was timed), ``gdn`` (speculative step with accepted-prefix commit and the
Replay-SSM verify; on every rank when N > 1), ``sustained`` (the decode call looped for seconds with the clocks
sampled) and, for N > 1, ``long_context`` (one sequence whose KV range is split across the ranks).
All inputs are seeded synthetic tensors with the shapes and distributions of the named configurations.

``--impl reference`` times the reference's CPU implementation of the same path (its torch oracle,
restated in ``oracle/attn_oracle.py``; the reference's CUDA is SM90 WGMMA and cannot be built for
sm_100) on the host cores, each step a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from greenattention_b200 import workloads as W  # noqa: E402

METRIC = "fp8_paged_decode_kv_bytes_per_s_B128"
UNIT = "TB/s"
WORKLOAD = "C2 production decode: B=128/GPU, QH64/KVH8, hd128, page 64, ctx~U[1k,32k], q_len 1"
ATOL = RTOL = 2e-2
# DRAM bytes (read + write) the decode kernel moved per algorithmic byte in an ncu capture of the same kernel
# at batch 16 (dram__bytes_read.sum + dram__bytes_write.sum over sum(ctx) * 2048); the kernel is a pure stream,
# so a full launch is scaled by its tokens.
DECODE_DRAM_PER_ALGORITHMIC_BYTE = 1.0121


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 0.0)), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001 - NVML missing: report nulls
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        med = sorted(self.samples)[len(self.samples) // 2] if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


def quantiles(ms_list):
    """min / p25 / median of per-call times (ms -> us), the statistics the reference's benches print
    (``bench/bench_attn_decode.py:82-97,153``)."""
    s = sorted(ms_list)
    n = len(s)
    return {"min_us": s[0] * 1e3, "p25_us": s[n // 4] * 1e3, "median_us": s[n // 2] * 1e3, "calls": n}


def timed_calls(fn, calls, flush, before=None):
    """One CUDA-event pair per call on the current stream, the L2 flushed by a 512 MB write before each call."""
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(calls)]
    for s, e in ev:
        if before is not None:
            before()
        flush.zero_()
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    return [s.elapsed_time(e) for s, e in ev]


def attn_parity(kw, out, requests):
    """Oracle check of ``requests`` of a call that was just timed: max abs error and whether every element is
    within atol 2e-2 + rtol 2e-2 (the oracle runs here only as the checker of what the kernels produced)."""
    from oracle import attn_oracle

    sub = W.extract_requests(kw, requests, "cpu")
    ref, _ = attn_oracle.paged_attention(sub)
    got = out[W.request_rows(kw, requests).to(out.device)].float().cpu()
    err = (got - ref).abs()
    return {"requests": [int(r) for r in requests], "rows": int(got.shape[0]) * int(got.shape[1]),
            "max_abs_err": float(err.max()), "within_atol_rtol_2e-2": bool((err <= ATOL + RTOL * ref.abs()).all())}


def cpu_oracle_sample(n_requests: int, seed: int, repeats: int = 1):
    """Times the CPU oracle on a seeded sample of the decode workload; returns (TB/s, cores, description)."""
    from oracle import attn_oracle

    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
    torch.set_num_threads(cores)
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(1024, 32769, (n_requests,), generator=g).tolist()
    kw = W.c2_production_decode("cpu", seed=seed, lens=lens)
    nbytes = W.attn_kv_bytes(kw)
    t0 = time.perf_counter()
    for _ in range(repeats):
        attn_oracle.paged_attention(kw)
    dt = (time.perf_counter() - t0) / repeats
    return nbytes / dt / 1e12, cores, f"{n_requests} seeded requests ({sum(lens)} KV tokens) of the C2 workload", dt


def run_reference(args, rank):
    if rank != 0:
        return
    times, val = [], 0.0
    for i in range(args.warmup + args.steps):
        val, cores, sample, dt = cpu_oracle_sample(8, seed=100 + i)
        if i >= args.warmup:
            times.append((val, dt))
    value = sum(v for v, _ in times) / len(times)
    ms = 1e3 * sum(d for _, d in times) / len(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32 (dequantised e4m3)", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "each step = CPU torch oracle over a seeded 8-request sample"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------- GDN


def bench_gdn(dev, calls, hbm_gbs, flush, check=True):
    """C5 (speculative step with accepted-prefix commit) and the Replay-SSM verify of the same shape."""
    from greenattention_b200 import gdn as gdn_mod
    from greenattention_b200 import gdn_recurrent

    gdn_mod.set_standalone(True)  # no SGLang runtime context to ask which backend serves
    gdn_recurrent.ensure_ready(dev)
    c = W.c5_gdn_spec(dev)
    nbytes = W.gdn_bytes(c)
    start = c["ssm_states"].clone()
    kw = dict(q=c["q"], k=c["k"], v=c["v"], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
              ssm_states=c["ssm_states"], cache_indices=c["cache_indices"], accept_lens=c["accept_lens"])
    out = torch.empty(c["v"].shape, dtype=torch.bfloat16, device=dev)
    for _ in range(3):
        gdn_recurrent.gdn_spec_decode(out=out, **kw)
    ms = timed_calls(lambda: gdn_recurrent.gdn_spec_decode(out=out, **kw), calls, flush,
                     before=lambda: c["ssm_states"].copy_(start))
    st = quantiles(ms)
    med = st["median_us"] * 1e-6
    tokens = c["q"].shape[0] * c["q"].shape[1]
    res = {
        "workload": "C5 GDN spec: B=256, H16/HV32, K=V=128, fp32 state, 4 draft tokens, accept~U{0..4}",
        "us_per_call": st["median_us"], "stats": st, "verified_tok_per_s": tokens / med, "tokens_per_call": tokens,
        "roofline": {"bound": "hbm", "achieved": nbytes / med / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": nbytes / med / 1e9 / hbm_gbs, "algorithmic_bytes": nbytes},
        "l2": "flushed by a 512 MB write before each call",
    }
    if check:
        from oracle import gdn_oracle

        n = 16  # the first 16 requests of the timed batch, from the same starting state
        c["ssm_states"].copy_(start)
        got = gdn_recurrent.gdn_spec_decode(out_dtype=torch.float32, **kw)[:n].cpu()
        idx = c["cache_indices"][:n].long().cpu()
        got_state = c["ssm_states"].cpu()[idx]
        ref_state = start.cpu()
        ref = gdn_oracle.recurrent_spec(*(c[k][:n].cpu() for k in ("q", "k", "v", "a", "b")), c["A_log"].cpu(),
                                        c["dt_bias"].cpu(), ref_state, c["cache_indices"][:n].cpu(),
                                        c["accept_lens"][:n].cpu())
        res["parity"] = {"requests": n, "out_max_err_over_max": float((got - ref).abs().max() / ref.abs().max()),
                         "state_rel_norm_err": float((got_state - ref_state[idx]).norm() / ref_state[idx].norm()),
                         "tolerance": "out 1e-3, state 1e-5"}
    del c, kw, start, out
    # Replay-SSM verify of the same shape: read-only checkpoint, ring of 32 with a random number of entries
    rc = W.make_gdn_replay_case([4] * 256, h=16, hv=32, ring_len=32, seed=7, device=dev)
    rbytes = W.gdn_replay_bytes({k: (v.cpu() if isinstance(v, torch.Tensor) and v.numel() < 4096 else v) for k, v in rc.items()})
    for _ in range(3):
        gdn_recurrent.gdn_replayssm_verify(**rc)
    st = quantiles(timed_calls(lambda: gdn_recurrent.gdn_replayssm_verify(**rc), calls, flush))
    med = st["median_us"] * 1e-6
    res["replay_verify"] = {
        "workload": "Replay-SSM verify: B=256, H16/HV32, fp32 checkpoint (read only), ring 32 with U{0..32} entries, 4 tokens",
        "us_per_call": st["median_us"], "stats": st, "verified_tok_per_s": 1024 / med,
        "roofline": {"bound": "hbm", "achieved": rbytes / med / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                     "frac": rbytes / med / 1e9 / hbm_gbs, "algorithmic_bytes": rbytes},
    }
    return res


# ------------------------------------------------------------------------------------------- verify / extend


def bench_attn_paths(dev, hbm_gbs, bf16_tflops, flush, calls=20, check=True):
    """Speculative verify (C3) and chunked-prefill extend (C4, full and sliding-window) through the plugin
    front-end: min / p25 / median us per call over L2-flushed calls, a roofline block each (HBM for the HBM-bound
    verify, FP8 tensor for extend) and an oracle check of one request of what was timed."""
    from greenattention_b200 import attn_decode

    out = {}
    fp8_peak = attn_decode.fp8_tensor_peak_tflops(dev)
    out["fp8_tensor_peak_tflops"] = {"value": fp8_peak, "how": "tcgen05 e4m3 issue loop on every SM, measured in this run",
                                     "twice_measured_bf16_burst": 2 * bf16_tflops}

    def timed(kw, select):
        run = select(kw)
        if not callable(run):
            return {"declined": run}, None
        o = torch.empty(kw["q"].shape, dtype=torch.bfloat16, device=dev)
        for _ in range(3):
            run(**dict(kw, out=o))
        return quantiles(timed_calls(lambda: run(**dict(kw, out=o)), calls, flush)), o

    kw = W.c3_spec_verify(dev)
    st, o = timed(kw, attn_decode.select)
    if o is None:
        out["verify"] = st
    else:
        nb, fl, med = W.attn_kv_bytes(kw), W.attn_flops(kw), st["median_us"] * 1e-6
        out["verify"] = {"workload": "C3 verify: B=64, q_len 5, QH32/KVH8, hd128, page 64, prefix 8k",
                         "us_per_call": st["median_us"], "stats": st, "tflops": fl / med / 1e12,
                         "roofline": {"bound": "hbm", "achieved": nb / med / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                                      "frac": nb / med / 1e9 / hbm_gbs, "algorithmic_bytes": nb}}
        if check:
            out["verify"]["parity"] = attn_parity(kw, o, [0, 63])
    del kw, o
    for name, window in (("extend_full", None), ("extend_window1024", 1024)):
        kw = W.c4_extend(dev, window=window)
        st, o = timed(kw, attn_decode.select_extend)
        if o is None:
            out[name] = st
        else:
            fl, med = W.attn_flops(kw), st["median_us"] * 1e-6
            nb = W.attn_kv_bytes(kw) + 2 * kw["q"].numel() * 2
            out[name] = {"workload": f"C4 extend: B=8, 2048 new on 16k prefix, QH16/KVH8, hd256, page 64, window={window}",
                         "us_per_call": st["median_us"], "stats": st, "flops": fl,
                         "roofline": {"bound": "tensor", "achieved": fl / med / 1e12, "peak": fp8_peak, "unit": "TFLOP/s",
                                      "frac": fl / med / 1e12 / fp8_peak, "peak_kind": "measured FP8 issue rate (above)"},
                         "min_hbm_bytes": nb, "hbm_frac_at_min_bytes": nb / med / 1e9 / hbm_gbs}
            if check:
                out[name]["parity"] = attn_parity(kw, o, [3])
        del kw, o
        torch.cuda.empty_cache()
    # The reference's other instance shapes (green_attention/attn_decode.py:58-62), decode step, B=64 x 8 192 tokens:
    # head_dim 256 with GQA 6 and with GQA 2 under a 1 024-token window, head_dim 512 with GQA 8. HBM-bound.
    shapes = {}
    for name, H, win in (("hd256_gqa6", dict(q_heads=24, kv_heads=4, head_dim=256), None),
                         ("hd256_gqa2_window1024", dict(q_heads=16, kv_heads=8, head_dim=256), (1023, 0)),
                         ("hd512_gqa8", dict(q_heads=32, kv_heads=4, head_dim=512), None)):
        extra = {"window": win} if win else {}
        kw = W.make_paged_case([8192] * 64, [1] * 64, 64, seed=13, device=dev, kv_std=0.5, descale="rand",
                               return_lse=False, **H, **extra)
        st, o = timed(kw, attn_decode.select)
        if o is None:
            shapes[name] = st
        else:
            nb, med = W.attn_kv_bytes(kw), st["median_us"] * 1e-6
            shapes[name] = {"workload": f"decode B=64 x 8192 tokens, QH{H['q_heads']}/KVH{H['kv_heads']}, hd{H['head_dim']}, page 64"
                                        + (f", window {win[0] + 1}" if win else ""),
                            "us_per_call": st["median_us"], "stats": st,
                            "roofline": {"bound": "hbm", "achieved": nb / med / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                                         "frac": nb / med / 1e9 / hbm_gbs, "algorithmic_bytes": nb}}
            if check:
                shapes[name]["parity"] = attn_parity(kw, o, [0, 63])
        del kw, o
        torch.cuda.empty_cache()
    out["instance_shapes"] = shapes
    out["status_word"] = attn_decode.workspace_status(dev)
    return out


# ------------------------------------------------------------------------------------------- long context


def bench_long_context(dev, rank, world, steps=20, total_tokens=1 << 20, check_tokens=65536):
    """One decode step of a single sequence whose KV range is split across the ranks: local split-KV decode on the
    shard, then the exchange of the packed (O, LSE) partials and their merge, as one kernel over peer memory
    (``kv_shard.PeerExchange``) and, beside it, as an NCCL all-gather plus a merge kernel. Max over ranks. Before the 1M-token
    timing a ``check_tokens``-token sequence goes through the same call on every rank and rank 0 compares the
    result with the oracle's attention over the whole sequence."""
    import torch.distributed as dist

    from greenattention_b200 import kv_shard

    def agree(ok: bool) -> bool:
        """All ranks take the same branch: true only if every rank says so."""
        t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t.item())

    def shard_case(total, seed):
        """Every rank builds the same whole sequence (same seed) and keeps its own page range of it."""
        full = W.make_paged_case([total], [1], 64, q_heads=64, kv_heads=8, head_dim=128, seed=seed, device=dev,
                                 kv_std=0.5, descale="rand", descale_range=(0.5, 2.0), extra_pages=8, return_lse=True)
        lo, hi = kv_shard.shard_ranges(total, world, 64)[rank]
        local = dict(full)
        local["page_table"] = full["page_table"][:, lo // 64:].contiguous()
        local["cache_seqlens"] = torch.tensor([hi - lo], dtype=torch.int32, device=dev)
        return full, local

    # ---- the fused exchange + merge kernel over peer memory, when the group can map it (every rank or none)
    exch, why = None, None
    if os.environ.get("GA_BENCH_NO_PEER_EXCHANGE") == "1":
        why = "switched off by GA_BENCH_NO_PEER_EXCHANGE"
    else:
        try:
            exch = kv_shard.PeerExchange(64, 128, dev)
        except Exception as exc:  # noqa: BLE001 - the NCCL path is measured instead
            why = f"{type(exc).__name__}: {exc}"[:200]
    if not agree(exch is not None):
        exch = None

    # ---- parity of the sharded path at a size the oracle handles
    parity = None
    full, local = shard_case(check_tokens, seed=12)
    got = kv_shard.decode_kv_sharded(local, exchange=exch)
    via_nccl = kv_shard.decode_kv_sharded(local)
    torch.cuda.synchronize()
    same = agree(bool(torch.equal(got, via_nccl)))
    if exch is not None:
        exch.check_status()
    if rank == 0:
        from oracle import attn_oracle

        ref, _ = attn_oracle.paged_attention({k: (v.cpu() if isinstance(v, torch.Tensor) else v) for k, v in full.items()})
        err = (got.float().cpu() - ref[0]).abs()
        parity = {"tokens": check_tokens, "ranks": world, "max_abs_err": float(err.max()),
                  "within_atol_rtol_2e-2": bool((err <= ATOL + RTOL * ref[0].abs()).all()),
                  "fused_exchange_equals_nccl_path_bitwise": same if exch is not None else None}
    del full, local, got, via_nccl
    torch.cuda.empty_cache()

    lo, hi = kv_shard.shard_ranges(total_tokens, world, 64)[rank]
    kw = W.make_paged_case([hi - lo], [1], 64, q_heads=64, kv_heads=8, head_dim=128, seed=11 + rank, device=dev,
                           kv_std=0.5, descale="rand", descale_range=(0.5, 2.0), extra_pages=8, return_lse=True)
    for name in ("q", "k_descale", "v_descale"):  # the request's query and scales are the same on every rank
        dist.broadcast(kw[name], 0)

    def time_path(exchange):
        """(eager us, graph-replay us or None, last output) of the step, max over ranks."""
        for _ in range(3):
            kv_shard.decode_kv_sharded(kw, exchange=exchange)
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            out = kv_shard.decode_kv_sharded(kw, exchange=exchange)
        e.record()
        dist.barrier()
        torch.cuda.synchronize()
        out = out.clone()
        eager_ms = s.elapsed_time(e) / steps
        # The step is a handful of small launches around a 33 KB exchange, so the host is its limit when it is issued
        # call by call; a serving loop replays it from a CUDA graph (a collective is captured with it). Capture can
        # fail on one rank only; the ranks agree on the outcome before any of them enters the replay.
        graph_ms, graph, out_g = float("nan"), None, None
        captured = False
        if os.environ.get("GA_BENCH_NO_GRAPH") != "1":
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out_g = kv_shard.decode_kv_sharded(kw, exchange=exchange)
                captured = True
            except Exception as exc:  # noqa: BLE001 - report the eager number only
                print(f"long-context graph capture skipped on rank {rank}: {exc}", file=sys.stderr)
        if agree(captured):
            for _ in range(3):
                graph.replay()
            dist.barrier()
            torch.cuda.synchronize()
            s.record()
            for _ in range(steps):
                graph.replay()
            e.record()
            dist.barrier()
            torch.cuda.synchronize()
            graph_ms = s.elapsed_time(e) / steps
            if not agree(bool(torch.equal(out_g, out))):  # a replay that does not reproduce the eager result is no measurement
                graph_ms = float("nan")
        t = torch.tensor([eager_ms, graph_ms if graph_ms == graph_ms else -1.0], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t[0].item() * 1e3, (t[1].item() * 1e3 if t[1].item() > 0 else None), out  # all ranks replayed or none

    nccl_eager_us, nccl_graph_us, out = time_path(None)
    nccl_us = nccl_graph_us if nccl_graph_us is not None else nccl_eager_us
    res = {"workload": f"one {total_tokens}-token sequence, KV range split over {world} GPUs, QH64/KVH8, hd128, page 64",
           "kv_bytes_per_gpu": (hi - lo) * 2048}
    if exch is not None:
        eager_us, graph_us, out_f = time_path(exch)
        exch.check_status()
        us = graph_us if graph_us is not None else eager_us
        res.update({"us_per_call": us, "us_per_call_eager": eager_us,
                    "issued_as": "cuda graph replay" if graph_us is not None else "eager calls",
                    "exchange": "one kernel: peer stores of the 33 KB partial into every rank's buffer as (value, call number) pairs, bounded poll, merge",
                    "nccl_path": {"us_per_call": nccl_us, "us_per_call_eager": nccl_eager_us,
                                  "exchange": "NCCL all-gather of 33 KB per rank + merge kernel"},
                    "same_result_as_nccl_path": agree(bool(torch.equal(out_f, out)))})
        out = out_f
    else:
        res.update({"us_per_call": nccl_us, "us_per_call_eager": nccl_eager_us,
                    "issued_as": "cuda graph replay" if nccl_graph_us is not None else "eager calls",
                    "exchange": "one NCCL all-gather of 33 KB per rank, read in place by the merge kernel",
                    "fused_exchange_unavailable": why})
    res["aggregate_tbps"] = total_tokens * 2048 / res["us_per_call"] / 1e6
    res["parity"] = parity
    res["finite"] = bool(torch.isfinite(out.float()).all())
    return res


# ------------------------------------------------------------------------------------------- main


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="green", choices=["green", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="requests per GPU (the named configuration uses 128)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gdn", action="store_true")
    ap.add_argument("--no-attn-paths", action="store_true", help="skip the verify (C3) and extend (C4) legs")
    ap.add_argument("--no-sustained", action="store_true")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle checks of what was timed")
    ap.add_argument("--sustained-seconds", type=float, default=2.5)
    ap.add_argument("--extra", action="store_true", help="accepted for compatibility: the verify / extend legs run by default")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "green" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch.distributed as dist

    from greenattention_b200 import _C, attn_decode, dispatch

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the green kernels have no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    attn_decode.ensure_ready(dev)
    hbm_gbs, bf16_tflops, peak_kind = peaks()

    # Weak scaling: per-GPU work is fixed as N grows, so every rank serves the same draw of context lengths (the
    # one the N = 1 line is quoted on) with its own data and page placement (seed 2 + rank).
    g_len = torch.Generator().manual_seed(2)
    lens = torch.randint(1024, 32769, (args.batch,), generator=g_len).tolist()
    kw = W.c2_production_decode(dev, seed=2 + rank, batch=args.batch, lens=lens)
    nbytes = W.attn_kv_bytes(kw)
    run = attn_decode.select(kw)
    if not callable(run):
        raise SystemExit(f"decode declined: {run}")
    out = torch.empty(kw["q"].shape, dtype=torch.bfloat16, device=dev)
    call = dict(kw, out=out)
    for _ in range(args.warmup):
        run(**call)
    torch.cuda.synchronize()
    launches_per_step = _C.lib().ga_last_launch_count()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing: K steps between two events
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(physical_gpu_index(local)) as clocks:
        barrier()
        start.record()
        for _ in range(args.steps):
            run(**call)
        stop.record()
        barrier()
    ms_total = start.elapsed_time(stop)

    # ---- end to end through the plugin call with host inputs: one pinned staging buffer holds the step's query,
    # page table and lengths, so a step is one H2D copy, the plugin call, one D2H copy and an event wait
    def stock(**_):
        raise RuntimeError("the stock kernel must not be reached")

    plugin_call = dispatch.with_kvcache(stock)
    names = ("q", "page_table", "cache_seqlens", "cu_seqlens_q")
    offs, total = {}, 0
    for n in names:
        offs[n] = total
        total += (kw[n].numel() * kw[n].element_size() + 255) // 256 * 256
    stage_host = torch.empty(total, dtype=torch.uint8).pin_memory()
    stage_dev = torch.empty(total, dtype=torch.uint8, device=dev)
    devbuf = {}
    for n in names:
        t = kw[n].contiguous()
        nb = t.numel() * t.element_size()
        stage_host[offs[n]:offs[n] + nb].copy_(t.cpu().view(torch.uint8).reshape(-1))
        devbuf[n] = stage_dev[offs[n]:offs[n] + nb].view(t.dtype).view(t.shape)
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = total
    d2h = out_host.numel() * out_host.element_size()
    e2e_kw = dict(kw, out=out, **devbuf)
    done = torch.cuda.Event()

    def e2e_step():
        stage_dev.copy_(stage_host, non_blocking=True)
        res = plugin_call(**e2e_kw)
        out_host.copy_(res, non_blocking=True)
        done.record()
        done.synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    step_ms = []  # host clock per step, beside the device-timed total: shows when one slow step carries the mean
    for _ in range(args.steps):
        t0 = time.perf_counter()
        e2e_step()
        step_ms.append((time.perf_counter() - t0) * 1e3)
    e_stop.record()
    barrier()
    e2e_ms_total = e_start.elapsed_time(e_stop)
    step_ms.sort()

    stats = torch.tensor([ms_total, e2e_ms_total, float(nbytes)], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_total, e2e_ms_total, total_bytes = mx[0].item(), mx[1].item(), sm[2].item()
    else:
        total_bytes = float(nbytes)
    ms_step = ms_total / args.steps
    value = total_bytes / (ms_step * 1e-3) / 1e12
    e2e_value = total_bytes / (e2e_ms_total / args.steps * 1e-3) / 1e12

    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    line = None
    if rank == 0:
        per_gpu_gbs = nbytes / (start.elapsed_time(stop) / args.steps * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "us_per_call": ms_step * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e4m3 -> f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "requests_per_gpu": args.batch, "kv_tokens_rank0": nbytes // 2048,
                       "partitioning": f"requests x{world}, same context-length draw on every rank", "l2": "inputs (4.4 GB/GPU) larger than the 126 MB L2"},
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms_total / args.steps,
                    "step_ms_host_clock_rank0": {"min": step_ms[0], "median": step_ms[len(step_ms) // 2], "max": step_ms[-1]}},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": per_gpu_gbs / hbm_gbs, "peak_kind": f"{peak_kind} copy bandwidth",
                         "frac_of_8TBps_nominal": per_gpu_gbs / 8000.0,
                         "traffic": int(nbytes * DECODE_DRAM_PER_ALGORITHMIC_BYTE),
                         "kernel": "attn_wide_kernel of attn_wide.cuh (+ attn_combine_kernel inside the same events)"},
        }
        # the same call, one event pair per call with the L2 flushed in between
        line["stats"] = quantiles(timed_calls(lambda: run(**call), max(args.steps, 20), flush))
        if not args.no_parity:
            lens_t = kw["cache_seqlens"].tolist()
            pick = sorted({0, 1, 2, 3, 4, 5, lens_t.index(min(lens_t)), lens_t.index(max(lens_t))})
            line["parity"] = attn_parity(kw, out, pick)
            line["parity"]["status_word"] = attn_decode.workspace_status(dev)

    # ---- sustained: the decode call looped for seconds (what a serving loop holds, under the power cap)
    if not args.no_sustained:
        n_loop = max(int(args.sustained_seconds / (ms_step * 1e-3)), 10)
        with ClockSampler(physical_gpu_index(local)) as sclk:
            barrier()
            start.record()
            for _ in range(n_loop):
                run(**call)
            stop.record()
            barrier()
        sus_ms = start.elapsed_time(stop) / n_loop
        if world > 1:
            t = torch.tensor([sus_ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            sus_ms = t.item()
        if rank == 0:
            line["sustained"] = {"calls": n_loop, "seconds": sus_ms * n_loop * 1e-3, "us_per_call": sus_ms * 1e3,
                                 "value": total_bytes / (sus_ms * 1e-3) / 1e12, "unit": UNIT,
                                 "frac_of_measured_hbm": nbytes / (sus_ms * 1e-3) / 1e9 / hbm_gbs, "clocks": sclk.summary()}

    kw = call = e2e_kw = devbuf = out = None
    del stage_dev
    torch.cuda.empty_cache()

    # ---- GDN: every rank runs its own 256 requests (partitioned, no collective); tokens/s is the aggregate
    if not args.no_gdn:
        try:
            gdn_res = bench_gdn(dev, max(args.steps, 20), hbm_gbs, flush, check=(rank == 0 and not args.no_parity))
            us = torch.tensor([gdn_res["us_per_call"], gdn_res["replay_verify"]["us_per_call"]], dtype=torch.float64, device=dev)
        except Exception as exc:  # noqa: BLE001 - the decode line must still print
            gdn_res = {"error": repr(exc)}
            us = torch.tensor([float("inf"), float("inf")], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(us, op=dist.ReduceOp.MAX)
        if rank == 0:
            if "error" not in gdn_res and bool(torch.isfinite(us).all()):
                gdn_res["n_gpus"] = world
                gdn_res["us_per_call_max_over_ranks"] = us[0].item()
                gdn_res["aggregate_verified_tok_per_s"] = world * gdn_res["tokens_per_call"] / (us[0].item() * 1e-6)
                gdn_res["replay_verify"]["aggregate_verified_tok_per_s"] = world * 1024 / (us[1].item() * 1e-6)
            line["gdn"] = gdn_res
        torch.cuda.empty_cache()

    if rank == 0 and world == 1 and not args.no_attn_paths:
        try:
            line["attn"] = bench_attn_paths(dev, hbm_gbs, bf16_tflops, flush, check=not args.no_parity)
        except Exception as exc:  # noqa: BLE001
            line["attn"] = {"error": repr(exc)}
        torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        val, cores, sample, _ = cpu_oracle_sample(32, seed=7)
        line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    long_ctx = None
    if world > 1:
        del flush
        torch.cuda.empty_cache()
        try:
            long_ctx = bench_long_context(dev, rank, world)
        except Exception as exc:  # noqa: BLE001
            long_ctx = {"error": repr(exc)}
    if rank == 0:
        if long_ctx is not None:
            line["long_context"] = long_ctx
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
