"""Benchmark of the hot path: FP8 (e4m3) paged-KV decode at the production configuration (batch 128, 64 query /
8 kv heads, head_dim 128, page 64, contexts uniform in [1k, 32k]) plus the Gated-DeltaNet speculative step
(batch 256, 16/32 heads, 4 draft tokens). Synthetic seeded inputs with those shapes and distributions.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl green|reference]

A step is one decode call over the whole batch. ``value`` is KV bytes attended per second (algorithmic bytes
``sum(ctx) * 2 * kv_heads * head_dim`` over the device time of the K timed steps), inputs resident in HBM;
``e2e`` is the same quantity through the plugin call (``dispatch.with_kvcache``) with the step's inputs
(query, page table, lengths) copied from pinned host memory and the output copied back every step; the KV
pool is the serving cache and stays resident, as it does in the server. With N > 1 every rank owns its own
128 requests and KV pool (requests are partitioned, no collective on the data path): weak scaling.

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


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


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
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


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


def bench_gdn(dev, steps, warmup, hbm_gbs):
    from greenattention_b200 import gdn as gdn_mod
    from greenattention_b200 import gdn_recurrent

    gdn_mod._green_on_sm100 = lambda: True  # standalone run: no SGLang runtime context to ask
    gdn_recurrent.ensure_ready(dev)
    c = W.c5_gdn_spec(dev)
    nbytes = W.gdn_bytes(c)
    start = c["ssm_states"].clone()
    kw = dict(q=c["q"], k=c["k"], v=c["v"], a=c["a"], b=c["b"], A_log=c["A_log"], dt_bias=c["dt_bias"],
              ssm_states=c["ssm_states"], cache_indices=c["cache_indices"], accept_lens=c["accept_lens"])
    out = torch.empty(c["v"].shape, dtype=torch.bfloat16, device=dev)
    for _ in range(warmup):
        gdn_recurrent.gdn_spec_decode(out=out, **kw)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in ev:
        c["ssm_states"].copy_(start)
        flush.zero_()  # 512 MB write: evicts the state from the 126 MB L2
        s.record()
        gdn_recurrent.gdn_spec_decode(out=out, **kw)
        e.record()
    torch.cuda.synchronize()
    ms = sorted(s.elapsed_time(e) for s, e in ev)
    med = ms[len(ms) // 2]
    tokens = c["q"].shape[0] * c["q"].shape[1]
    res = {
        "workload": "C5 GDN spec: B=256, H16/HV32, K=V=128, fp32 state, 4 draft tokens, accept~U{0..4}",
        "us_per_call": med * 1e3, "verified_tok_per_s": tokens / (med * 1e-3), "algorithmic_bytes": nbytes,
        "hbm_gbs": nbytes / (med * 1e-3) / 1e9, "hbm_frac": nbytes / (med * 1e-3) / 1e9 / hbm_gbs,
        "l2": "flushed by a 512 MB write before each call",
    }
    del c, kw, start, out
    # Replay-SSM verify of the same shape: read-only checkpoint, ring of 32 with a random number of entries
    rc = W.make_gdn_replay_case([4] * 256, h=16, hv=32, ring_len=32, seed=7, device=dev)
    rbytes = W.gdn_replay_bytes({k: (v.cpu() if isinstance(v, torch.Tensor) and v.numel() < 4096 else v) for k, v in rc.items()})
    for _ in range(warmup):
        gdn_recurrent.gdn_replayssm_verify(**rc)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s, e in ev:
        flush.zero_()
        s.record()
        gdn_recurrent.gdn_replayssm_verify(**rc)
        e.record()
    torch.cuda.synchronize()
    ms = sorted(s.elapsed_time(e) for s, e in ev)
    med = ms[len(ms) // 2]
    res["replay_verify"] = {
        "workload": "Replay-SSM verify: B=256, H16/HV32, fp32 checkpoint (read only), ring 32 with U{0..32} entries, 4 tokens",
        "us_per_call": med * 1e3, "verified_tok_per_s": 1024 / (med * 1e-3), "algorithmic_bytes": rbytes,
        "hbm_gbs": rbytes / (med * 1e-3) / 1e9, "hbm_frac": rbytes / (med * 1e-3) / 1e9 / hbm_gbs,
    }
    return res


def bench_attn_extra(dev, hbm_gbs, steps=5):
    """Speculative verify (C3) and chunked-prefill extend (C4, full and sliding-window) through the plugin
    front-end: us/call, HBM GB/s for the HBM-bound verify, TFLOP/s for the tensor-bound extend."""
    from greenattention_b200 import attn_decode

    out = {}
    fp8_peak = attn_decode.fp8_tensor_peak_tflops(dev)
    out["fp8_tensor_peak_tflops"] = {"value": fp8_peak, "how": "tcgen05 e4m3 issue loop on every SM, measured in this run"}
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def timed(kw, select):
        run = select(kw)
        if not callable(run):
            return {"declined": run}
        o = torch.empty(kw["q"].shape, dtype=torch.bfloat16, device=dev)
        for _ in range(2):
            run(**dict(kw, out=o))
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for s, e in ev:
            flush.zero_()
            s.record()
            run(**dict(kw, out=o))
            e.record()
        torch.cuda.synchronize()
        ms = sorted(s.elapsed_time(e) for s, e in ev)
        return ms[len(ms) // 2]

    kw = W.c3_spec_verify(dev)
    ms = timed(kw, attn_decode.select)
    if isinstance(ms, dict):
        out["verify"] = ms
    else:
        nb, fl = W.attn_kv_bytes(kw), W.attn_flops(kw)
        out["verify"] = {"workload": "C3 verify: B=64, q_len 5, QH32/KVH8, hd128, prefix 8k", "us_per_call": ms * 1e3,
                         "hbm_gbs": nb / ms / 1e6, "hbm_frac": nb / ms / 1e6 / hbm_gbs, "tflops": fl / ms / 1e9}
    del kw
    for name, window in (("extend_full", None), ("extend_window1024", 1024)):
        kw = W.c4_extend(dev, window=window)
        ms = timed(kw, attn_decode.select_extend)
        if isinstance(ms, dict):
            out[name] = ms
        else:
            fl = W.attn_flops(kw)
            out[name] = {"workload": f"C4 extend: B=8, 2048 new on 16k prefix, QH16/KVH8, hd256, window={window}",
                         "us_per_call": ms * 1e3, "tflops": fl / ms / 1e9, "flops": fl,
                         "frac_of_fp8_peak": fl / ms / 1e9 / fp8_peak}
        del kw
    return out


def bench_long_context(dev, rank, world, steps=20, total_tokens=1 << 20):
    """One decode step of a single 1M-token sequence whose KV range is split across the ranks: local split-KV
    decode on the shard, NCCL all-gather of the packed (O, LSE) partials, local merge. Max over ranks."""
    import torch.distributed as dist

    from greenattention_b200 import kv_shard

    lo, hi = kv_shard.shard_ranges(total_tokens, world, 64)[rank]
    kw = W.make_paged_case([hi - lo], [1], 64, q_heads=64, kv_heads=8, head_dim=128, seed=11 + rank, device=dev,
                           kv_std=0.5, descale="rand", descale_range=(0.5, 2.0), extra_pages=8, return_lse=True)
    for name in ("q", "k_descale", "v_descale"):  # the request's query and scales are the same on every rank
        dist.broadcast(kw[name], 0)
    for _ in range(3):
        kv_shard.decode_kv_sharded(kw)
    dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        out = kv_shard.decode_kv_sharded(kw)
    e.record()
    dist.barrier()
    torch.cuda.synchronize()
    eager_ms = s.elapsed_time(e) / steps
    # The step is a handful of small launches around a 33 KB exchange, so the host is its limit when it is issued
    # call by call; a serving loop replays it from a CUDA graph (the collective is captured with it).
    graph_ms = float("nan")
    if os.environ.get("GA_BENCH_NO_GRAPH") != "1":
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out_g = kv_shard.decode_kv_sharded(kw)
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
            if not torch.equal(out_g, out):
                graph_ms = float("nan")  # a replay that does not reproduce the eager result is not a measurement
        except Exception as exc:  # noqa: BLE001 - report the eager number only
            print(f"long-context graph capture skipped: {exc}", file=sys.stderr)
    t = torch.tensor([eager_ms, graph_ms if graph_ms == graph_ms else -1.0], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    mn = torch.tensor([graph_ms if graph_ms == graph_ms else -1.0], dtype=torch.float64, device=dev)
    dist.all_reduce(mn, op=dist.ReduceOp.MIN)
    eager_us = t[0].item() * 1e3
    graph_us = t[1].item() * 1e3 if mn.item() > 0 else None  # only if every rank replayed it
    us = graph_us if graph_us is not None else eager_us
    local_bytes = (hi - lo) * 2048
    return {"workload": f"one {total_tokens}-token sequence, KV range split over {world} GPUs, QH64/KVH8, hd128, page 64",
            "us_per_call": us, "us_per_call_eager": eager_us, "issued_as": "cuda graph replay" if graph_us is not None else "eager calls",
            "kv_bytes_per_gpu": local_bytes, "aggregate_tbps": total_tokens * 2048 / us / 1e6,
            "exchange": "one NCCL all-gather of 33 KB per rank + local merge kernel", "finite": bool(torch.isfinite(out.float()).all())}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="green", choices=["green", "reference"])
    ap.add_argument("--batch", type=int, default=128, help="requests per GPU (the named configuration uses 128)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gdn", action="store_true")
    ap.add_argument("--extra", action="store_true", help="also time the verify (C3) and extend (C4) configurations")
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
    hbm_gbs, peak_kind = peaks()

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

    # ---- end to end through the plugin call with host inputs
    def stock(**_):
        raise RuntimeError("the stock kernel must not be reached")

    plugin_call = dispatch.with_kvcache(stock)
    host = {n: kw[n].cpu().pin_memory() for n in ("q", "page_table", "cache_seqlens", "cu_seqlens_q")}
    devbuf = {n: torch.empty_like(kw[n]) for n in host}
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def e2e_step():
        for n, t in host.items():
            devbuf[n].copy_(t, non_blocking=True)
        res = plugin_call(**dict(kw, out=out, **devbuf))
        out_host.copy_(res, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        e2e_step()
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e_start.record()
    for _ in range(args.steps):
        e2e_step()
    e_stop.record()
    barrier()
    e2e_ms_total = e_start.elapsed_time(e_stop)

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
                    "ms_per_step": e2e_ms_total / args.steps},
            "gpu_launches": launches_per_step * args.steps,
            "roofline": {"bound": "hbm", "achieved": per_gpu_gbs, "peak": hbm_gbs, "unit": "GB/s",
                         "frac": per_gpu_gbs / hbm_gbs, "peak_kind": f"{peak_kind} copy bandwidth",
                         "frac_of_8TBps_nominal": per_gpu_gbs / 8000.0,
                         # DRAM bytes per launch: ncu capture of the same kernel at batch 16 read+wrote 1.0125 x
                         # its algorithmic bytes (profiles/attn_rows_decode.md); scaled by the tokens of this launch
                         "traffic": int(nbytes * 1.0125),
                         "kernel": "attn_rows_kernel<128,1,3,1,0,true,6,1,2> (+ attn_combine_kernel, ~1.4 % of "
                                   "the call, inside the same events)"},
        }
        if not args.no_gdn:
            try:
                line["gdn"] = bench_gdn(dev, max(args.steps, 10), 3, hbm_gbs)
            except Exception as exc:  # noqa: BLE001 - the decode line must still print
                line["gdn"] = {"error": repr(exc)}
        if args.extra:
            try:
                kw = call = None
                torch.cuda.empty_cache()
                line["attn_extra"] = bench_attn_extra(dev, hbm_gbs)
            except Exception as exc:  # noqa: BLE001
                line["attn_extra"] = {"error": repr(exc)}
        if world == 1 and not args.no_cpu_baseline:
            val, cores, sample, _ = cpu_oracle_sample(32, seed=7)
            line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}
    long_ctx = None
    if world > 1:
        try:
            kw = call = None
            torch.cuda.empty_cache()
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
