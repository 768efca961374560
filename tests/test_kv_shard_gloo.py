"""Host logic of the KV-range-sharded decode on CPU: the shard planner, the packed (O, LSE) exchange over a
world-size-2 (and 3) ``gloo`` group, and the merge, with the CPU oracle standing in for the two CUDA calls."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from greenattention_b200 import kv_shard
from greenattention_b200 import workloads as W


def test_shard_ranges_cover_the_sequence_page_aligned():
    for total, world, page in [(1 << 20, 8, 64), (1000, 3, 16), (5, 4, 64), (0, 2, 16), (129, 2, 64), (64, 8, 64)]:
        ranges = kv_shard.shard_ranges(total, world, page)
        assert len(ranges) == world
        pos = 0
        for lo, hi in ranges:
            assert lo == pos or lo == hi == total or (lo == hi and lo >= pos)
            if hi > lo:
                assert lo == pos and lo % page == 0
                pos = hi
        assert pos == total
        sizes = [-(-(hi - lo) // page) for lo, hi in ranges]
        assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, result_dir):
    from oracle import attn_oracle

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        kw = W.make_paged_case([total], [1], 16, q_heads=8, kv_heads=2, head_dim=128, seed=77, descale="rand")
        lo, hi = kv_shard.shard_ranges(total, world, 16)[rank]

        def partial(**call):  # the oracle restricted to this rank's key range stands in for the CUDA call
            o_parts, l_parts = attn_oracle.kv_range_partials(call, [(lo, hi)])
            return o_parts[0][None], l_parts[0][:, None]

        def merge(o_parts, lse_parts):
            return attn_oracle.merge_partials(o_parts, lse_parts)[0]

        out = kv_shard.decode_kv_sharded(kw, partial_fn=partial, merge_fn=merge)
        whole, _ = attn_oracle.paged_attention(kw)
        err = (out - whole[0]).abs().max().item()
        with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
            f.write(repr(err))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,total", [(2, 1000), (3, 40), (2, 7)])
def test_sharded_decode_over_gloo_matches_whole_sequence(world, total, tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, total, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        err = float(open(tmp_path / f"rank{r}.txt").read())
        assert err <= 1e-5, (r, err)
