"""KV-range-sharded decode of one sequence on 2 GPUs against the CPU oracle of the whole sequence: the NCCL form
(all-gather of the partials + local merge kernel) and the fused form (``kv_shard.PeerExchange``: one kernel that stores
the partial into the peer's buffer, waits with a limit and merges), which must agree bitwise over several calls (both
buffer parities). Skipped with fewer than two devices."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from greenattention_b200 import kv_shard
from greenattention_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, total, result_dir):
    from greenattention_b200 import attn_decode
    from oracle import attn_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        attn_decode.ensure_ready(dev)
        full = W.make_paged_case([total], [1], 64, q_heads=32, kv_heads=4, head_dim=128, seed=91, descale="rand", kv_std=0.5)
        lo, hi = kv_shard.shard_ranges(total, world, 64)[rank]
        local = W.case_to(full, dev)
        local["page_table"] = local["page_table"][:, lo // 64:].contiguous()  # this rank's pages only
        local["cache_seqlens"] = torch.tensor([hi - lo], dtype=torch.int32, device=dev)
        out = kv_shard.decode_kv_sharded(local)
        torch.cuda.synchronize()
        whole, _ = attn_oracle.paged_attention(full)
        err = (out.float().cpu() - whole[0]).abs()
        ok = bool((err <= 2e-2 + 2e-2 * whole[0].abs()).all())
        exch = kv_shard.PeerExchange(32, 128, dev)
        for _ in range(3):  # call numbers 1, 2, 3: both halves of the double buffer
            fused = kv_shard.decode_kv_sharded(local, exchange=exch).clone()
            torch.cuda.synchronize()
            ok = ok and bool(torch.equal(fused, out))
        exch.check_status()
        ok = ok and exch.epoch.tolist() == [3, 0]
        with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
            f.write(f"{int(ok)} {err.max().item()}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("total", [20000, 100])
def test_two_gpu_sharded_decode_matches_whole_sequence(total, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), total, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        ok, err = open(tmp_path / f"rank{r}.txt").read().split()
        assert ok == "1", (r, err)
