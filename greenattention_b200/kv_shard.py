"""Decode of ONE long sequence whose KV range is split across GPUs (one process per GPU).

The reference has no multi-GPU path; its only long-context mechanism is single-GPU split-KV with an LSE combine
(``csrc/sm90/attn_decode_fp8/kernel.cuh:197-253,659-749``). This module is the same (O, LSE) merge one level up:

1. rank r owns the contiguous, page-aligned KV range ``shard_ranges(...)[r]`` of the sequence in its own local
   page pool and runs the ordinary split-KV decode kernel on it, asking for a normalised fp32 partial output and
   the natural-log LSE (``attn_decode.decode_partial``);
2. the partials (``q_heads * head_dim + q_heads`` floats per rank, ~33 KB) are all-gathered with NCCL into a
   LOCAL buffer on every rank;
3. a local merge kernel (``attn_decode.merge_partials`` -> ``ga_attn_merge``) folds the ``world`` partials.

No kernel reads another GPU's memory and nothing on this path uses multicast loads. The exchange is latency
bound, so both tensors travel in one packed buffer (one collective per call).

``PeerExchange`` replaces steps 2 and 3 by ONE kernel (``ga_attn_exchange_merge``): every rank stores its partial
into the peers' gather buffers with plain peer stores (each float with its call number in one 8-byte store, so no
fence and no flag), polls (bounded) for the peers' rows and merges, so the collective's launch and latency and the second kernel drop out of a step that is all
latency. The buffers are torch symmetric memory (ordinary device memory mapped into every process of the group;
multicast is switched off). Without it (CPU ranks, a group that cannot map peer memory) the NCCL path stays.
"""

from __future__ import annotations

import ctypes
import os
from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_ranges(total_tokens: int, world: int, page_size: int) -> List[Tuple[int, int]]:
    """Contiguous ``[lo, hi)`` token ranges, one per rank, cut at page boundaries and balanced to one page.
    Ranks past the end of a short sequence get an empty range."""
    if world <= 0 or page_size <= 0:
        raise ValueError("world and page_size must be positive")
    pages = -(-max(total_tokens, 0) // page_size)
    out, lo_page = [], 0
    for r in range(world):
        n = pages // world + (1 if r < pages % world else 0)
        lo, hi = lo_page * page_size, min((lo_page + n) * page_size, total_tokens)
        out.append((min(lo, total_tokens), max(min(lo, total_tokens), hi)))
        lo_page += n
    return out


def pack_partial(o: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
    """``o [rows, HD]`` fp32 and ``lse [rows]`` fp32 -> one ``[rows * (HD + 1)]`` buffer (O first, then LSE)."""
    return torch.cat([o.reshape(-1).float(), lse.reshape(-1).float()])


def unpack_partials(buf: torch.Tensor, world: int, rows: int, hd: int):
    buf = buf.view(world, rows * (hd + 1))
    return buf[:, : rows * hd].reshape(world, rows, hd), buf[:, rows * hd:].reshape(world, rows)


class PeerExchange:
    """Buffers and state of the fused exchange + merge for one (group, rows, head_dim): a gather buffer in symmetric
    memory, the device array of its peer pointers, the call counter and a status word.
    Construction is collective over ``group`` (every rank, same arguments). ``merge(mine)`` is what a decode step
    calls; it allocates nothing and can be captured in a CUDA graph (every rank must replay the same calls)."""

    STATUS_PEER_WAIT = 6

    def __init__(self, rows: int, head_dim: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 wait_polls: int = 0):
        # ordinary peer mappings only: no multicast object is created for these buffers
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.group, self.rows, self.head_dim, self.device = group, int(rows), int(head_dim), torch.device(device)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.wait_polls = int(wait_polls)
        n = self.rows * (self.head_dim + 1)
        # every float travels as an 8-byte (value, call number) pair: [2 parities][world][n][2] 32-bit words
        self.buf = symm_mem.empty(2 * self.world * n * 2, dtype=torch.int32, device=self.device)
        self.buf.zero_()
        self._buf_hdl = symm_mem.rendezvous(self.buf, group)
        self.buf_ptrs = torch.tensor(list(self._buf_hdl.buffer_ptrs), dtype=torch.int64, device=self.device)
        self.epoch = torch.zeros(2, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.out = torch.empty((self.rows, self.head_dim), dtype=torch.bfloat16, device=self.device)
        torch.cuda.synchronize(self.device)
        dist.barrier(group)  # every rank's zeros are in place before anyone stores into a peer

    def merge(self, mine: torch.Tensor) -> torch.Tensor:
        """``mine``: this rank's packed partial ``[rows * (head_dim + 1)]`` fp32. Returns the merged bf16
        ``[rows, head_dim]`` (the same tensor every call)."""
        from greenattention_b200 import _C

        if mine.dtype != torch.float32 or mine.numel() != self.rows * (self.head_dim + 1) or not mine.is_contiguous():
            raise ValueError("PeerExchange.merge: a dense fp32 partial of rows * (head_dim + 1) elements is expected")
        x = _C.GaExchangeParams()
        x.mine, x.peer_bufs, x.peer_flags = mine.data_ptr(), self.buf_ptrs.data_ptr(), None
        x.epoch, x.rank, x.world, x.rows, x.head_dim = self.epoch.data_ptr(), self.rank, self.world, self.rows, self.head_dim
        x.out, x.lse, x.status, x.wait_polls = self.out.data_ptr(), None, self.status.data_ptr(), self.wait_polls
        with torch.cuda.device(self.device):
            _C.check(_C.lib().ga_attn_exchange_merge(ctypes.byref(x), torch.cuda.current_stream(self.device).cuda_stream),
                     "ga_attn_exchange_merge")
        return self.out

    def check_status(self) -> None:
        """Raises if a wait for a peer ran out since the last check (synchronises)."""
        st = int(self.status.item())
        if st:
            self.status.zero_()
            raise RuntimeError(f"PeerExchange: status {st} (a peer's partial did not arrive within the limit)")


def decode_kv_sharded(
    local_kw: dict,
    group: Optional[dist.ProcessGroup] = None,
    partial_fn: Optional[Callable] = None,
    merge_fn: Optional[Callable] = None,
    exchange: Optional[PeerExchange] = None,
):
    """One decode step of a KV-range-sharded sequence. ``local_kw`` is this rank's ordinary decode call over its
    own shard (batch 1, one query token, ``cache_seqlens`` = tokens held locally, 0 allowed). Returns the merged
    bf16 output ``[q_heads, head_dim]`` on every rank.

    ``partial_fn(**local_kw) -> (o [1, QH, HD] fp32, lse [QH, 1])`` and ``merge_fn(o_parts, lse_parts) -> out``
    default to the CUDA entry points; tests of the exchange logic on CPU pass stand-ins. With ``exchange`` (a
    ``PeerExchange`` built for ``q_heads`` rows) the all-gather and the merge kernel are one kernel over peer memory.
    """
    default_kernels = partial_fn is None
    if partial_fn is None or merge_fn is None:
        from greenattention_b200 import attn_decode

        partial_fn = partial_fn or attn_decode.decode_partial
        merge_fn = merge_fn or attn_decode.merge_partials
    q = local_kw["q"]
    if q.shape[0] != 1:
        raise ValueError("decode_kv_sharded handles one query token of one sequence")
    qh, hd = q.shape[1], q.shape[2]
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n = qh * (hd + 1)
    if default_kernels:
        # The kernel writes O and LSE straight into this rank's slot of the packed send buffer and the merge kernel
        # reads the gathered buffer where it landed: no copy kernels between the decode, the collective and the merge.
        mine = torch.empty(n, dtype=torch.float32, device=q.device)
        partial_fn(into=mine, **local_kw)
    else:
        o, lse = partial_fn(**local_kw)
        mine = pack_partial(o[0], lse[:, 0])
    if exchange is not None and default_kernels:
        return exchange.merge(mine)
    if world == 1:
        gathered = mine
    else:
        gathered = torch.empty(world * n, dtype=torch.float32, device=mine.device)
        dist.all_gather_into_tensor(gathered, mine, group=group)
    o_parts, lse_parts = unpack_partials(gathered, world, qh, hd)
    return merge_fn(o_parts, lse_parts)
