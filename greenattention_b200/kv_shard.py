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
"""

from __future__ import annotations

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


def decode_kv_sharded(
    local_kw: dict,
    group: Optional[dist.ProcessGroup] = None,
    partial_fn: Optional[Callable] = None,
    merge_fn: Optional[Callable] = None,
):
    """One decode step of a KV-range-sharded sequence. ``local_kw`` is this rank's ordinary decode call over its
    own shard (batch 1, one query token, ``cache_seqlens`` = tokens held locally, 0 allowed). Returns the merged
    bf16 output ``[q_heads, head_dim]`` on every rank.

    ``partial_fn(**local_kw) -> (o [1, QH, HD] fp32, lse [QH, 1])`` and ``merge_fn(o_parts, lse_parts) -> out``
    default to the CUDA entry points; tests of the exchange logic on CPU pass stand-ins.
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
    if world == 1:
        gathered = mine
    else:
        gathered = torch.empty(world * n, dtype=torch.float32, device=mine.device)
        dist.all_gather_into_tensor(gathered, mine, group=group)
    o_parts, lse_parts = unpack_partials(gathered, world, qh, hd)
    return merge_fn(o_parts, lse_parts)
