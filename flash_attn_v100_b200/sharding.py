"""Head-shard rule for running one batch on several GPUs (one process per GPU).

Follows the reference's partition (tensor_parallel.py:435-457): rank r of `world`
owns KV heads [r*H_KV/world, (r+1)*H_KV/world) and the query heads that map to
them, [r*H_Q/world, (r+1)*H_Q/world); both counts must divide by `world`
(tensor_parallel.py:439-440).  Because h_kv = h_q // (H_Q // H_KV), the two ranges
are consistent and attention needs no communication: each rank's output is the
[.., H_Q/world, ..] slice of the full output.  `block_table` / `seq_lens` are
replicated.  Shards are meant to be *born* sharded (each rank projects only its
own heads), so there is no scatter kernel; `shard_heads` exists for tests and
for callers that start from full tensors.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch


@dataclass(frozen=True)
class HeadShard:
    rank: int
    world: int
    q_heads: Tuple[int, int]   # [begin, end)
    kv_heads: Tuple[int, int]


def head_shard(H_Q: int, H_KV: int, rank: int, world: int) -> HeadShard:
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if H_Q % H_KV != 0:
        raise ValueError("H_Q must be divisible by H_KV")
    if H_Q % world != 0 or H_KV % world != 0:
        raise ValueError(f"H_Q={H_Q} and H_KV={H_KV} must both be divisible by world={world}")
    q = H_Q // world
    kv = H_KV // world
    return HeadShard(rank, world, (rank * q, (rank + 1) * q), (rank * kv, (rank + 1) * kv))


def shard_heads(t: torch.Tensor, begin: int, end: int, head_dim: int = 1) -> torch.Tensor:
    """Contiguous copy of heads [begin, end) along `head_dim`."""
    return t.narrow(head_dim, begin, end - begin).contiguous()


def shard_decode_inputs(q, k, v, rank: int, world: int):
    """Slices of q [B,H_Q,1,D] and k/v ([B,H_KV,N,D] or [pages,H_KV,16,D]) owned by `rank`."""
    s = head_shard(q.size(1), k.size(1), rank, world)
    return (shard_heads(q, *s.q_heads), shard_heads(k, *s.kv_heads), shard_heads(v, *s.kv_heads), s)


def gather_head_outputs(local_out: torch.Tensor, world: int, group=None) -> torch.Tensor:
    """All-gather per-rank outputs [B, H_Q/world, ...] into [B, H_Q, ...] (only for callers
    that need the full tensor on every rank; the attention path itself never calls this)."""
    import torch.distributed as dist
    parts = [torch.empty_like(local_out) for _ in range(world)]
    dist.all_gather(parts, local_out.contiguous(), group=group)
    return torch.cat(parts, dim=1)
