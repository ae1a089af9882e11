"""Paged KV block manager in the kernels' layout.

Host-side bookkeeping that mirrors `PagedKVCacheManager` of the reference
(flash_attn_llm/kv_cache/manager.py:158-711: LIFO free list :207/:260-292, per-request block
tables :298-315/:336-344, release :436-463, batch tables :623-662) but keeps, per layer,
separate K and V pools `[num_blocks, H_KV, 16, D]` — the layout the paged decode kernel reads
(flash_attn_kernel.cu:3446) — instead of the reference's `(num_blocks, 2, block, H_KV, D)` pool, and
a device-resident block table that is updated incrementally (only new entries are copied to the
device) instead of being rebuilt every step (tensor_parallel.py:218-228).

Tokens are written by the fused rotary + append kernel (`ops.rope_append_paged_fp16`), not by
per-token Python copies (manager.py:350-357).  Prefix caching and sliding-window eviction of the
reference are not built.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

BLOCK_SIZE = 16


class PagedKVCache:
    def __init__(self, num_blocks: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 max_batch: int, max_blocks_per_seq: int, device="cuda", dtype=torch.float16):
        if num_blocks <= 0 or num_layers <= 0 or max_batch <= 0 or max_blocks_per_seq <= 0:
            raise ValueError("num_blocks, num_layers, max_batch and max_blocks_per_seq must be positive")
        self.num_blocks, self.num_layers = num_blocks, num_layers
        self.num_kv_heads, self.head_dim = num_kv_heads, head_dim
        self.max_batch, self.max_blocks_per_seq = max_batch, max_blocks_per_seq
        self.device = torch.device(device)
        shape = (num_blocks, num_kv_heads, BLOCK_SIZE, head_dim)
        self.k_pools = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        self.v_pools = [torch.zeros(shape, dtype=dtype, device=self.device) for _ in range(num_layers)]
        # LIFO free list: the most recently freed block is reused first (manager.py:207, :260-275)
        self._free: List[int] = list(range(num_blocks - 1, -1, -1))
        self._tables: Dict[str, List[int]] = {}
        self._tokens: Dict[str, int] = {}
        self._row: Dict[str, int] = {}
        self._free_rows: List[int] = list(range(max_batch - 1, -1, -1))
        # device-resident table: one row per live request, -1 = unused (manager.py:640-650)
        self.block_table = torch.full((max_batch, max_blocks_per_seq), -1, dtype=torch.int32, device=self.device)

    # ---- allocation ---------------------------------------------------------------
    def get_num_free_blocks(self) -> int:
        return len(self._free)

    def can_allocate(self, num_tokens: int) -> bool:
        return (num_tokens + BLOCK_SIZE - 1) // BLOCK_SIZE <= len(self._free)

    def _take_blocks(self, n: int) -> List[int]:
        if n > len(self._free):
            raise MemoryError(f"paged KV cache exhausted: need {n} blocks, {len(self._free)} free")  # manager.py:269-292
        return [self._free.pop() for _ in range(n)]

    def allocate(self, request_id: str, num_tokens: int = 0) -> int:
        """Register a request and reserve blocks for `num_tokens` tokens; returns its table row."""
        if request_id in self._tables:
            raise ValueError(f"request {request_id!r} already allocated")
        if not self._free_rows:
            raise MemoryError("no free row in the device block table (max_batch live requests)")
        self._tables[request_id] = []
        self._tokens[request_id] = 0
        self._row[request_id] = self._free_rows.pop()
        try:
            self.reserve(request_id, num_tokens)
        except MemoryError:
            self.release(request_id)
            raise
        return self._row[request_id]

    def reserve(self, request_id: str, new_total_tokens: int) -> None:
        """Grow the request's block table so that `new_total_tokens` tokens fit (manager.py:336-344)."""
        table = self._tables[request_id]
        need = (new_total_tokens + BLOCK_SIZE - 1) // BLOCK_SIZE
        if need > self.max_blocks_per_seq:
            raise MemoryError(f"request needs {need} blocks, more than max_blocks_per_seq={self.max_blocks_per_seq}")
        if need > len(table):
            first_new = len(table)
            extra = self._take_blocks(need - len(table))
            table.extend(extra)
            row = self._row[request_id]
            self.block_table[row, first_new:need] = torch.tensor(extra, dtype=torch.int32)  # only the new entries

    def commit(self, request_id: str, num_new_tokens: int) -> None:
        """Advance the token count after the step's tokens were written into every layer."""
        total = self._tokens[request_id] + num_new_tokens
        if total > len(self._tables[request_id]) * BLOCK_SIZE:
            raise ValueError("commit beyond the reserved blocks")
        self._tokens[request_id] = total

    def release(self, request_id: str) -> None:
        """Return the request's blocks and its table row (manager.py:436-463)."""
        table = self._tables.pop(request_id)
        self._tokens.pop(request_id)
        row = self._row.pop(request_id)
        self._free.extend(reversed(table))
        self._free_rows.append(row)
        if table:
            self.block_table[row, : len(table)] = -1

    # ---- queries ------------------------------------------------------------------
    def get_cache_len(self, request_id: str) -> int:
        return self._tokens[request_id]

    def get_block_table(self, request_id: str) -> List[int]:
        return list(self._tables[request_id])

    def row_of(self, request_id: str) -> int:
        return self._row[request_id]

    def batch_rows(self, request_ids: Sequence[str]) -> torch.Tensor:
        return torch.tensor([self._row[r] for r in request_ids], dtype=torch.long, device=self.device)

    def batch_view(self, request_ids: Sequence[str], extra_tokens: int = 0):
        """(block_table [B, max_blocks_per_seq], seq_lens [B]) on the device for a batch of requests
        (manager.py:623-662).  When the batch occupies rows 0..B-1 in order the table is a view of the
        resident tensor; otherwise the rows are gathered."""
        rows = [self._row[r] for r in request_ids]
        lens = torch.tensor([self._tokens[r] + extra_tokens for r in request_ids], dtype=torch.int32).to(self.device)
        if rows == list(range(len(rows))):
            return self.block_table[: len(rows)], lens
        return self.block_table[self.batch_rows(request_ids)].contiguous(), lens

    # ---- data path ----------------------------------------------------------------
    def append_decode(self, layer: int, request_ids: Sequence[str], q, k, v, cos, sin):
        """One decode step for one layer: rotate q / k and store k, v of each request's new token at
        its next slot.  Call `reserve` (once per step) before, `commit` (once per step) after."""
        from . import ops
        table, lens = self.batch_view(request_ids)
        return ops.rope_append_paged_fp16(q, k, v, cos, sin, self.k_pools[layer], self.v_pools[layer], table, lens,
                                          self.max_blocks_per_seq)

    def append_prefill(self, layer: int, request_ids: Sequence[str], q, k, v, cos, sin, cu_seqlens):
        """Packed prompts for one layer: rotate q / k, store k / v from each request's current length on;
        returns (q_rot, k_rot) for the prefill attention."""
        from . import ops
        table, lens = self.batch_view(request_ids)
        return ops.rope_append_paged_fp16(q, k, v, cos, sin, self.k_pools[layer], self.v_pools[layer], table, lens,
                                          self.max_blocks_per_seq, cu_seqlens=cu_seqlens, return_k=True)
