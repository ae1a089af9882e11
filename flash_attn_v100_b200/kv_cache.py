"""Paged KV block manager in the kernels' layout.

Host-side bookkeeping that mirrors `PagedKVCacheManager` of the reference
(flash_attn_llm/kv_cache/manager.py:158-711: LIFO free list :207/:260-292, per-request block
tables :298-315/:336-344, release :436-463, batch tables :623-662) but keeps, per layer,
separate K and V pools `[num_blocks, H_KV, 16, D]` — the layout the paged decode kernel reads
(flash_attn_kernel.cu:3446) — instead of the reference's `(num_blocks, 2, block, H_KV, D)` pool, and
a device-resident block table that is updated incrementally (only new entries are copied to the
device) instead of being rebuilt every step (tensor_parallel.py:218-228).

Tokens are written by the fused rotary + append kernel (`ops.rope_append_paged_fp16`), not by
per-token Python copies (manager.py:350-357).

Prefix caching (manager.py:496-571) and sliding-window block eviction (manager.py:577-617) follow the
reference's rules — block-aligned prefixes keyed by the SHA-256 of the comma-joined token ids, longest
match first; blocks that lie entirely before `length - sliding_window` are given up after an append —
with two differences that the kernel layout and correctness ask for:
  * every physical block carries its own reference count (requests that hold it + cache entries that
    pin it).  The reference decrements a prefix entry once per shared BLOCK of the released request
    (manager.py:452-461), which drops a multi-block prefix that other requests still read and appends
    its remaining blocks to the free list a second time;
  * an evicted block leaves a -1 at its position of the block table instead of shifting the table
    (manager.py:597-599 cuts the head off, after which position // block_size no longer finds a
    token's block): logical block i is entry i for the whole life of the request.
`allocate(..., token_ids=...)` adopts a cached prefix, so the prompt's first `get_cache_len()` tokens
need no prefill (the reference's `allocate` documents this and does not do it, manager.py:298-315).
"""
from __future__ import annotations

import hashlib
from typing import Dict, List, Optional, Sequence, Set

import torch

BLOCK_SIZE = 16


class PagedKVCache:
    def __init__(self, num_blocks: int, num_layers: int, num_kv_heads: int, head_dim: int,
                 max_batch: int, max_blocks_per_seq: int, device="cuda", dtype=torch.float16,
                 enable_prefix_cache: bool = True, sliding_window: int = 0):
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
        # sharing: holders of each physical block (request tables + prefix-cache entries)
        self._refs: List[int] = [0] * num_blocks
        self.enable_prefix_cache = bool(enable_prefix_cache)      # manager.py:52, :186
        self.sliding_window = int(sliding_window) if sliding_window else 0
        self._prefix_cache: Dict[str, List[int]] = {}             # key -> physical blocks (manager.py:216)
        self._prefix_ref_count: Dict[str, int] = {}               # key -> live requests attached to it (:220)
        self._req_keys: Dict[str, Set[str]] = {}                  # request -> keys it is attached to
        self._evicted: Dict[str, int] = {}                        # request -> leading blocks given up
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
        out = [self._free.pop() for _ in range(n)]
        for b in out:
            self._refs[b] = 1
        return out

    def _drop_ref(self, block: int) -> None:
        """One holder less; the block returns to the free list with its last holder (manager.py:277-279)."""
        self._refs[block] -= 1
        if self._refs[block] == 0:
            self._free.append(block)
        elif self._refs[block] < 0:
            raise RuntimeError(f"block {block} released more often than it was held")

    def allocate(self, request_id: str, num_tokens: int = 0, token_ids: Optional[Sequence[int]] = None) -> int:
        """Register a request and reserve blocks for `num_tokens` tokens; returns its table row.

        With `token_ids` (the prompt) and prefix caching on, the longest cached block-aligned prefix is
        adopted: its blocks open the request's table, `get_cache_len()` starts at the adopted length and
        only the rest of the prompt needs a prefill.  At least one prompt token is always left to compute
        (a prompt that is cached in full still needs the logits of its last token)."""
        if request_id in self._tables:
            raise ValueError(f"request {request_id!r} already allocated")
        if not self._free_rows:
            raise MemoryError("no free row in the device block table (max_batch live requests)")
        self._tables[request_id] = []
        self._tokens[request_id] = 0
        self._row[request_id] = self._free_rows.pop()
        self._req_keys[request_id] = set()
        self._evicted[request_id] = 0
        try:
            if token_ids is not None and self.enable_prefix_cache:
                self._adopt_prefix(request_id, token_ids)
            self.reserve(request_id, max(num_tokens, self._tokens[request_id]))
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
        """Advance the token count after the step's tokens were written into every layer; with a sliding
        window, blocks that have left it are given up (manager.py:359-363)."""
        total = self._tokens[request_id] + num_new_tokens
        if total > len(self._tables[request_id]) * BLOCK_SIZE:
            raise ValueError("commit beyond the reserved blocks")
        self._tokens[request_id] = total
        if self.sliding_window > 0 and total > self.sliding_window:
            self._evict_sliding_window(request_id)

    def release(self, request_id: str) -> None:
        """Return the request's blocks and its table row (manager.py:436-463).  A block shared with other
        requests or pinned by a prefix entry that other requests are attached to stays allocated."""
        table = self._tables.pop(request_id)
        self._tokens.pop(request_id)
        row = self._row.pop(request_id)
        self._evicted.pop(request_id, None)
        for key in self._req_keys.pop(request_id, ()):
            self._detach(key)
        for b in reversed(table):
            if b >= 0:
                self._drop_ref(b)
        self._free_rows.append(row)
        if table:
            self.block_table[row, : len(table)] = -1

    # ---- prefix cache (manager.py:496-571) --------------------------------------------
    @staticmethod
    def get_prefix_cache_key(token_ids: Sequence[int]) -> str:
        """SHA-256 of the comma-joined token ids (manager.py:496-506)."""
        return hashlib.sha256(",".join(str(int(t)) for t in token_ids).encode()).hexdigest()

    def _longest_cached(self, token_ids: Sequence[int], max_blocks: int):
        for n in range(max_blocks, 0, -1):                       # longest block-aligned prefix first (:523-529)
            key = self.get_prefix_cache_key(token_ids[: n * BLOCK_SIZE])
            if key in self._prefix_cache:
                return key, self._prefix_cache[key]
        return None, None

    def lookup_prefix(self, token_ids: Sequence[int]) -> Optional[List[int]]:
        """Physical blocks of the longest cached block-aligned prefix of `token_ids`, or None (manager.py:508-531)."""
        if not self.enable_prefix_cache:
            return None
        _, blocks = self._longest_cached(token_ids, len(token_ids) // BLOCK_SIZE)
        return None if blocks is None else list(blocks)

    def cache_prefix(self, token_ids: Sequence[int], request_id: str) -> int:
        """Publish the full blocks of `request_id`'s prompt for reuse; returns the number of tokens cached
        (manager.py:533-571).  The tokens must have been written and committed.  The entry lives as long as
        a request is attached to it (the publisher and every request that adopted or re-published it)."""
        if not self.enable_prefix_cache:
            return 0
        n = len(token_ids) // BLOCK_SIZE
        if n == 0:
            return 0
        table = self._tables.get(request_id, [])
        if len(table) < n or self._tokens.get(request_id, 0) < n * BLOCK_SIZE or any(b < 0 for b in table[:n]):
            return 0                                              # (:559-561; also: evicted or unwritten blocks)
        key = self.get_prefix_cache_key(token_ids[: n * BLOCK_SIZE])
        if key not in self._prefix_cache:
            self._prefix_cache[key] = list(table[:n])
            self._prefix_ref_count[key] = 0
            for b in table[:n]:
                self._refs[b] += 1                                # the entry's own hold on its blocks
        if key not in self._req_keys[request_id]:
            self._req_keys[request_id].add(key)
            self._prefix_ref_count[key] += 1
        return n * BLOCK_SIZE

    def _adopt_prefix(self, request_id: str, token_ids: Sequence[int]) -> None:
        if len(token_ids) == 0:
            return
        key, blocks = self._longest_cached(token_ids, len(token_ids) // BLOCK_SIZE)
        if blocks is None:
            return
        blocks = blocks[: min((len(token_ids) - 1) // BLOCK_SIZE, self.max_blocks_per_seq)]
        if not blocks:
            return
        for b in blocks:
            self._refs[b] += 1
        self._tables[request_id] = list(blocks)
        self._tokens[request_id] = len(blocks) * BLOCK_SIZE
        self._req_keys[request_id].add(key)
        self._prefix_ref_count[key] += 1
        row = self._row[request_id]
        self.block_table[row, : len(blocks)] = torch.tensor(blocks, dtype=torch.int32)

    def _detach(self, key: str) -> None:
        self._prefix_ref_count[key] -= 1
        if self._prefix_ref_count[key] <= 0:                      # last attached request gone (:455-461)
            del self._prefix_ref_count[key]
            for b in self._prefix_cache.pop(key):
                self._drop_ref(b)

    # ---- sliding window (manager.py:577-617) -------------------------------------------
    def _evict_sliding_window(self, request_id: str) -> None:
        """Give up the blocks whose tokens all lie before `length - sliding_window`."""
        evictable_blocks = (self._tokens[request_id] - self.sliding_window) // BLOCK_SIZE      # (:588-596)
        done = self._evicted[request_id]
        if evictable_blocks <= done:
            return
        table = self._tables[request_id]
        for i in range(done, evictable_blocks):
            self._drop_ref(table[i])                              # shared blocks live on with their other holders
            table[i] = -1
        self._evicted[request_id] = evictable_blocks
        self.block_table[self._row[request_id], done:evictable_blocks] = -1

    def window_start(self, request_id: str) -> int:
        """Position of the first token whose block is still held (0 without eviction)."""
        return self._evicted.get(request_id, 0) * BLOCK_SIZE

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
