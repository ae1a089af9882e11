"""Seeded synthetic inputs with the shapes and distributions of the benchmark
configurations (no dataset is involved anywhere on this path)."""
from __future__ import annotations

import torch

PAGE = 16


def make_paged_tables(B: int, min_len: int, max_len: int, seed: int = 0):
    """seq_lens uniform int in [min_len, max_len]; a pool of sum(ceil(len/16)) pages;
    block_table rows filled from one seeded random permutation of the pool, -1 padded."""
    g = torch.Generator().manual_seed(seed)
    seq_lens = torch.randint(min_len, max_len + 1, (B,), generator=g, dtype=torch.int32)
    pages = (seq_lens + PAGE - 1) // PAGE
    n_pages = int(pages.sum())
    perm = torch.randperm(n_pages, generator=g).to(torch.int32)
    max_blocks = max(int(pages.max()), 1)
    block_table = torch.full((B, max_blocks), -1, dtype=torch.int32)
    cur = 0
    for b in range(B):
        n = int(pages[b])
        block_table[b, :n] = perm[cur:cur + n]
        cur += n
    return dict(seq_lens=seq_lens, block_table=block_table, n_pages=n_pages, max_num_blocks=max_blocks, generator=g)


def make_paged_decode_batch(B: int, H_Q: int, H_KV: int, D: int, min_len: int, max_len: int,
                            table_seed: int = 0, value_seed: int = 0, pin: bool = False):
    """A whole paged-decode batch on the HOST, drawn from seeded CPU generators so that every consumer
    (a GPU run, a CPU run of the same workload) sees identical tensors: q [B,H_Q,1,D] and the K / V pools
    [pages,H_KV,16,D] as fp16 N(0,1), plus the tables of `make_paged_tables(B, min_len, max_len, table_seed)`."""
    t = make_paged_tables(B, min_len, max_len, table_seed)
    g = torch.Generator().manual_seed(1_000_003 * (value_seed + 1))
    q = torch.randn(B, H_Q, 1, D, generator=g).half()
    n_pages = t["n_pages"]
    k_cache = torch.empty(n_pages, H_KV, PAGE, D, dtype=torch.float16, pin_memory=pin)
    v_cache = torch.empty(n_pages, H_KV, PAGE, D, dtype=torch.float16, pin_memory=pin)
    chunk = 4096
    for s in range(0, n_pages, chunk):
        e = min(s + chunk, n_pages)
        k_cache[s:e] = torch.randn(e - s, H_KV, PAGE, D, generator=g).half()
        v_cache[s:e] = torch.randn(e - s, H_KV, PAGE, D, generator=g).half()
    return dict(q=q, k_cache=k_cache, v_cache=v_cache, block_table=t["block_table"], seq_lens=t["seq_lens"],
                n_pages=n_pages, max_num_blocks=t["max_num_blocks"])
