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
