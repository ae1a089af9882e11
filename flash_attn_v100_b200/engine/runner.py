"""Static-batch generation: packed prompt prefill in chunks, then greedy decode steps replayed
from a CUDA graph.  (The reference's scheduler, flash_attn_llm/engine/scheduler.py:15-247, does block
accounting for continuous batching; this slice serves one fixed batch, the shape of BASELINE
configuration 5.)"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kv_cache import PagedKVCache
from .model import TPDecoder


class GenerationRunner:
    def __init__(self, model: TPDecoder, max_batch: int, max_seq_len: int, use_cuda_graph: bool = True):
        cfg = model.cfg
        self.model = model
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.max_blocks = (max_seq_len + 15) // 16
        self.kv = PagedKVCache(num_blocks=max_batch * self.max_blocks, num_layers=cfg.num_layers,
                               num_kv_heads=model.kl, head_dim=cfg.head_dim, max_batch=max_batch,
                               max_blocks_per_seq=self.max_blocks, device=model.device)
        # The decode step is replayed from one CUDA graph on a single rank.  With tensor parallelism the
        # step contains NCCL collectives; capturing them is left out (steps run eagerly) until the step is
        # split into graph segments between the collectives.
        self.use_cuda_graph = use_cuda_graph and model.world == 1
        self._graph = None

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, prefill_chunk: int = 32, logits_out: Optional[list] = None):
        """prompts [B, P] int64 (equal lengths); returns generated tokens [B, max_new_tokens] int64.
        `logits_out` (a list, eager mode only) receives this rank's logits of every step."""
        m, kv, dev = self.model, self.kv, self.model.device
        B, P = prompts.shape
        assert B <= self.max_batch and P + max_new_tokens <= self.max_seq_len
        ids = [f"r{i}" for i in range(B)]
        for r in ids:
            kv.allocate(r, P + max_new_tokens)          # blocks for the whole generation: the table is static
        table = kv.block_table[:B]
        out = torch.empty((B, max_new_tokens), dtype=torch.int64, device=dev)
        # ---- prefill, `prefill_chunk` sequences per pass ----
        first = torch.empty(B, dtype=torch.int64, device=dev)
        for b0 in range(0, B, prefill_chunk):
            b1 = min(b0 + prefill_chunk, B)
            nb = b1 - b0
            toks = prompts[b0:b1].reshape(-1).to(dev)
            cu = (torch.arange(nb + 1, dtype=torch.int32, device=dev) * P)
            pos = torch.arange(P, dtype=torch.int32, device=dev).repeat(nb)
            slots = torch.zeros(nb, dtype=torch.int32, device=dev)
            hidden = m.forward(toks, pos, kv, table[b0:b1], slots, self.max_blocks, cu_seqlens=cu, max_seqlen=P)
            tok, lg = m.greedy_token(hidden)
            first[b0:b1] = tok
            if logits_out is not None:
                logits_out.append(("prefill", b0, lg))
        for r in ids:
            kv.commit(r, P)
        out[:, 0] = first
        # ---- decode ----
        cur = first.clone()
        slot = torch.full((B,), P, dtype=torch.int32, device=dev)        # slot of the token being fed

        def step():
            hidden = m.forward(cur, slot, kv, table, slot, self.max_blocks, seq_lens_after=slot + 1)
            nxt, lg = m.greedy_token(hidden)
            if logits_out is not None:
                logits_out.append(("decode", 0, lg))
            cur.copy_(nxt)
            slot.add_(1)

        n_steps = max_new_tokens - 1
        if self.use_cuda_graph and n_steps > 2 and logits_out is None:
            # warm up on a side stream (allocator, cuBLAS workspaces, NCCL), restore state, capture, replay
            saved_cur, saved_slot = cur.clone(), slot.clone()
            s = torch.cuda.Stream(device=dev)
            s.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(s):
                step()
            torch.cuda.current_stream(dev).wait_stream(s)
            cur.copy_(saved_cur); slot.copy_(saved_slot)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=s):     # same stream as the warm-up: same scratch buffers
                step()
            cur.copy_(saved_cur); slot.copy_(saved_slot)
            for i in range(n_steps):
                graph.replay()
                out[:, i + 1] = cur
            self._graph = graph
        else:
            for i in range(n_steps):
                step()
                out[:, i + 1] = cur
        for r in ids:
            kv.commit(r, max_new_tokens - 1)
            kv.release(r)
        return out
