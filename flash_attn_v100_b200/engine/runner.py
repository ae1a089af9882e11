"""Static-batch generation: packed prompt prefill in chunks, then greedy decode steps replayed
from a CUDA graph.  (The reference's scheduler, flash_attn_llm/engine/scheduler.py:15-247, does block
accounting for continuous batching; this slice serves one fixed batch: 256 requests with 1024-token
prompts and 256 new tokens each is the shape it is measured on.)"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..kv_cache import PagedKVCache
from .model import Segments, TPDecoder


class GenerationRunner:
    def __init__(self, model: TPDecoder, max_batch: int, max_seq_len: int, use_cuda_graph: bool = True,
                 peer_collectives: bool = False):
        cfg = model.cfg
        self.model = model
        self.max_batch, self.max_seq_len = max_batch, max_seq_len
        self.max_blocks = (max_seq_len + 15) // 16
        self.kv = PagedKVCache(num_blocks=max_batch * self.max_blocks, num_layers=cfg.num_layers,
                               num_kv_heads=model.kl, head_dim=cfg.head_dim, max_batch=max_batch,
                               max_blocks_per_seq=self.max_blocks, device=model.device, dtype=model.attn_dtype)
        # The decode step is replayed from one CUDA graph on a single rank.  Under tensor parallelism it is a
        # chain of graphs with the NCCL collectives issued eagerly in between (NCCL calls are not captured),
        # or - with peer_collectives - again one CUDA graph, the collectives being the library's peer-memory
        # kernels inside it.
        self.use_cuda_graph = use_cuda_graph
        self._gather_off = 0
        if peer_collectives and model.world > 1:
            from ..comm import PeerCollectives
            import torch.distributed as dist
            rows = (max_batch * cfg.hidden_size * 2 + 255) // 256 * 256
            # four [max_batch, hidden] regions (the two row-parallel GEMM outputs, the residual stream and the
            # normed activations of the fused all-reduce + norm) and the greedy candidates behind them
            self._gather_off = 4 * rows
            model.comm = PeerCollectives(model.group if model.group is not None else dist.group.WORLD, model.device,
                                         4 * rows + model.world * max_batch * 8)
        self._side_stream = torch.cuda.Stream(device=model.device)   # decode runs here (one scratch workspace)
        # Under tensor parallelism prompt chunks are prefilled two at a time, each on its own stream and
        # advanced in turn from one all-reduce to the next, so that one chunk's NCCL all-reduce (134 MB per
        # 16 x 1024 tokens) overlaps the other chunk's compute.
        self._prefill_streams = [torch.cuda.Stream(device=model.device) for _ in range(2)] if model.world > 1 else []
        self._decode_cache = {}     # batch size -> (step graph(s), cur, slot, gathered): captured once, replayed by later calls

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, max_new_tokens: int, prefill_chunk: int = 32, logits_out: Optional[list] = None):
        """prompts [B, P] int64 (equal lengths); returns generated tokens [B, max_new_tokens] int64.
        `logits_out` (a list, eager mode only) receives this rank's logits of every step."""
        m, kv, dev = self.model, self.kv, self.model.device
        B, P = prompts.shape
        assert B <= self.max_batch and P + max_new_tokens <= self.max_seq_len
        ids = [f"r{i}" for i in range(B)]
        allocated = []
        try:
            rows = []
            for r in ids:
                rows.append(kv.allocate(r, P + max_new_tokens))   # blocks for the whole generation: the table is static
                allocated.append(r)
            # the captured decode graphs address rows 0..B-1 of the resident table: anything else (another user
            # of the cache holding rows, rows leaked by an earlier failure) must not go unnoticed
            if rows != list(range(B)):
                raise RuntimeError(f"generate() needs table rows 0..{B - 1} of the KV cache, got {rows}")
            return self._generate(prompts, max_new_tokens, prefill_chunk, logits_out, ids)
        finally:
            for r in reversed(allocated):       # rows and blocks return in the order the next call takes them
                kv.release(r)

    def _generate(self, prompts, max_new_tokens, prefill_chunk, logits_out, ids):
        m, kv, dev = self.model, self.kv, self.model.device
        B, P = prompts.shape
        table = kv.block_table[:B]
        out = torch.empty((B, max_new_tokens), dtype=torch.int64, device=dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        ev[0].record()
        # ---- prefill, `prefill_chunk` sequences per pass ----
        first = torch.empty(B, dtype=torch.int64, device=dev)

        def chunk_args(b0, b1):
            nb = b1 - b0
            return dict(token_ids=prompts[b0:b1].reshape(-1).to(dev),
                        positions=torch.arange(P, dtype=torch.int32, device=dev).repeat(nb), kv=kv,
                        block_table=table[b0:b1], slots=torch.zeros(nb, dtype=torch.int32, device=dev),
                        max_blocks=self.max_blocks,
                        cu_seqlens=(torch.arange(nb + 1, dtype=torch.int32, device=dev) * P), max_seqlen=P)

        chunks = [(b0, min(b0 + prefill_chunk, B)) for b0 in range(0, B, prefill_chunk)]
        group = len(self._prefill_streams) if (self._prefill_streams and logits_out is None) else 1
        main = torch.cuda.current_stream(dev)
        for g0 in range(0, len(chunks), group):
            part = chunks[g0:g0 + group]
            batches = [chunk_args(b0, b1) for b0, b1 in part]
            if len(part) == 1:
                hiddens = [m.forward(**batches[0])]
            else:
                streams = self._prefill_streams[:len(part)]
                for s_ in streams:
                    s_.wait_stream(main)
                hiddens = m.forward_overlapped(batches, streams)
                for s_ in streams:
                    main.wait_stream(s_)
            for (b0, b1), hidden in zip(part, hiddens):
                tok, lg = m.greedy_token(hidden)
                first[b0:b1] = tok
                if logits_out is not None:
                    logits_out.append(("prefill", b0, lg))
            del batches, hiddens
        for r in ids:
            kv.commit(r, P)
        out[:, 0] = first
        ev[1].record()
        # ---- decode ----
        cached = self._decode_cache.get(B) if (self.use_cuda_graph and logits_out is None) else None
        if cached is not None:
            graph, cur, slot, gathered = cached
        else:
            graph = None
            cur = torch.empty(B, dtype=torch.int64, device=dev)                    # token being fed
            slot = torch.empty(B, dtype=torch.int32, device=dev)                   # its cache slot
            if m.comm is not None:
                gathered = m.comm.view(self._gather_off, (m.world, B, 2), torch.float32)
            else:
                gathered = torch.empty((m.world, B, 2), dtype=torch.float32, device=dev)
        cur.copy_(first)
        slot.fill_(P)

        def step(seg=None):
            hidden = m.forward(cur, slot, kv, table, slot, self.max_blocks, seg=seg)
            st = {}

            def head():
                st["pair"], st["logits"] = m.greedy_local(hidden)

            def tail():
                cur.copy_(m.greedy_select(gathered))
                slot.add_(1)

            gather = lambda pair: m.greedy_gather(pair, gathered)
            if seg is None:
                head(); gather(st["pair"]); tail()
            else:
                seg.run(head)
                seg.collective(gather, st["pair"])
                seg.run(tail)
            if logits_out is not None:
                logits_out.append(("decode", 0, st["logits"]))

        n_steps = max_new_tokens - 1
        graphs_ok = self.use_cuda_graph and logits_out is None and (graph is not None or n_steps > 3)
        side = self._side_stream
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            done = 0
            if graphs_ok and graph is None:
                # first call for this batch size: a warm-up step, then the capture.  One graph for the whole
                # step on a single rank; under tensor parallelism a chain of graphs with the NCCL collectives
                # in between (every captured segment is run right after its capture, so that step is real).
                step(); out[:, 1] = cur; done = 1
                if m.world == 1 or m.comm is not None:
                    graph = torch.cuda.CUDAGraph()
                    # (thread-local capture mode: the NCCL watchdog thread of the process group may poll events)
                    with torch.cuda.graph(graph, stream=side, capture_error_mode="thread_local"):
                        step()
                else:
                    graph = Segments(capture=True, stream=side)
                    step(graph); out[:, 2] = cur; done = 2
                self._decode_cache[B] = (graph, cur, slot, gathered)
            if graphs_ok:
                for i in range(done, n_steps):
                    graph.replay()
                    out[:, i + 1] = cur
            else:
                for i in range(n_steps):
                    step()
                    out[:, i + 1] = cur
        torch.cuda.current_stream(dev).wait_stream(side)
        ev[2].record()
        self._events = ev
        for r in ids:
            kv.commit(r, max_new_tokens - 1)
        # device-side conditions recorded by the kernels of this call (a block-table entry outside the pool, a
        # bounded wait that ran out, a collective that gave up on a rank) surface here, not as wrong tokens
        from .. import ops
        torch.cuda.synchronize(dev)
        ops.check_async_errors(dev)
        ops.check_prefill_errors(dev)
        if m.comm is not None:
            m.comm.check()
        return out

    def close(self):
        """Release the peer-memory buffers (all ranks call it; no-op without peer collectives)."""
        self._decode_cache.clear()
        if self.model.comm is not None:
            self.model.comm.close()
            self.model.comm = None

    def last_timing_ms(self):
        """(prefill ms, decode ms) of the last generate() call; synchronises."""
        torch.cuda.synchronize(self.model.device)
        return self._events[0].elapsed_time(self._events[1]), self._events[1].elapsed_time(self._events[2])
