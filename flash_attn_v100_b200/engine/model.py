"""Tensor-parallel Qwen3-style decoder on the paged attention operators.

Standard pre-norm block: x += o_proj(attn(rope(qk_norm(qkv(ln1(x)))))); x += down(silu(gate) * up)(ln2(x)).
(The reference's layer, flash_attn_llm/models/decoder_layer.py:53-129, applies post_attention_layernorm to
the attention output and again before the MLP and scales the embeddings by sqrt(hidden); those are
quirks of that code, not of the model family, and are not reproduced.)

Per rank (tensor_parallel.py:451-457): H_Q/ws query heads and H_KV/ws KV heads, column-parallel qkv and
gate/up, row-parallel o and down followed by a sum all-reduce over NCCL
(flash_attn_llm/kernels/linear.py:200-207); attention itself needs no communication.  GEMMs go to
cuBLAS through torch.matmul; everything between them is this library's kernels.  Activations are
bf16; the attention operators run in fp16 (q, k, v are cast by the fused QK-norm kernel).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _lib, ops
from .config import ModelConfig


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


class TPDecoder:
    def __init__(self, cfg: ModelConfig, weights, rank: int = 0, world: int = 1, group=None, device="cuda"):
        cfg.validate(world)
        self.cfg, self.w, self.rank, self.world, self.group = cfg, weights, rank, world, group
        # Optional `comm.PeerCollectives`: when set, the decode step sums its row-parallel outputs and gathers
        # the greedy candidates with the library's peer-memory kernels (capturable into the step's CUDA graph)
        # instead of NCCL calls.  Prefill keeps NCCL (large messages, not replayed from a graph).
        self.comm = None
        # one launch for QK-norm + cast + rotary + cache append (False: the norm kernel and the rotary/append
        # kernel one after the other; same values, kept for the parity test of the fused kernel)
        self.fused_qkv = True
        # the decode step's all-reduces take the residual add and the RMS norm that follow them into the same
        # kernel (False: all-reduce, then the add + norm kernel; same values, kept for the parity test)
        self.fused_norm = True
        # element type of q / k / v and of the KV pages: fp16 (the reference's operators) or bfloat16 (the
        # library's *_bf16 twins: the activations' own type, no cast and no fp16 range limit); the KV cache
        # handed to forward() must hold the same type
        self.attn_dtype = torch.float16
        self.device = torch.device(device)
        self.ql = cfg.num_heads // world
        self.kl = cfg.num_kv_heads // world
        self.il = cfg.intermediate_size // world
        self.vl = cfg.vocab_size // world
        self.lib = _lib.load()
        self.inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, dtype=torch.float32,
                                                               device=self.device) / cfg.head_dim))

    # ---- small wrappers over the C ABI -------------------------------------------------
    def _stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)

    def _add_rmsnorm(self, x, delta, w):
        out = torch.empty_like(x)
        _lib.check(self.lib.fa_add_rmsnorm_bf16(_p(x), _p(delta) if delta is not None else None, _p(w), _p(out),
                                                x.size(0), x.size(1), self.cfg.rms_norm_eps, self._stream()))
        return out

    def _qk_norm_split(self, qkv, lw):
        T, D = qkv.size(0), self.cfg.head_dim
        q = torch.empty((T, self.ql, D), dtype=torch.float16, device=self.device)
        k = torch.empty((T, self.kl, D), dtype=torch.float16, device=self.device)
        v = torch.empty((T, self.kl, D), dtype=torch.float16, device=self.device)
        qn = _p(lw["qn"]) if self.cfg.qk_norm else None
        kn = _p(lw["kn"]) if self.cfg.qk_norm else None
        _lib.check(self.lib.fa_qk_norm_split_f16(_p(qkv), qn, kn, _p(q), _p(k), _p(v), T, self.ql, self.kl, D,
                                                 self.cfg.rms_norm_eps, self._stream()))
        return q, k, v

    def _qkv_rope_append(self, qkv, lw, cos, sin, k_pool, v_pool, block_table, slots, max_blocks, cu_seqlens):
        """Per-head QK-norm, cast to fp16, rotary embedding and the append of k / v to the pages in ONE launch
        (the two-kernel path is `_qk_norm_split` + `ops.rope_append_paged_fp16`; same values).  Returns q_rot
        and, for packed prompts, the rotated k and v the prefill attention reads."""
        T, D = qkv.size(0), self.cfg.head_dim
        prefill = cu_seqlens is not None
        if k_pool.dtype != self.attn_dtype:
            raise RuntimeError(f"the KV cache holds {k_pool.dtype}, the model's attn_dtype is {self.attn_dtype}")
        q = torch.empty((T, self.ql, D), dtype=self.attn_dtype, device=self.device)
        k = torch.empty((T, self.kl, D), dtype=self.attn_dtype, device=self.device) if prefill else None
        v = torch.empty((T, self.kl, D), dtype=self.attn_dtype, device=self.device) if prefill else None
        batch = cu_seqlens.numel() - 1 if prefill else T
        if block_table.stride(1) != 1 or block_table.stride(0) != max_blocks or batch * max_blocks > block_table.numel():
            raise RuntimeError("block_table rows must be contiguous with stride max_blocks")
        qn = _p(lw["qn"]) if self.cfg.qk_norm else None
        kn = _p(lw["kn"]) if self.cfg.qk_norm else None
        entry = self.lib.fa_qkv_rope_append_bf16 if self.attn_dtype == torch.bfloat16 else self.lib.fa_qkv_rope_append_f16
        _lib.check(entry(
            _p(qkv), qn, kn, _p(cos), _p(sin), _p(q), _p(k) if prefill else None, _p(v) if prefill else None,
            _p(k_pool), _p(v_pool), _p(block_table), _p(slots), _p(cu_seqlens) if prefill else None, T, batch,
            self.ql, self.kl, D, self.cfg.rms_norm_eps, k_pool.size(0), max_blocks, self._stream()))
        return q, k, v

    def _silu_mul(self, gu):
        out = torch.empty((gu.size(0), self.il), dtype=gu.dtype, device=self.device)
        _lib.check(self.lib.fa_silu_mul_bf16(_p(gu), _p(out), gu.size(0), self.il, self._stream()))
        return out

    def _to_bf16(self, x16):
        out = torch.empty(x16.shape, dtype=torch.bfloat16, device=self.device)
        _lib.check(self.lib.fa_half_to_bf16(_p(x16), _p(out), x16.numel(), self._stream()))
        return out

    def _all_reduce(self, t):
        if self.world > 1:
            torch.distributed.all_reduce(t, group=self.group)
        return t

    def _peer_rows(self, T):
        """Two [T, hidden] bf16 views of the peer buffer (attention and MLP outputs), or None when the step
        does not go through the peer collectives."""
        c = self.comm
        if c is None or self.world == 1:
            return None
        nbytes = (T * self.cfg.hidden_size * 2 + 255) // 256 * 256
        if 2 * nbytes > c.data_bytes or (T * self.cfg.hidden_size) % (8 * self.world) != 0:
            return None
        views = [c.view(i * nbytes, (T, self.cfg.hidden_size), torch.bfloat16) for i in range(2)]
        # with room for two more regions (residual stream and normed activations) and whole rows per rank, the
        # all-reduces also do the residual add and the norm
        if self.fused_norm and 4 * nbytes <= c.data_bytes and T % self.world == 0 and self.cfg.hidden_size <= 16384:
            views += [c.view(i * nbytes, (T, self.cfg.hidden_size), torch.bfloat16) for i in (2, 3)]
        return tuple(views)

    def rope_tables(self, positions):
        """fp32 cos/sin [T, D] exactly as the reference computes them (rope.py:228-266)."""
        freqs = torch.outer(positions.float(), self.inv_freq)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos().contiguous(), emb.sin().contiguous()

    # ---- one decoder stack pass -------------------------------------------------------
    def _stages(self, token_ids, positions, kv, block_table, slots, max_blocks, cu_seqlens, max_seqlen,
                seq_lens_after):
        """The pass as closures over a shared state dict: `first`, per layer (`attention_half`, `mlp_half`),
        `last`.  After `attention_half` the row-parallel output st["o"] and after `mlp_half` st["delta"]
        still have to be summed over the ranks, unless st["peer"] is set: then the halves have already done
        it with the peer-memory all-reduce."""
        cfg = self.cfg
        prefill = cu_seqlens is not None
        st = {"delta": None}
        peer = None if prefill else self._peer_rows(token_ids.numel())
        st["peer"] = peer
        fused = peer is not None and len(peer) == 4    # peer[2]: residual stream x, peer[3]: normed activations h
        n_layers = len(self.w["layers"])

        def first():
            if fused:
                st["x"] = torch.index_select(self.w["embed"], 0, token_ids, out=peer[2])
                st["h"] = self._add_rmsnorm(st["x"], None, self.w["layers"][0]["ln1"])
            else:
                st["x"] = self.w["embed"][token_ids]                      # [T, hidden] bf16
            st["cos"], st["sin"] = self.rope_tables(positions)
            # decode: lengths including the new token (derived here so that a replayed step recomputes them)
            st["lens"] = seq_lens_after if (prefill or seq_lens_after is not None) else slots + 1

        layers = []
        for l, lw in enumerate(self.w["layers"]):
            def attention_half(l=l, lw=lw):
                x = st["x"]
                # x += delta (previous MLP); h = ln1(x) — done by the previous all-reduce on the fused path
                h = st["h"] if fused else self._add_rmsnorm(x, st["delta"], lw["ln1"])
                qkv = h @ lw["wqkv"].t()
                if self.fused_qkv:
                    q_rot, k_rot, v = self._qkv_rope_append(qkv, lw, st["cos"], st["sin"], kv.k_pools[l], kv.v_pools[l],
                                                            block_table, slots, max_blocks, cu_seqlens)
                    if not prefill:
                        q_rot = q_rot.unsqueeze(2)
                else:
                    q, k, v = self._qk_norm_split(qkv, lw)
                    if prefill:
                        q_rot, k_rot = ops.rope_append_paged_fp16(q, k, v, st["cos"], st["sin"], kv.k_pools[l],
                                                                  kv.v_pools[l], block_table, slots, max_blocks,
                                                                  cu_seqlens=cu_seqlens, return_k=True)
                    else:
                        q_rot = ops.rope_append_paged_fp16(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), st["cos"],
                                                           st["sin"], kv.k_pools[l], kv.v_pools[l], block_table, slots,
                                                           max_blocks)
                if self.attn_dtype == torch.bfloat16:
                    if not self.fused_qkv:
                        raise RuntimeError("attn_dtype bfloat16 needs fused_qkv (the split kernels cast to fp16)")
                    if prefill:
                        attn = ops.forward_varlen_prefill_bf16(q_rot, k_rot, v, cu_seqlens, max_seqlen, True)
                    else:
                        attn = ops.forward_paged_decode_gqa_bf16(q_rot, kv.k_pools[l], kv.v_pools[l], block_table,
                                                                 st["lens"], max_blocks)
                elif prefill:
                    attn = ops.forward_varlen_prefill_fp16(q_rot, k_rot, v, cu_seqlens, max_seqlen, True,
                                                           out_dtype=torch.bfloat16)
                else:
                    attn = ops.forward_paged_decode_gqa_fp16(q_rot, kv.k_pools[l], kv.v_pools[l], block_table,
                                                             st["lens"], max_blocks, out_dtype=torch.bfloat16)
                a = attn.reshape(x.size(0), self.ql * cfg.head_dim)   # bf16 straight from the attention epilogue
                if peer is None:
                    st["o"] = a @ lw["wo"].t()
                elif fused:                # GEMM into the peer buffer; sum over the ranks, x += sum, h = ln2(x)
                    st["h"] = self.comm.all_reduce_add_rmsnorm_(torch.mm(a, lw["wo"].t(), out=peer[0]), peer[2],
                                                                peer[3], lw["ln2"], cfg.rms_norm_eps)
                else:                      # GEMM straight into the peer buffer, summed in place over the ranks
                    st["o"] = self.comm.all_reduce_(torch.mm(a, lw["wo"].t(), out=peer[0]))

            def mlp_half(l=l, lw=lw):
                # x += attention; h = ln2(x) — done by the attention half's all-reduce on the fused path
                h = st["h"] if fused else self._add_rmsnorm(st["x"], st["o"], lw["ln2"])
                gu = h @ lw["wgu"].t()
                if peer is None:
                    st["delta"] = self._silu_mul(gu) @ lw["wd"].t()
                elif fused:                # ... x += sum, h = the next layer's ln1(x), or the final norm
                    w_next = self.w["layers"][l + 1]["ln1"] if l + 1 < n_layers else self.w["final_ln"]
                    st["h"] = self.comm.all_reduce_add_rmsnorm_(torch.mm(self._silu_mul(gu), lw["wd"].t(), out=peer[1]),
                                                                peer[2], peer[3], w_next, cfg.rms_norm_eps)
                else:
                    st["delta"] = self.comm.all_reduce_(torch.mm(self._silu_mul(gu), lw["wd"].t(), out=peer[1]))

            layers.append((attention_half, mlp_half))

        def last():
            if fused:                      # the last all-reduce has applied the final norm
                st["hidden"] = st["h"]
                return
            if prefill:
                idx = (cu_seqlens[1:] - 1).long()
                x_last, d_last = st["x"][idx].contiguous(), st["delta"][idx].contiguous()
            else:
                x_last, d_last = st["x"], st["delta"]
            st["hidden"] = self._add_rmsnorm(x_last, d_last, self.w["final_ln"])   # final norm of (x + last MLP)

        return st, first, layers, last

    def forward(self, token_ids, positions, kv, block_table, slots, max_blocks, *, cu_seqlens=None, max_seqlen=0,
                seq_lens_after=None, seg=None):
        """token_ids [T] int64; positions [T] int32 (rotary position of every token).
        Prefill (cu_seqlens given): packed prompts, `slots` [batch] = first cache slot per sequence; returns the
        hidden state of the last token of every sequence.  Decode: one token per sequence, `slots` [B] = slot of
        the new token, `seq_lens_after` [B] = lengths including it (default: slots + 1); returns [B, hidden].
        `seg` (see `Segments`) receives the compute between two collectives as one unit, so that a decode
        step can be replayed as a chain of CUDA graphs with the NCCL calls in between."""
        seg = seg or Segments(capture=False)
        st, first, layers, last = self._stages(token_ids, positions, kv, block_table, slots, max_blocks, cu_seqlens,
                                               max_seqlen, seq_lens_after)
        seg.run(first)
        for attention_half, mlp_half in layers:
            seg.run(attention_half)
            if st["peer"] is None:
                seg.collective(self._all_reduce, st["o"])
            seg.run(mlp_half)
            if st["peer"] is None:
                seg.collective(self._all_reduce, st["delta"])
        seg.run(last)
        return st["hidden"]

    def forward_stages(self, token_ids, positions, kv, block_table, slots, max_blocks, *, cu_seqlens=None,
                       max_seqlen=0, seq_lens_after=None):
        """The same pass as a generator: it yields every tensor that has to be summed over the ranks (the
        caller all-reduces it in place before resuming) and finally returns the hidden state through
        StopIteration.  Several passes over independent token batches can thus be advanced in turn, each on
        its own stream, so that one batch's all-reduce overlaps the other's compute (`forward_overlapped`)."""
        st, first, layers, last = self._stages(token_ids, positions, kv, block_table, slots, max_blocks, cu_seqlens,
                                               max_seqlen, seq_lens_after)
        first()
        for attention_half, mlp_half in layers:
            attention_half()
            if st["peer"] is None:
                yield st["o"]
            mlp_half()
            if st["peer"] is None:
                yield st["delta"]
        last()
        return st["hidden"]

    def forward_overlapped(self, batches, streams):
        """Run one pass per entry of `batches` (dicts of forward() arguments), entry i on streams[i], advancing
        them in turn from one collective to the next; returns the hidden states in order.  The caller orders the
        streams against whatever produced the inputs and consumes the outputs."""
        gens = [self.forward_stages(**b) for b in batches]
        out = [None] * len(gens)
        live = list(range(len(gens)))
        while live:
            for i in list(live):
                with torch.cuda.stream(streams[i]):
                    try:
                        t = next(gens[i])
                        self._all_reduce(t)
                    except StopIteration as done:
                        out[i] = done.value
                        live.remove(i)
        return out

    def greedy_local(self, hidden):
        """This rank's best (value, index) per sequence over its vocabulary shard, and the shard's logits."""
        logits = (hidden @ self.w["lm_head"].t()).float()                 # [B, vocab/world]
        val, idx = logits.max(dim=-1)
        pair = torch.stack([val, (idx + self.rank * self.vl).float()], dim=-1).contiguous()   # indices < 2^24: exact
        return pair, logits

    def greedy_gather(self, pair, out=None):
        """All-gather of the per-rank (value, index) pairs into `out` [world, B, 2] (allocated if None)."""
        if out is None:
            out = torch.empty((self.world,) + pair.shape, dtype=pair.dtype, device=pair.device)
        if self.world == 1:
            out[0].copy_(pair)
        elif self.comm is not None and self.comm.owns(out):
            self.comm.all_gather_into(out, pair)
        else:
            torch.distributed.all_gather_into_tensor(out, pair, group=self.group)
        return out

    @staticmethod
    def greedy_select(gathered):
        best = gathered[..., 0].argmax(dim=0)                              # first maximum = lowest rank on ties
        return gathered[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).long()

    def greedy_token(self, hidden):
        """argmax over the vocabulary sharded across ranks: local max / argmax, then an all-gather of the
        (value, index) pairs (the reference's `allgather`, parallel/tensor_parallel.py:172-190)."""
        pair, logits = self.greedy_local(hidden)
        return self.greedy_select(self.greedy_gather(pair)), logits


class Segments:
    """Runs a step as alternating compute segments and collectives.  With capture=True every compute
    segment is captured into its own CUDA graph (sharing one memory pool) and replayed at once, the
    collectives run eagerly in between; `replay()` then repeats the whole chain.  NCCL calls are never
    captured."""

    def __init__(self, capture: bool, stream=None):
        self.capture, self.stream, self.items, self.pool = capture, stream, [], None

    def run(self, fn):
        if not self.capture:
            fn()
            return
        g = torch.cuda.CUDAGraph()
        # thread-local capture mode: the NCCL watchdog thread may poll events of the collectives issued
        # between two segments while the next segment is being captured
        with torch.cuda.graph(g, pool=self.pool, stream=self.stream, capture_error_mode="thread_local"):
            fn()
        self.pool = g.pool()
        self.items.append(g)
        g.replay()                      # capture records only: run it, the following collective needs the data

    def collective(self, fn, tensor):
        out = fn(tensor)
        if self.capture:
            self.items.append((fn, tensor))
        return out

    def replay(self):
        for it in self.items:
            if isinstance(it, tuple):
                it[0](it[1])
            else:
                it.replay()
