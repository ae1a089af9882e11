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

    def rope_tables(self, positions):
        """fp32 cos/sin [T, D] exactly as the reference computes them (rope.py:228-266)."""
        freqs = torch.outer(positions.float(), self.inv_freq)
        emb = torch.cat([freqs, freqs], dim=-1)
        return emb.cos().contiguous(), emb.sin().contiguous()

    # ---- one decoder stack pass -------------------------------------------------------
    def forward(self, token_ids, positions, kv, block_table, slots, max_blocks, *, cu_seqlens=None, max_seqlen=0,
                seq_lens_after=None):
        """token_ids [T] int64; positions [T] int32 (rotary position of every token).
        Prefill (cu_seqlens given): packed prompts, `slots` [batch] = first cache slot per sequence; returns the
        hidden state of the last token of every sequence.  Decode: one token per sequence, `slots` [B] = slot of
        the new token, `seq_lens_after` [B] = lengths including it; returns [B, hidden]."""
        cfg = self.cfg
        x = self.w["embed"][token_ids]                                   # [T, hidden] bf16
        cos, sin = self.rope_tables(positions)
        delta = None
        prefill = cu_seqlens is not None
        for l, lw in enumerate(self.w["layers"]):
            h = self._add_rmsnorm(x, delta, lw["ln1"])                    # x += delta (previous MLP); h = ln1(x)
            qkv = h @ lw["wqkv"].t()
            q, k, v = self._qk_norm_split(qkv, lw)
            if prefill:
                q_rot, k_rot = ops.rope_append_paged_fp16(q, k, v, cos, sin, kv.k_pools[l], kv.v_pools[l], block_table,
                                                          slots, max_blocks, cu_seqlens=cu_seqlens, return_k=True)
                attn = ops.forward_varlen_prefill_fp16(q_rot, k_rot, v, cu_seqlens, max_seqlen, True)
            else:
                q_rot = ops.rope_append_paged_fp16(q.unsqueeze(2), k.unsqueeze(2), v.unsqueeze(2), cos, sin,
                                                   kv.k_pools[l], kv.v_pools[l], block_table, slots, max_blocks)
                attn = ops.forward_paged_decode_gqa_fp16(q_rot, kv.k_pools[l], kv.v_pools[l], block_table,
                                                         seq_lens_after, max_blocks)
            a = self._to_bf16(attn.reshape(x.size(0), self.ql * cfg.head_dim))
            o = self._all_reduce(a @ lw["wo"].t())
            h = self._add_rmsnorm(x, o, lw["ln2"])                        # x += attention; h = ln2(x)
            gu = h @ lw["wgu"].t()
            delta = self._all_reduce(self._silu_mul(gu) @ lw["wd"].t())
        if prefill:
            last = (cu_seqlens[1:] - 1).long()
            x_last, d_last = x[last].contiguous(), delta[last].contiguous()
        else:
            x_last, d_last = x, delta
        return self._add_rmsnorm(x_last, d_last, self.w["final_ln"])      # final norm of (x + last MLP)

    def greedy_token(self, hidden):
        """argmax over the vocabulary sharded across ranks: local max / argmax, then an all-gather of the
        (value, index) pairs (the reference's `allgather`, parallel/tensor_parallel.py:172-190)."""
        logits = (hidden @ self.w["lm_head"].t()).float()                 # [B, vocab/world]
        val, idx = logits.max(dim=-1)
        idx = idx + self.rank * self.vl
        if self.world > 1:
            pair = torch.stack([val, idx.float()], dim=-1).contiguous()   # indices < 2^24 are exact in fp32
            gathered = torch.empty((self.world,) + pair.shape, dtype=pair.dtype, device=pair.device)
            torch.distributed.all_gather_into_tensor(gathered, pair, group=self.group)
            best = gathered[..., 0].argmax(dim=0)                          # first maximum = lowest rank on ties
            idx = gathered[..., 1].gather(0, best.unsqueeze(0)).squeeze(0).long()
        return idx, logits
