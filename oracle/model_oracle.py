"""CPU/eager PyTorch restatement of the decoder block for engine parity.  TEST INFRASTRUCTURE ONLY.

A plain single-device, full-weight, fp32 evaluation of the same standard pre-norm Qwen3-style block the
engine implements (RMSNorm: flash_attn_llm/models/norm.py:25-33; QK-norm + rotary + causal attention:
flash_attn_llm/models/attention.py:191-276 with rope.py:302-348; SwiGLU: flash_attn_llm/models/mlp.py:27;
greedy loop: flash_attn_llm/models/causal_lm.py:316-374), recomputing the whole sequence every step
(no cache).  Weights are the engine's own seeded full matrices.
"""
from __future__ import annotations

import torch

from flash_attn_v100_b200.engine.weights import make_full_globals, make_full_layer


def rmsnorm(x, w, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)) * w.float()


def rotate_half(x):
    h = x.shape[-1] // 2
    return torch.cat((-x[..., h:], x[..., :h]), dim=-1)


@torch.no_grad()
def forward_logits(cfg, seed, tokens, gen_device="cpu"):
    """tokens [B, S] -> fp32 logits [B, S, vocab] of the full model (fp32 math on bf16-valued weights)."""
    B, S = tokens.shape
    D, HQ, HKV = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    glob = make_full_globals(cfg, seed, gen_device)
    x = glob["embed"].float()[tokens]
    pos = torch.arange(S, dtype=torch.float32)
    inv_freq = 1.0 / (cfg.rope_theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    emb = torch.cat([torch.outer(pos, inv_freq)] * 2, dim=-1)
    cos, sin = emb.cos()[None, None], emb.sin()[None, None]
    mask = torch.triu(torch.ones(S, S, dtype=torch.bool), diagonal=1)
    for l in range(cfg.num_layers):
        w = {k: v.float() for k, v in make_full_layer(cfg, l, seed, gen_device).items()}
        h = rmsnorm(x, w["ln1"], cfg.rms_norm_eps)
        q = (h @ w["wq"].t()).view(B, S, HQ, D).transpose(1, 2)
        k = (h @ w["wk"].t()).view(B, S, HKV, D).transpose(1, 2)
        v = (h @ w["wv"].t()).view(B, S, HKV, D).transpose(1, 2)
        if cfg.qk_norm:
            q = rmsnorm(q, w["qn"], cfg.rms_norm_eps)
            k = rmsnorm(k, w["kn"], cfg.rms_norm_eps)
        q = q * cos + rotate_half(q) * sin
        k = k * cos + rotate_half(k) * sin
        k = k.repeat_interleave(HQ // HKV, dim=1)
        v = v.repeat_interleave(HQ // HKV, dim=1)
        s = (q @ k.transpose(-1, -2)) / (D ** 0.5)
        s = s.masked_fill(mask, float("-inf"))
        a = torch.softmax(s, dim=-1) @ v
        x = x + a.transpose(1, 2).reshape(B, S, HQ * D) @ w["wo"].t()
        h = rmsnorm(x, w["ln2"], cfg.rms_norm_eps)
        x = x + (torch.nn.functional.silu(h @ w["wg"].t()) * (h @ w["wu"].t())) @ w["wd"].t()
    x = rmsnorm(x, glob["final_ln"], cfg.rms_norm_eps)
    return x @ glob["lm_head"].float().t()


@torch.no_grad()
def greedy_generate(cfg, seed, prompts, max_new_tokens):
    """Greedy continuation [B, max_new_tokens]; also returns the logits that chose every token."""
    toks = prompts.clone()
    outs, all_logits = [], []
    for _ in range(max_new_tokens):
        logits = forward_logits(cfg, seed, toks)[:, -1]
        nxt = logits.argmax(-1)
        outs.append(nxt)
        all_logits.append(logits)
        toks = torch.cat([toks, nxt[:, None]], dim=1)
    return torch.stack(outs, dim=1), torch.stack(all_logits, dim=1)
