"""Seeded random-initialised weights, generated full-size and sliced per tensor-parallel rank.

Sharding follows the reference's rules (flash_attn_llm/parallel/tensor_parallel.py:129-146
`chunk(tp_size, dim)[rank]`; shard specs flash_attn_llm/weights/mapper.py:149-184): q/k/v/gate/up are
column-parallel (output rows split; q and k/v by head, so that rank r owns KV heads
[r*H_KV/ws, ...) and the matching query heads, tensor_parallel.py:451-457), o/down are row-parallel
(input columns split), embeddings replicated, the LM head split over the vocabulary.
Every rank draws the same full matrix from the same seed and keeps its slice, so any tensor-parallel
size reproduces the same model.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from .config import ModelConfig


def _randn(shape, gen, std, device, dtype):
    return (torch.randn(shape, generator=gen, device=gen.device, dtype=torch.float32) * std).to(dtype).to(device)


def make_full_layer(cfg: ModelConfig, layer: int, seed: int, gen_device, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=gen_device).manual_seed(seed * 100003 + layer)
    H, D = cfg.hidden_size, cfg.head_dim
    return {
        "wq": _randn((cfg.num_heads * D, H), g, cfg.init_std, gen_device, dtype),
        "wk": _randn((cfg.num_kv_heads * D, H), g, cfg.init_std, gen_device, dtype),
        "wv": _randn((cfg.num_kv_heads * D, H), g, cfg.init_std, gen_device, dtype),
        "wo": _randn((H, cfg.num_heads * D), g, cfg.init_std, gen_device, dtype),
        "wg": _randn((cfg.intermediate_size, H), g, cfg.init_std, gen_device, dtype),
        "wu": _randn((cfg.intermediate_size, H), g, cfg.init_std, gen_device, dtype),
        "wd": _randn((H, cfg.intermediate_size), g, cfg.init_std, gen_device, dtype),
        # norm weights: 1 + small noise so that parity tests exercise them
        "ln1": (1.0 + _randn((H,), g, cfg.init_std, gen_device, torch.float32)).to(dtype),
        "ln2": (1.0 + _randn((H,), g, cfg.init_std, gen_device, torch.float32)).to(dtype),
        "qn": (1.0 + _randn((D,), g, cfg.init_std, gen_device, torch.float32)).to(dtype),
        "kn": (1.0 + _randn((D,), g, cfg.init_std, gen_device, torch.float32)).to(dtype),
    }


def make_full_globals(cfg: ModelConfig, seed: int, gen_device, dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    g = torch.Generator(device=gen_device).manual_seed(seed * 100003 + 99991)
    return {
        "embed": _randn((cfg.vocab_size, cfg.hidden_size), g, cfg.init_std, gen_device, dtype),
        "lm_head": _randn((cfg.vocab_size, cfg.hidden_size), g, cfg.init_std, gen_device, dtype),
        "final_ln": (1.0 + _randn((cfg.hidden_size,), g, cfg.init_std, gen_device, torch.float32)).to(dtype),
    }


def shard_layer(cfg: ModelConfig, full: Dict[str, torch.Tensor], rank: int, world: int, device) -> Dict[str, torch.Tensor]:
    D = cfg.head_dim
    ql, kl = cfg.num_heads // world, cfg.num_kv_heads // world
    il = cfg.intermediate_size // world
    q0, k0, i0 = rank * ql * D, rank * kl * D, rank * il
    out = {
        # fused column-parallel projection: my q heads, my k heads, my v heads
        "wqkv": torch.cat([full["wq"][q0:q0 + ql * D], full["wk"][k0:k0 + kl * D], full["wv"][k0:k0 + kl * D]]).contiguous(),
        "wo": full["wo"][:, q0:q0 + ql * D].contiguous(),                       # row-parallel
        "wgu": torch.cat([full["wg"][i0:i0 + il], full["wu"][i0:i0 + il]]).contiguous(),
        "wd": full["wd"][:, i0:i0 + il].contiguous(),                           # row-parallel
        "ln1": full["ln1"], "ln2": full["ln2"], "qn": full["qn"], "kn": full["kn"],
    }
    return {k: v.to(device) for k, v in out.items()}


def make_rank_weights(cfg: ModelConfig, rank: int, world: int, seed: int, device, gen_device=None,
                      dtype=torch.bfloat16):
    """Weights of one rank: {'layers': [dict per layer], 'embed', 'lm_head' (vocab shard), 'final_ln'}."""
    cfg.validate(world)
    gen_device = gen_device or device
    layers: List[Dict[str, torch.Tensor]] = []
    for l in range(cfg.num_layers):
        full = make_full_layer(cfg, l, seed, gen_device, dtype)
        layers.append(shard_layer(cfg, full, rank, world, device))
        del full
    glob = make_full_globals(cfg, seed, gen_device, dtype)
    vl = cfg.vocab_size // world
    return {
        "layers": layers,
        "embed": glob["embed"].to(device),
        "lm_head": glob["lm_head"][rank * vl:(rank + 1) * vl].contiguous().to(device),
        "final_ln": glob["final_ln"].to(device),
    }
