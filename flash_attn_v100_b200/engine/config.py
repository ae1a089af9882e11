"""Model shape (the reference's `ModelConfig`, flash_attn_llm/models/config.py:7-104, reduced to what
a Qwen3-style decoder needs)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class ModelConfig:
    num_layers: int
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    qk_norm: bool = True          # per-head RMSNorm on q and k (Qwen3)
    init_std: float = 0.02

    def validate(self, world: int) -> None:
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be divisible by num_kv_heads")
        for name, v in (("num_heads", self.num_heads), ("num_kv_heads", self.num_kv_heads),
                        ("intermediate_size", self.intermediate_size), ("vocab_size", self.vocab_size)):
            if v % world:
                raise ValueError(f"{name}={v} must be divisible by the tensor-parallel size {world}")
        if self.head_dim not in (64, 128, 256):
            raise ValueError("head_dim must be 64, 128 or 256")


def qwen3_8b_shaped() -> ModelConfig:
    """36 layers, hidden 4096, 32 query / 8 KV heads of 128, SwiGLU 12288, vocabulary 151936."""
    return ModelConfig(num_layers=36, hidden_size=4096, num_heads=32, num_kv_heads=8, head_dim=128,
                       intermediate_size=12288, vocab_size=151936)


def tiny_config() -> ModelConfig:
    """Small shape for parity tests (same structure, divisible by 2 for TP=2)."""
    return ModelConfig(num_layers=2, hidden_size=256, num_heads=8, num_kv_heads=2, head_dim=64,
                       intermediate_size=512, vocab_size=1024)
