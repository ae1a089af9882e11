"""Tensor-parallel decoder engine slice (Qwen3-shaped) built on the attention operators."""
from .config import ModelConfig, qwen3_8b_shaped, tiny_config  # noqa: F401
from .weights import make_rank_weights  # noqa: F401
from .model import TPDecoder  # noqa: F401
from .runner import GenerationRunner  # noqa: F401
