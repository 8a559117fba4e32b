"""Model definitions built only from registry operators (the reference has toy models only)."""

from rl_engine.models.config import (
    ModelConfig, llama3_8b, llama3_70b, llama31_8b, qwen25_7b, qwen3_8b, qwen3_30b_a3b, qwen3_32b, tiny_llama,
)
from rl_engine.models.llama import LlamaModel

__all__ = ["ModelConfig", "LlamaModel", "llama3_8b", "llama3_70b", "llama31_8b", "qwen25_7b", "qwen3_8b", "qwen3_30b_a3b", "qwen3_32b",
           "tiny_llama"]
