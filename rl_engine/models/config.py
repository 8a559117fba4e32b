"""Architecture presets used by the benchmarks and tests."""

from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional, Tuple


@dataclass(frozen=True)
class ModelConfig:
    name: str
    vocab_size: int
    hidden_size: int
    num_layers: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    ffn_size: int
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0
    # mixture of experts (0 experts = dense SwiGLU FFN)
    num_experts: int = 0
    experts_per_token: int = 0
    moe_ffn_size: int = 0
    qk_norm: bool = False
    # context extension of the rotary embedding: None, or (kind, factor, a, b, original_max_positions) with kind
    # "linear", "llama3" (a, b = low / high frequency factors) or "yarn" (a, b = beta_fast, beta_slow); see
    # ``rope_cos_sin``
    rope_scaling: Optional[Tuple[str, float, float, float, int]] = None
    # the LM head is the embedding matrix (small Llama-3.2 / Qwen3 models).  The model still stores both; they start
    # equal and the optimiser gives both the summed gradient, so they stay equal bit for bit.
    tie_word_embeddings: bool = False
    # Qwen2 / Qwen2.5: the q, k and v projections carry a bias (the output projection and the FFN do not)
    qkv_bias: bool = False

    @property
    def q_dim(self) -> int:
        return self.num_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def with_layers(self, n: int) -> "ModelConfig":
        return replace(self, num_layers=n)

    def param_count(self) -> int:
        attn = self.hidden_size * (self.q_dim + 2 * self.kv_dim) + self.q_dim * self.hidden_size
        if self.qkv_bias:
            attn += self.q_dim + 2 * self.kv_dim
        if self.num_experts:
            ffn = self.num_experts * 3 * self.hidden_size * self.moe_ffn_size + self.hidden_size * self.num_experts
        else:
            ffn = 3 * self.hidden_size * self.ffn_size
        per_layer = attn + ffn + 2 * self.hidden_size
        return self.num_layers * per_layer + 2 * self.vocab_size * self.hidden_size + self.hidden_size


def require_no_qkv_bias(cfg: ModelConfig, what: str) -> None:
    if cfg.qkv_bias:
        raise ValueError(f"{what} does not support biased q/k/v projections (Qwen2-style models run on LlamaModel with the "
                         f"one-GPU, data-parallel, context-parallel and pipeline trainers)")


def require_untied(cfg: ModelConfig, what: str) -> None:
    """Tied embeddings are kept equal by ``FlatAdamW`` (one GPU).  The sharded, tensor-parallel and pipeline trainers
    step the embedding and the head in different buckets, ranks or stages and would let them drift apart."""
    if cfg.tie_word_embeddings:
        raise ValueError(f"{what} does not support tied embeddings: train this model with GRPOTrainer on one GPU, or "
                         f"untie it (dataclasses.replace(cfg, tie_word_embeddings=False))")


def llama3_8b() -> ModelConfig:
    """Llama-3-8B: 32 layers, hidden 4096, 32 q / 8 kv heads of 128, FFN 14336, vocab 128256."""
    return ModelConfig("llama3-8b", 128256, 4096, 32, 32, 8, 128, 14336, rms_eps=1e-5, rope_theta=500000.0)


def llama31_8b() -> ModelConfig:
    """Llama-3.1-8B: the Llama-3-8B architecture with the "llama3" rotary scaling (factor 8 over 8 192 positions)."""
    return replace(llama3_8b(), name="llama3.1-8b", rope_scaling=("llama3", 8.0, 1.0, 4.0, 8192))


def llama3_70b() -> ModelConfig:
    """Llama-3-70B: 80 layers, hidden 8192, 64 q / 8 kv heads of 128, FFN 28672, vocab 128256."""
    return ModelConfig("llama3-70b", 128256, 8192, 80, 64, 8, 128, 28672, rms_eps=1e-5, rope_theta=500000.0)


def qwen25_7b() -> ModelConfig:
    """Qwen2.5-7B: 28 layers, hidden 3584, 28 q / 4 kv heads of 128 with biased q/k/v projections, FFN 18944."""
    return ModelConfig("qwen2.5-7b", 152064, 3584, 28, 28, 4, 128, 18944, rms_eps=1e-6, rope_theta=1000000.0, qkv_bias=True)


def qwen3_8b() -> ModelConfig:
    """Qwen3-8B (dense): 36 layers, hidden 4096, 32 q / 8 kv heads of 128 with per-head q/k norms, FFN 12288."""
    return ModelConfig("qwen3-8b", 151936, 4096, 36, 32, 8, 128, 12288, rms_eps=1e-6, rope_theta=1000000.0, qk_norm=True)


def qwen3_32b() -> ModelConfig:
    """Qwen3-32B (dense): 64 layers, hidden 5120, 64 q / 8 kv heads of 128 with per-head q/k norms, FFN 25600."""
    return ModelConfig("qwen3-32b", 151936, 5120, 64, 64, 8, 128, 25600, rms_eps=1e-6, rope_theta=1000000.0, qk_norm=True)


def qwen3_30b_a3b() -> ModelConfig:
    """Qwen3-30B-A3B: 48 layers, hidden 2048, 32 q / 4 kv heads of 128, 128 experts top-8, expert FFN 768."""
    return ModelConfig(
        "qwen3-30b-a3b", 151936, 2048, 48, 32, 4, 128, 6144, rms_eps=1e-6, rope_theta=1000000.0,
        num_experts=128, experts_per_token=8, moe_ffn_size=768, qk_norm=True,
    )


def tiny_llama(head_dim: int = 64) -> ModelConfig:
    """2 layers, hidden 256, 4 heads, SwiGLU 688, vocab 32000 (the CPU fp32 GRPO configuration)."""
    return ModelConfig("tiny-llama", 32000, 4 * head_dim, 2, 4, 4, head_dim, 688, rms_eps=1e-5, rope_theta=10000.0)
