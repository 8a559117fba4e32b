"""A Llama layer under tensor + sequence parallelism, built on the fused all-gather->GEMM / GEMM->reduce-scatter kernels.

Between the linears the activations are sharded by tokens (``[T / W, H]`` per rank); inside the attention and
the FFN they are sharded by heads / FFN columns:

    x_local [T/W, H] -> RMSNorm -> column_parallel(Wqkv shard)   [T, (hq + 2 hkv) / W * 128]     (tp_ag_gemm)
                     -> RoPE + packed flash attention over this rank's heads, all T tokens
                     -> row_parallel(Wo shard)                   [T/W, H]  + residual            (tp_gemm_rs)
                     -> RMSNorm -> column_parallel([gate | up] shard) -> SwiGLU
                     -> row_parallel(Wdown shard)                [T/W, H]  + residual

Weights are sharded with ``shard_layer_weights`` from a ``LlamaModel`` layer (q / k / v heads and the gate / up
halves are sliced separately so that every rank's packed layout matches the single-GPU one).  The two norm
weights are replicated: their gradients are partial sums over this rank's token rows and must be summed over
the ranks by the caller, like any data-parallel parameter.

The reference has no tensor-parallel layers; the oracle is ``LlamaModel._layer`` with the full weights.
"""

from __future__ import annotations

import math
from typing import Dict

import torch

from rl_engine.models.config import ModelConfig
from rl_engine.models.llama import _FusedAttentionBlock, rms_norm, swiglu_packed
from rl_engine.parallel.tp_linear import TensorParallelLinears


def shard_layer_weights(model, index: int, rank: int, world: int) -> Dict[str, torch.Tensor]:
    """This rank's shard of layer ``index`` (detached clones; set ``requires_grad_`` as needed)."""
    cfg: ModelConfig = model.cfg
    if cfg.num_heads % world or cfg.num_kv_heads % world or cfg.ffn_size % world or cfg.num_experts:
        raise ValueError("heads, kv heads and the FFN width must divide by the TP size (dense layers only)")
    d, h = cfg.head_dim, cfg.hidden_size
    hq, hkv, f = cfg.num_heads // world, cfg.num_kv_heads // world, cfg.ffn_size // world
    v = lambda n: model.view(f"l{index}.{n}").detach()
    wqkv = v("wqkv")
    q_rows = wqkv[: cfg.q_dim].view(cfg.num_heads, d, h)[rank * hq:(rank + 1) * hq]
    k_rows = wqkv[cfg.q_dim: cfg.q_dim + cfg.kv_dim].view(cfg.num_kv_heads, d, h)[rank * hkv:(rank + 1) * hkv]
    v_rows = wqkv[cfg.q_dim + cfg.kv_dim:].view(cfg.num_kv_heads, d, h)[rank * hkv:(rank + 1) * hkv]
    gu = v("w_gate_up")
    gate, up = gu[: cfg.ffn_size], gu[cfg.ffn_size:]
    return {
        "attn_norm": v("attn_norm").clone(),
        "mlp_norm": v("mlp_norm").clone(),
        "wqkv": torch.cat([q_rows.reshape(-1, h), k_rows.reshape(-1, h), v_rows.reshape(-1, h)], 0).contiguous(),
        "wo": v("wo")[:, rank * hq * d:(rank + 1) * hq * d].contiguous(),
        "w_gate_up": torch.cat([gate[rank * f:(rank + 1) * f], up[rank * f:(rank + 1) * f]], 0).contiguous(),
        "w_down": v("w_down")[:, rank * f:(rank + 1) * f].contiguous(),
    }


class TensorParallelLlamaLayer:
    def __init__(self, cfg: ModelConfig, weights: Dict[str, torch.Tensor], tp: TensorParallelLinears,
                 rope_cos: torch.Tensor, rope_sin: torch.Tensor) -> None:
        if cfg.head_dim != 128:
            raise ValueError("the fused attention path needs head_dim == 128")
        self.cfg, self.w, self.tp = cfg, weights, tp
        self.rope_cos, self.rope_sin = rope_cos, rope_sin
        self.hq = cfg.num_heads // tp.world
        self.hkv = cfg.num_kv_heads // tp.world

    def __call__(self, x_local: torch.Tensor, positions: torch.Tensor, layout) -> torch.Tensor:
        """``x_local [T / W, H]`` (this rank's token rows, rank-major order) -> same shape."""
        cfg, w, tp = self.cfg, self.w, self.tp
        h = rms_norm(x_local, w["attn_norm"], cfg.rms_eps)
        qkv = tp.column_parallel(h, w["wqkv"])                                   # [T, (hq + 2 hkv) * 128]
        t = qkv.shape[0]
        attn = _FusedAttentionBlock.apply(qkv.view(t, self.hq + 2 * self.hkv, cfg.head_dim), positions, self.rope_cos,
                                          self.rope_sin, layout, self.hq, self.hkv, 1.0 / math.sqrt(cfg.head_dim))
        x = x_local + tp.row_parallel(attn.reshape(t, self.hq * cfg.head_dim), w["wo"])
        h = rms_norm(x, w["mlp_norm"], cfg.rms_eps)
        act = swiglu_packed(tp.column_parallel(h, w["w_gate_up"]))               # [T, F / W]
        return x + tp.row_parallel(act, w["w_down"])
