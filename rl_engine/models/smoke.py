"""Tiny end-to-end GRPO step on ``cuda:0`` through the native kernels."""

from __future__ import annotations

import torch


def run_smoke() -> None:
    from rl_engine.kernels.ops.base import check_device_errors, require_ext
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    ext = require_ext()
    assert torch.cuda.is_available(), "smoke() needs a GPU"
    cfg = ModelConfig("smoke", vocab_size=4096, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2,
                      head_dim=128, ffn_size=1024)
    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda:0", seed=0)
    trainer = GRPOTrainer(model, lr=1e-3)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=192, group=4, completion_len=128, seed=1).pin()
    before = ext.launch_count()
    l0 = trainer.step(batch)
    l1 = trainer.step(batch)
    torch.cuda.synchronize()
    check_device_errors(0)
    assert l0 == l0 and l1 == l1, "loss is NaN"
    print(f"smoke ok: loss {l0:.6f} -> {l1:.6f}; native kernel launches: {ext.launch_count() - before}")
