"""Seeded synthetic RL batch: G samples per prompt sharing the prompt tokens.

Parity: reference ``rl_engine/testing/rl_batch.py:12-199`` — same dataclass fields, helper
methods, metadata keys and validation messages.  The random stream layout differs (this build
draws every field from its own forked generator so adding a field never shifts the others).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch


@dataclass(frozen=True)
class SyntheticRLKernelBatch:
    input_ids: torch.Tensor          # [B, P+C]
    attention_mask: torch.Tensor     # [B, P+C] bool
    prompt_mask: torch.Tensor        # [B, P+C] bool
    completion_mask: torch.Tensor    # [B, C] bool
    token_ids: torch.Tensor          # [B, C] completion ids
    rewards: torch.Tensor            # [B]
    advantages: torch.Tensor         # [B, C]
    old_logps: torch.Tensor          # [B, C]
    ref_logps: torch.Tensor          # [B, C]
    valid_indices: Optional[torch.Tensor]
    metadata: Dict[str, Any]

    @property
    def batch_size(self) -> int:
        return int(self.input_ids.shape[0])

    @property
    def total_seq_len(self) -> int:
        return int(self.input_ids.shape[1])

    @property
    def prompt_len(self) -> int:
        return int(self.metadata["prompt_len"])

    @property
    def completion_len(self) -> int:
        return int(self.metadata["completion_len"])

    @property
    def flat_completion_mask(self) -> torch.Tensor:
        return self.completion_mask.reshape(-1)

    @property
    def flat_token_ids(self) -> torch.Tensor:
        return self.token_ids.reshape(-1)

    def dense_completion_token_ids(self) -> torch.Tensor:
        return self.token_ids

    def dense_completion_values(self, values: torch.Tensor) -> torch.Tensor:
        want = (self.batch_size, self.completion_len)
        if tuple(values.shape[:2]) != want:
            raise ValueError(f"expected leading shape {want}, got {tuple(values.shape[:2])}")
        return values

    def compact_completion_values(self, values: torch.Tensor) -> torch.Tensor:
        dense = self.dense_completion_values(values)
        return dense.reshape(-1, *dense.shape[2:])[self.flat_completion_mask]

    def compact_token_ids(self) -> torch.Tensor:
        return self.flat_token_ids[self.flat_completion_mask]

    def benchmark_metadata(self) -> Dict[str, Any]:
        keys = ("num_prompts", "samples_per_prompt")
        out = {k: self.metadata[k] for k in keys}
        out.update(
            batch_size=self.batch_size,
            prompt_len=self.prompt_len,
            completion_len=self.completion_len,
            total_seq_len=self.total_seq_len,
            vocab_size=self.metadata["vocab_size"],
            valid_density=self.metadata["valid_density"],
            valid_tokens=int(self.flat_completion_mask.sum()),
            dtype=str(self.metadata["dtype"]),
            device=str(self.input_ids.device),
            seed=self.metadata["seed"],
        )
        return out


def make_synthetic_rl_kernel_batch(
    *,
    num_prompts: int,
    samples_per_prompt: int,
    prompt_len: int,
    completion_len: int,
    vocab_size: int,
    valid_density: float = 1.0,
    dtype: torch.dtype = torch.float32,
    device: torch.device | str = "cpu",
    seed: int = 0,
) -> SyntheticRLKernelBatch:
    if num_prompts <= 0:
        raise ValueError("num_prompts must be greater than zero")
    if samples_per_prompt <= 0:
        raise ValueError("samples_per_prompt must be greater than zero")
    if prompt_len < 0:
        raise ValueError("prompt_len must be non-negative")
    if completion_len <= 0:
        raise ValueError("completion_len must be greater than zero")
    if vocab_size <= 1:
        raise ValueError("vocab_size must be greater than one")
    if not 0.0 <= valid_density <= 1.0:
        raise ValueError("valid_density must be in [0.0, 1.0]")

    dev = torch.device(device)
    b = num_prompts * samples_per_prompt
    total = prompt_len + completion_len

    def stream(tag: int) -> torch.Generator:
        gen = torch.Generator(device="cpu")
        gen.manual_seed(seed * 1_000_003 + tag)
        return gen

    completions = torch.randint(0, vocab_size, (b, completion_len), generator=stream(1))
    prompts = torch.randint(0, vocab_size, (num_prompts, prompt_len), generator=stream(2))
    input_ids = torch.cat([prompts.repeat_interleave(samples_per_prompt, 0), completions], dim=1)

    completion_mask = torch.zeros(b * completion_len, dtype=torch.bool)
    n_valid = int(round(b * completion_len * valid_density))
    if n_valid:
        completion_mask[torch.randperm(b * completion_len, generator=stream(3))[:n_valid]] = True
    completion_mask = completion_mask.reshape(b, completion_len)

    prompt_mask = torch.zeros(b, total, dtype=torch.bool)
    prompt_mask[:, :prompt_len] = True
    attention_mask = torch.cat([torch.ones(b, prompt_len, dtype=torch.bool), completion_mask], dim=1)

    def normal(shape, tag):
        return torch.randn(shape, generator=stream(tag)).to(dtype)

    meta: Dict[str, Any] = dict(
        num_prompts=num_prompts, samples_per_prompt=samples_per_prompt, batch_size=b, prompt_len=prompt_len,
        completion_len=completion_len, total_seq_len=total, vocab_size=vocab_size, valid_density=valid_density,
        valid_tokens=n_valid, dtype=dtype, device=str(dev), seed=seed,
    )
    return SyntheticRLKernelBatch(
        input_ids=input_ids.to(dev),
        attention_mask=attention_mask.to(dev),
        prompt_mask=prompt_mask.to(dev),
        completion_mask=completion_mask.to(dev),
        token_ids=completions.clone().to(dev),
        rewards=normal((b,), 4).to(dev),
        advantages=normal((b, completion_len), 5).to(dev),
        old_logps=normal((b, completion_len), 6).to(dev),
        ref_logps=normal((b, completion_len), 7).to(dev),
        valid_indices=completion_mask.reshape(-1).nonzero().squeeze(-1).to(dev),
        metadata=meta,
    )
