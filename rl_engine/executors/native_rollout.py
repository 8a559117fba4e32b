"""Native rollout engine: G completions of one prompt with prefix-shared attention and the fused sampler.

The prompt is stored once in the packed batch ``[prompt | completion_0 | ...]``; every decoding step
re-runs the stateless forward over the packed tokens (no KV cache is kept between steps -- the same
"stateless" trade the scoring executor makes) and draws the next token of every completion with the
``sample_topk_topp`` kernel.  Rollout log-probs come from ``linear_logp``, the kernel the trainer
differentiates, so training-time and rollout-time log-probs of the same tokens agree bitwise.
The reference has no rollout engine of its own (it delegates to vLLM).
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch


class NativeRolloutEngine:
    def __init__(self, model: torch.nn.Module, seed: int = 0) -> None:
        self.model = model
        self.seed = seed
        self._offset = 0

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, *, num_generations: int, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = 50, top_p: Optional[float] = 1.0) -> Dict[str, Any]:
        from rl_engine.kernels.ops.sm100.attention import grpo_group_layout
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.kernels.sampling import SamplerBackend

        model = self.model
        dev = model.flat.device
        prompt = prompt_ids.to(dev).long().reshape(-1)
        p, g = prompt.numel(), num_generations
        sampler = SamplerBackend(seed=self.seed)
        sampler._offset = self._offset
        completions = torch.zeros(g, 0, dtype=torch.long, device=dev)
        head = model.lm_head_weight()
        for step in range(max_new_tokens):
            l = completions.shape[1]
            if l == 0:
                layout = grpo_group_layout(p, 0, 1, dev)
                tokens, positions = prompt, torch.arange(p, device=dev)
                rows = torch.full((g,), p - 1, device=dev)
            else:
                layout = grpo_group_layout(p, g, l, dev)
                tokens = torch.cat([prompt, completions.reshape(-1)])
                positions = torch.cat([torch.arange(p, device=dev), (p + torch.arange(l, device=dev)).repeat(g)])
                rows = p + torch.arange(g, device=dev) * l + (l - 1)
            hidden = model.hidden_states(tokens, positions, layout)
            last = hidden.index_select(0, rows)
            logits = kernel_registry.get_op("lm_head")(last, head)
            nxt = sampler.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature)
            completions = torch.cat([completions, nxt.reshape(g, 1)], dim=1)
        self._offset = sampler._offset
        logps = self.score(prompt, completions)
        return {"prompt_ids": prompt, "completion_ids": completions, "rollout_logps": logps}

    @torch.no_grad()
    def score(self, prompt: torch.Tensor, completions: torch.Tensor) -> torch.Tensor:
        """Log-probs of ``completions [G, L]`` under the current weights, via the training-path kernels."""
        from rl_engine.models.grpo import GRPOBatch, policy_logps

        g, l = completions.shape
        zeros = torch.zeros(g, l, device=prompt.device)
        batch = GRPOBatch(prompt, completions, torch.zeros(g, device=prompt.device), zeros, zeros,
                          torch.ones(g, l, dtype=torch.bool, device=prompt.device))
        return policy_logps(self.model, batch)
