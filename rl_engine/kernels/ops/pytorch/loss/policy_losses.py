"""CPU/PyTorch oracles for the PPO-clip and DPO losses in log-prob space.

The reference advertises PPO and DPO kernels (``README.md:19``) but ships only the GRPO loss;
its ``ratio_kl`` doc (``docs/operators/ratio-kl.md:3-33``) describes PPO as "ratio_kl + a
caller-written clipped surrogate".  These two classes are that missing tail.

* PPO: per-token advantages ``[B, T]``; ``loss = mean_mask(-min(r*A, clip(r)*A)) + beta*kl``.
* DPO: sequence-summed log-probs; ``loss = -logsigmoid(beta * ((pc - pr) - (rc - rr)))`` with
  optional label smoothing; also returns the implicit rewards.
"""

from __future__ import annotations

from typing import Tuple

import torch
import torch.nn.functional as F

from rl_engine.kernels.ops.pytorch.loss.grpo_loss import clipped_surrogate
from rl_engine.kernels.ops.pytorch.loss.ratio_kl import ratio_kl_from_logps


class NativePPOLossOp:
    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def forward(
        self,
        policy_logps: torch.Tensor,
        old_logps: torch.Tensor,
        advantages: torch.Tensor,
        mask: torch.Tensor,
        *,
        ref_logps: torch.Tensor | None = None,
        clip_eps: float = 0.2,
        beta: float = 0.0,
    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        keep = mask.bool()
        ref = policy_logps.detach() if ref_logps is None else ref_logps.detach()
        ratio, kl_terms = ratio_kl_from_logps(policy_logps, ref, old_logps, keep)
        adv = torch.where(keep, advantages.float(), torch.zeros_like(advantages, dtype=torch.float32))
        return clipped_surrogate(ratio, kl_terms, adv, keep, clip_eps, beta)


class NativeDPOLossOp:
    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    @staticmethod
    def sequence_logps(token_logps: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        keep = mask.bool()
        return torch.where(keep, token_logps.float(), torch.zeros_like(token_logps, dtype=torch.float32)).sum(-1)

    def forward(
        self,
        policy_chosen_logps: torch.Tensor,
        policy_rejected_logps: torch.Tensor,
        ref_chosen_logps: torch.Tensor,
        ref_rejected_logps: torch.Tensor,
        *,
        beta: float = 0.1,
        label_smoothing: float = 0.0,
    ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        pi = policy_chosen_logps.float() - policy_rejected_logps.float()
        ref = ref_chosen_logps.float() - ref_rejected_logps.float()
        h = beta * (pi - ref.detach())
        per_pair = -(1.0 - label_smoothing) * F.logsigmoid(h) - label_smoothing * F.logsigmoid(-h)
        chosen_reward = beta * (policy_chosen_logps.float() - ref_chosen_logps.float()).detach()
        rejected_reward = beta * (policy_rejected_logps.float() - ref_rejected_logps.float()).detach()
        return per_pair.mean(), chosen_reward, rejected_reward
