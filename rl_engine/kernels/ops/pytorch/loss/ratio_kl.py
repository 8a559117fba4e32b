"""CPU/PyTorch oracle for the fused policy-ratio + reference-KL front end.

Parity: reference ``rl_engine/kernels/ops/pytorch/loss/ratio_kl.py:13-58``.
``ratio = exp(logp_policy - old_logps)`` and ``kl = exp(d) - d - 1`` with
``d = logp_ref - logp_policy`` (the k3 estimator); masked positions give ``ratio = 1`` and
``kl = 0`` and may hold arbitrary action ids; an out-of-range id at an *active* position raises.
"""

from __future__ import annotations

from typing import Tuple

import torch

from rl_engine.kernels.ops.pytorch.loss.logp import NativeLogpOp


def ratio_kl_from_logps(
    logp_policy: torch.Tensor,
    logp_ref: torch.Tensor,
    old_logps: torch.Tensor,
    mask: torch.Tensor,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Logp-space tail shared by the logits-space op and the logp-space losses."""
    keep = mask.to(torch.bool)
    zero = torch.zeros((), dtype=torch.float32, device=logp_policy.device)
    delta = torch.where(keep, logp_policy.float() - old_logps.float(), zero)
    diff = torch.where(keep, logp_ref.float() - logp_policy.float(), zero)
    return torch.exp(delta), torch.exp(diff) - diff - 1.0


class NativeRatioKLOp:
    def __init__(self) -> None:
        self._logp = NativeLogpOp()

    def __call__(self, policy_logits, ref_logits, action_ids, attention_mask, old_logps):
        return self.forward(policy_logits, ref_logits, action_ids, attention_mask, old_logps)

    def forward(
        self,
        policy_logits: torch.Tensor,
        ref_logits: torch.Tensor,
        action_ids: torch.Tensor,
        attention_mask: torch.Tensor,
        old_logps: torch.Tensor,
    ) -> Tuple[torch.Tensor, torch.Tensor]:
        keep = attention_mask.to(torch.bool)
        vocab = policy_logits.shape[-1]
        if bool((keep & ((action_ids < 0) | (action_ids >= vocab))).any()):
            raise ValueError(
                f"action_ids at active (unmasked) positions must be in [0, {vocab}); "
                "found out-of-range ids."
            )
        ids = torch.where(keep, action_ids, torch.zeros_like(action_ids))
        logp_policy = self._logp.apply_fp32(policy_logits, ids)
        with torch.no_grad():
            logp_ref = self._logp.apply_fp32(ref_logits, ids)
        return ratio_kl_from_logps(logp_policy, logp_ref, old_logps, keep)
