"""CPU/PyTorch oracle for the GRPO loss (group-normalised advantages + clipped surrogate + KL).

Parity: reference ``rl_engine/kernels/ops/pytorch/loss/grpo_loss.py:13-206``:
``group_advantages`` (population std, ``var`` clamped at ``eps**2``), ``expand_advantages``,
``apply`` (per-sequence advantages in, ``(loss, policy_loss, kl)`` out), ``forward`` (rewards in)
and the exactly-one-of ``samples_per_prompt`` (>= 2) / CSR ``group_boundaries`` rule.

New here (the reference only has the logits-space entry): ``apply_from_logps`` runs the same
tail on selected-token log-probs, which is what ``linear_logp`` produces without ever
materialising ``[N, V]`` logits.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple, Union

import torch

from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp, ratio_kl_from_logps

Boundaries = Union[Sequence[int], torch.Tensor]


def resolve_group_ids(
    num_sequences: int,
    *,
    device: torch.device,
    samples_per_prompt: Optional[int],
    group_boundaries: Optional[Boundaries],
) -> torch.Tensor:
    """Map each sequence to its group index from either a uniform size or CSR offsets."""
    if (samples_per_prompt is None) == (group_boundaries is None):
        raise ValueError("Provide exactly one of samples_per_prompt or group_boundaries.")
    if samples_per_prompt is not None:
        if samples_per_prompt < 2:
            raise ValueError("samples_per_prompt must be at least 2 for group normalization.")
        if num_sequences % samples_per_prompt:
            raise ValueError(
                f"num_sequences ({num_sequences}) must be divisible by "
                f"samples_per_prompt ({samples_per_prompt})."
            )
        return torch.arange(num_sequences, device=device) // samples_per_prompt
    offsets = torch.as_tensor(group_boundaries, dtype=torch.long, device=device)
    if offsets.ndim != 1 or offsets.numel() < 2:
        raise ValueError("group_boundaries must be a 1D tensor of length num_groups + 1.")
    sizes = offsets.diff()
    total = int(sizes.sum())
    if total != num_sequences:
        raise ValueError(f"group sizes sum to {total} but there are {num_sequences} sequences.")
    if bool((sizes < 1).any()):
        raise ValueError("each group must contain at least one sequence.")
    return torch.repeat_interleave(torch.arange(sizes.numel(), device=device), sizes)


def masked_mean(values: torch.Tensor, keep: torch.Tensor, eps: float = 1e-8) -> torch.Tensor:
    total = torch.where(keep, values, torch.zeros_like(values)).sum()
    return total / keep.sum().to(values.dtype).clamp_min(eps)


def clipped_surrogate(
    ratio: torch.Tensor, kl_terms: torch.Tensor, adv_tok: torch.Tensor, keep: torch.Tensor,
    clip_eps: float, beta: float,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    lo, hi = 1.0 - clip_eps, 1.0 + clip_eps
    per_tok = -torch.minimum(ratio * adv_tok, ratio.clamp(lo, hi) * adv_tok)
    policy_loss = masked_mean(per_tok, keep)
    kl = masked_mean(kl_terms, keep)
    return policy_loss + beta * kl, policy_loss, kl


class NativeGRPOLossOp:
    def __init__(self) -> None:
        self._ratio_kl = NativeRatioKLOp()

    def __call__(self, policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask, **kw):
        return self.forward(policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask, **kw)

    def group_advantages(
        self,
        rewards: torch.Tensor,
        *,
        samples_per_prompt: Optional[int] = None,
        group_boundaries: Optional[Boundaries] = None,
        eps: float = 1e-6,
    ) -> torch.Tensor:
        r = rewards.reshape(-1).float()
        gid = resolve_group_ids(
            r.numel(), device=r.device, samples_per_prompt=samples_per_prompt, group_boundaries=group_boundaries
        )
        n_groups = int(gid.max()) + 1 if r.numel() else 0
        zeros = r.new_zeros(n_groups)
        count = zeros.index_add(0, gid, torch.ones_like(r))
        mean = zeros.index_add(0, gid, r) / count
        second = zeros.index_add(0, gid, r * r) / count
        std = (second - mean * mean).clamp_min(eps * eps).sqrt()
        return (r - mean[gid]) / std[gid]

    @staticmethod
    def expand_advantages(sample_advantages: torch.Tensor, completion_mask: torch.Tensor) -> torch.Tensor:
        keep = completion_mask.bool()
        tok = sample_advantages.reshape(-1, 1).expand(keep.shape)
        return torch.where(keep, tok, torch.zeros_like(tok))

    def apply(
        self, policy_logits, ref_logits, action_ids, old_logps, sample_advantages, completion_mask,
        *, clip_eps: float = 0.2, beta: float = 0.0,
    ):
        ratio, kl_terms = self._ratio_kl(policy_logits, ref_logits, action_ids, completion_mask, old_logps)
        keep = completion_mask.bool()
        adv = self.expand_advantages(sample_advantages, completion_mask).float()
        return clipped_surrogate(ratio, kl_terms, adv, keep, clip_eps, beta)

    def apply_from_logps(
        self, policy_logps, ref_logps, old_logps, sample_advantages, completion_mask,
        *, clip_eps: float = 0.2, beta: float = 0.0,
    ):
        """Same loss, but from selected-token log-probs ``[B, T]`` instead of logits."""
        keep = completion_mask.bool()
        ratio, kl_terms = ratio_kl_from_logps(policy_logps, ref_logps.detach(), old_logps, keep)
        adv = self.expand_advantages(sample_advantages, completion_mask).float()
        return clipped_surrogate(ratio, kl_terms, adv, keep, clip_eps, beta)

    def forward(
        self, policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask,
        *, clip_eps: float = 0.2, beta: float = 0.0, samples_per_prompt: Optional[int] = None,
        group_boundaries: Optional[Boundaries] = None, eps: float = 1e-6,
    ):
        adv = self.group_advantages(
            rewards, samples_per_prompt=samples_per_prompt, group_boundaries=group_boundaries, eps=eps
        )
        return self.apply(
            policy_logits, ref_logits, action_ids, old_logps, adv, completion_mask, clip_eps=clip_eps, beta=beta
        )

    # kept as static helpers because callers of the reference reach for them by these names
    _masked_mean = staticmethod(masked_mean)
    _resolve_group_ids = staticmethod(resolve_group_ids)
