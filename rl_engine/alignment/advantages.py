"""Per-token advantages for the PPO-clip loss.

``ppo_loss`` (the registry operator) takes per-token advantages; these helpers produce them from rewards and a value
model the usual way.  The reference advertises PPO next to GRPO (``README.md:19``) and documents ``ratio_kl`` as their
shared front end (``docs/operators/ratio-kl.md:3-11``) but ships neither the clipped objective nor an advantage
estimator; the objective is ``rl_engine.kernels.ops.*.policy_losses``, the estimator is here.

All functions work on ``[B, T]`` tensors with a boolean ``mask`` of real completion positions, keep masked positions at
zero, and run on whatever device the inputs live on (plain PyTorch: the scan over ``T`` is tiny next to a model step).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch


def kl_shaped_rewards(sequence_rewards: torch.Tensor, policy_logps: torch.Tensor, ref_logps: torch.Tensor,
                      mask: torch.Tensor, *, kl_coef: float = 0.05) -> torch.Tensor:
    """Per-token rewards ``[B, T]``: ``-kl_coef * (logp - ref_logp)`` at every real position plus the sequence-level
    reward ``[B]`` on the last real position of each row (the shaping used by PPO-style RLHF)."""
    keep = mask.bool()
    rewards = torch.where(keep, -kl_coef * (policy_logps.float() - ref_logps.float()), torch.zeros_like(policy_logps, dtype=torch.float32))
    lengths = keep.long().sum(dim=1)
    has_tokens = lengths > 0
    last = (keep.long() * torch.arange(1, keep.shape[1] + 1, device=keep.device)).argmax(dim=1)
    rows = torch.arange(keep.shape[0], device=keep.device)[has_tokens]
    rewards[rows, last[has_tokens]] += sequence_rewards.float()[has_tokens]
    return rewards


def gae_advantages(rewards: torch.Tensor, values: torch.Tensor, mask: torch.Tensor, *, gamma: float = 1.0,
                   lam: float = 0.95) -> Tuple[torch.Tensor, torch.Tensor]:
    """Generalised advantage estimation over the real positions of every row.

    ``rewards``, ``values``: ``[B, T]`` (value of the state BEFORE emitting the token at that position).  The value
    after the last real token is zero (the episode ends).  Masked positions are skipped, not treated as steps: the
    recursion runs over each row's real tokens in order, wherever they sit.  Returns ``(advantages, returns)`` with
    ``returns = advantages + values``; both are zero at masked positions."""
    keep = mask.bool()
    r = torch.where(keep, rewards.float(), torch.zeros_like(rewards, dtype=torch.float32))
    v = torch.where(keep, values.float(), torch.zeros_like(values, dtype=torch.float32))
    b, t = r.shape
    adv = torch.zeros_like(r)
    running = torch.zeros(b, dtype=torch.float32, device=r.device)      # advantage of the next real position
    next_value = torch.zeros(b, dtype=torch.float32, device=r.device)   # value of the next real position
    for i in range(t - 1, -1, -1):
        here = keep[:, i]
        delta = r[:, i] + gamma * next_value - v[:, i]
        current = delta + gamma * lam * running
        adv[:, i] = torch.where(here, current, adv[:, i])
        running = torch.where(here, current, running)
        next_value = torch.where(here, v[:, i], next_value)
    return adv, torch.where(keep, adv + v, torch.zeros_like(adv))


def whiten(values: torch.Tensor, mask: torch.Tensor, *, shift_mean: bool = True, eps: float = 1e-8) -> torch.Tensor:
    """Normalise over the real positions of the whole batch to unit variance (and zero mean with ``shift_mean``)."""
    keep = mask.bool()
    x = values.float()
    n = keep.sum().clamp(min=1)
    mean = torch.where(keep, x, torch.zeros_like(x)).sum() / n
    var = torch.where(keep, (x - mean) ** 2, torch.zeros_like(x)).sum() / n
    out = (x - mean) * torch.rsqrt(var + eps)
    if not shift_mean:
        out = out + mean
    return torch.where(keep, out, torch.zeros_like(out))


def value_loss(values: torch.Tensor, old_values: torch.Tensor, returns: torch.Tensor, mask: torch.Tensor, *,
               clip_range: Optional[float] = 0.2) -> torch.Tensor:
    """Clipped squared error of a value head (PPO): ``0.5 * mean(max((v - R)^2, (clip(v, old +- range) - R)^2))`` over
    the real positions; ``clip_range=None`` gives the plain squared error."""
    keep = mask.bool()
    v, target = values.float(), returns.float()
    err = (v - target) ** 2
    if clip_range is not None:
        clipped = old_values.float() + (v - old_values.float()).clamp(-clip_range, clip_range)
        err = torch.maximum(err, (clipped - target) ** 2)
    n = keep.sum().clamp(min=1)
    return 0.5 * torch.where(keep, err, torch.zeros_like(err)).sum() / n
