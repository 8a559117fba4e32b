"""GRPO loss on sm_100a kernels: group advantages, ratio/KL front end, clipped surrogate.

Parity: ``TritonGRPOLossOp`` (``rl_engine/kernels/ops/triton/loss/grpo_loss.py:58-246``) —
``group_advantages``, ``apply``, ``forward`` with the same keyword arguments and return triple
``(loss, policy_loss, kl)``.  Where the reference finishes with ~10 torch elementwise/reduction
launches (``:185-214``), the tail here is one surrogate kernel with a fixed-order reduction plus a
one-thread finisher, and its backward is one kernel.

``apply_from_logps`` is the entry the training step uses: selected-token log-probs in, so no
``[B, T, V]`` tensor exists anywhere.
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.grpo_loss import Boundaries, NativeGRPOLossOp
from rl_engine.kernels.ops.sm100.ratio_kl import FusedRatioKLSM100Op


class _Surrogate(torch.autograd.Function):
    """(loss, policy_loss, kl) from log-probs; differentiable w.r.t. the policy log-probs."""

    @staticmethod
    def forward(ctx, logp, ref_logp, old_logp, adv_seq, adv_tok, mask, T, clip_eps, beta):
        out4, d_pl, d_kl, _, _ = require_ext().surrogate_fwd(
            logp, ref_logp, old_logp, adv_seq, adv_tok, mask, T, clip_eps, beta, False
        )
        ctx.save_for_backward(out4, d_pl, d_kl)
        ctx.beta = beta
        ctx.shape = logp.shape
        return out4[0], out4[1], out4[2]

    @staticmethod
    def backward(ctx, g_loss, g_pl, g_kl):
        out4, d_pl, d_kl = ctx.saved_tensors
        zero = torch.zeros((), device=out4.device)
        g3 = torch.stack([zero if g is None else g.float().reshape(()) for g in (g_loss, g_pl, g_kl)])
        grad = require_ext().surrogate_bwd(d_pl, d_kl, out4, g3, ctx.beta)
        return grad.reshape(ctx.shape), None, None, None, None, None, None, None, None


def surrogate_from_logps(
    policy_logps: torch.Tensor,
    ref_logps: Optional[torch.Tensor],
    old_logps: torch.Tensor,
    mask: torch.Tensor,
    *,
    sample_advantages: Optional[torch.Tensor] = None,
    token_advantages: Optional[torch.Tensor] = None,
    clip_eps: float = 0.2,
    beta: float = 0.0,
):
    """Clipped surrogate + k3 KL over ``[B, T]`` log-probs (GRPO: per-sequence advantages; PPO: per-token)."""
    if (sample_advantages is None) == (token_advantages is None):
        raise ValueError("pass exactly one of sample_advantages / token_advantages")
    t = policy_logps.shape[-1] if policy_logps.ndim > 1 else 1
    flat = lambda x: None if x is None else x.detach().reshape(-1).float().contiguous()
    lp = policy_logps.reshape(-1).float().contiguous()
    return _Surrogate.apply(
        lp, flat(ref_logps), flat(old_logps), flat(sample_advantages), flat(token_advantages),
        mask.reshape(-1).to(torch.bool).contiguous(), t, float(clip_eps), float(beta),
    )


class FusedGRPOLossSM100Op:
    def __init__(self) -> None:
        self._native = NativeGRPOLossOp()
        self._ratio_kl = FusedRatioKLSM100Op()

    def __call__(self, policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask, **kw):
        return self.forward(policy_logits, ref_logits, action_ids, old_logps, rewards, completion_mask, **kw)

    def group_advantages(
        self, rewards: torch.Tensor, *, samples_per_prompt: Optional[int] = None,
        group_boundaries: Optional[Boundaries] = None, eps: float = 1e-6,
    ) -> torch.Tensor:
        if not rewards.is_cuda:
            return self._native.group_advantages(
                rewards, samples_per_prompt=samples_per_prompt, group_boundaries=group_boundaries, eps=eps
            )
        flat = rewards.reshape(-1).float().contiguous()
        n = flat.numel()
        if (samples_per_prompt is None) == (group_boundaries is None):
            raise ValueError("Provide exactly one of samples_per_prompt or group_boundaries.")
        if samples_per_prompt is not None:
            if samples_per_prompt < 2:
                raise ValueError("samples_per_prompt must be at least 2 for group normalization.")
            if n % samples_per_prompt:
                raise ValueError(
                    f"num_sequences ({n}) must be divisible by samples_per_prompt ({samples_per_prompt})."
                )
            return require_ext().group_advantages(flat, None, int(samples_per_prompt), float(eps))
        host = torch.as_tensor(group_boundaries, dtype=torch.long).cpu()
        if host.ndim != 1 or host.numel() < 2:
            raise ValueError("group_boundaries must be a 1D tensor of length num_groups + 1.")
        sizes = host.diff()
        if int(sizes.sum()) != n or int(host[0]) != 0:
            raise ValueError(f"group sizes sum to {int(sizes.sum())} but there are {n} sequences.")
        if bool((sizes < 1).any()):
            raise ValueError("each group must contain at least one sequence.")
        return require_ext().group_advantages(flat, host.to(flat.device), 0, float(eps))

    expand_advantages = staticmethod(NativeGRPOLossOp.expand_advantages)

    def apply(
        self, policy_logits, ref_logits, action_ids, old_logps, sample_advantages, completion_mask,
        *, clip_eps: float = 0.2, beta: float = 0.0,
    ):
        if not policy_logits.is_cuda:
            return self._native.apply(
                policy_logits, ref_logits, action_ids, old_logps, sample_advantages, completion_mask,
                clip_eps=clip_eps, beta=beta,
            )
        # logits -> selected log-probs on the streaming kernels, then the fused tail.  The ratio/KL
        # front end already produces exp(lp - old) and the k3 terms with the right masking, but the
        # tail needs log-probs, so route through the differentiable log-prob kernel pair instead.
        from rl_engine.kernels.ops.sm100.logp_autograd import selected_logprobs

        keep = completion_mask.to(torch.bool)
        v = policy_logits.shape[-1]
        if bool((keep & ((action_ids < 0) | (action_ids >= v))).any()):
            raise ValueError(
                f"action_ids at active (unmasked) positions must be in [0, {v}); found out-of-range ids."
            )
        ids = torch.where(keep, action_ids, torch.zeros_like(action_ids))
        lp = selected_logprobs(policy_logits, ids, keep)
        with torch.no_grad():
            lr = selected_logprobs(ref_logits.to(policy_logits.dtype), ids, keep)
        return surrogate_from_logps(
            lp, lr, old_logps, keep, sample_advantages=sample_advantages, clip_eps=clip_eps, beta=beta
        )

    def apply_from_logps(
        self, policy_logps, ref_logps, old_logps, sample_advantages, completion_mask,
        *, clip_eps: float = 0.2, beta: float = 0.0,
    ):
        if not policy_logps.is_cuda:
            return self._native.apply_from_logps(
                policy_logps, ref_logps, old_logps, sample_advantages, completion_mask, clip_eps=clip_eps, beta=beta
            )
        return surrogate_from_logps(
            policy_logps, ref_logps, old_logps, completion_mask, sample_advantages=sample_advantages,
            clip_eps=clip_eps, beta=beta,
        )

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
