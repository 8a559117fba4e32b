"""PPO-clip and DPO losses in log-prob space on sm_100a kernels.

The reference advertises these (``README.md:19``) but ships neither; see
``rl_engine/kernels/ops/pytorch/loss/policy_losses.py`` for the oracle definitions.
"""

from __future__ import annotations

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.policy_losses import NativeDPOLossOp, NativePPOLossOp
from rl_engine.kernels.ops.sm100.grpo_loss import surrogate_from_logps


class FusedPPOLossSM100Op:
    def __init__(self) -> None:
        self._native = NativePPOLossOp()

    def __call__(self, *a, **k):
        return self.forward(*a, **k)

    def forward(self, policy_logps, old_logps, advantages, mask, *, ref_logps=None, clip_eps=0.2, beta=0.0):
        if not policy_logps.is_cuda:
            return self._native(policy_logps, old_logps, advantages, mask, ref_logps=ref_logps, clip_eps=clip_eps, beta=beta)
        return surrogate_from_logps(
            policy_logps, ref_logps, old_logps, mask, token_advantages=advantages, clip_eps=clip_eps, beta=beta
        )


class _DPO(torch.autograd.Function):
    @staticmethod
    def forward(ctx, pc, pr, rc, rr, beta, ls):
        loss, chosen, rejected, dh = require_ext().dpo_fwd(pc, pr, rc, rr, beta, ls)
        ctx.save_for_backward(dh)
        ctx.shape = pc.shape
        ctx.mark_non_differentiable(chosen, rejected)
        return loss[0], chosen.reshape(pc.shape), rejected.reshape(pc.shape)

    @staticmethod
    def backward(ctx, g_loss, _gc, _gr):
        (dh,) = ctx.saved_tensors
        g = (g_loss * dh).reshape(ctx.shape)
        return g, -g, None, None, None, None


class FusedDPOLossSM100Op:
    sequence_logps = staticmethod(NativeDPOLossOp.sequence_logps)

    def __init__(self) -> None:
        self._native = NativeDPOLossOp()

    def __call__(self, *a, **k):
        return self.forward(*a, **k)

    def forward(self, policy_chosen_logps, policy_rejected_logps, ref_chosen_logps, ref_rejected_logps,
                *, beta: float = 0.1, label_smoothing: float = 0.0):
        if not policy_chosen_logps.is_cuda:
            return self._native(policy_chosen_logps, policy_rejected_logps, ref_chosen_logps, ref_rejected_logps,
                                beta=beta, label_smoothing=label_smoothing)
        return _DPO.apply(
            policy_chosen_logps.float(), policy_rejected_logps.float(), ref_chosen_logps.detach().float(),
            ref_rejected_logps.detach().float(), float(beta), float(label_smoothing),
        )
