"""Differentiable selected-token log-prob over logits, built from the ratio/KL kernel pair.

``d logp / d logits = onehot - softmax`` is exactly what ``ratio_kl_bwd`` writes when called with
``ratio = 1`` and ``g_kl = 0``, and ``ratio_kl_fwd`` with no reference streams each row once and
returns the log-prob and its log-sum-exp, so the same two kernels serve plain log-prob autograd.
Masked rows return 0 and get a zero gradient.
"""

from __future__ import annotations

import torch

from rl_engine.kernels.ops.base import require_ext


class _SelectedLogp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits2d, ids, mask):
        zeros = torch.zeros(logits2d.shape[0], dtype=torch.float32, device=logits2d.device)
        _, _, d, lse, _, lp = require_ext().ratio_kl_fwd(logits2d, None, ids, mask, zeros)
        ctx.save_for_backward(logits2d, ids, mask, d, lse)
        return lp

    @staticmethod
    def backward(ctx, g):
        logits2d, ids, mask, d, lse = ctx.saved_tensors
        grad = require_ext().ratio_kl_bwd(
            logits2d, ids, mask, g.float().contiguous(), torch.zeros_like(lse), torch.ones_like(lse), d, lse
        )
        return grad, None, None


def selected_logprobs(logits: torch.Tensor, ids: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    v = logits.shape[-1]
    rows = logits.reshape(-1, v)
    if rows.stride(1) != 1:
        rows = rows.contiguous()
    out = _SelectedLogp.apply(rows, ids.reshape(-1).long().contiguous(), mask.reshape(-1).bool().contiguous())
    return out.reshape(logits.shape[:-1])
