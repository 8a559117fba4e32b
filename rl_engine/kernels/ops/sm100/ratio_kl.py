"""Fused policy-ratio + k3-KL front end over logits (sm_100a), with autograd.

Parity: ``TritonRatioKLOp`` (``rl_engine/kernels/ops/triton/loss/ratio_kl.py:125-196``) and the
native op's semantics (``ops/pytorch/loss/ratio_kl.py:33-58``): masked rows give ratio 1 / kl 0,
an out-of-range id at an active position raises, gradients flow to ``policy_logits`` only.
"""

from __future__ import annotations

from typing import Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.ratio_kl import NativeRatioKLOp


class _RatioKL(torch.autograd.Function):
    @staticmethod
    def forward(ctx, policy, ref, ids, mask, old):
        ratio, kl, d, lse, bad, _lp = require_ext().ratio_kl_fwd(policy, ref, ids, mask, old)
        ctx.save_for_backward(policy, ids, mask, ratio, d, lse)
        ctx.mark_non_differentiable(bad)
        return ratio, kl, bad

    @staticmethod
    def backward(ctx, g_ratio, g_kl, _g_bad):
        policy, ids, mask, ratio, d, lse = ctx.saved_tensors
        g_ratio = torch.zeros_like(ratio) if g_ratio is None else g_ratio
        g_kl = torch.zeros_like(ratio) if g_kl is None else g_kl
        grad = require_ext().ratio_kl_bwd(policy, ids, mask, g_ratio.contiguous(), g_kl.contiguous(), ratio, d, lse)
        return grad, None, None, None, None


class FusedRatioKLSM100Op:
    def __init__(self, check_ids: bool = True) -> None:
        self._native = NativeRatioKLOp()
        self.check_ids = check_ids

    def __call__(self, policy_logits, ref_logits, action_ids, attention_mask, old_logps):
        return self.forward(policy_logits, ref_logits, action_ids, attention_mask, old_logps)

    def forward(self, policy_logits, ref_logits, action_ids, attention_mask, old_logps) -> Tuple[torch.Tensor, torch.Tensor]:
        if not policy_logits.is_cuda or policy_logits.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            return self._native(policy_logits, ref_logits, action_ids, attention_mask, old_logps)
        lead = policy_logits.shape[:-1]
        if tuple(action_ids.shape) != tuple(lead) or tuple(attention_mask.shape) != tuple(lead):
            raise ValueError("action_ids and attention_mask must match the leading shape of the logits")
        if ref_logits.shape != policy_logits.shape:
            raise ValueError("ref_logits must match policy_logits")
        v = policy_logits.shape[-1]
        pol = policy_logits.reshape(-1, v)
        ref = ref_logits.detach().reshape(-1, v).to(policy_logits.dtype)
        if pol.stride(1) != 1:
            pol = pol.contiguous()
        if ref.stride(1) != 1:
            ref = ref.contiguous()
        ids = action_ids.reshape(-1).to(torch.long).contiguous()
        mask = attention_mask.reshape(-1).to(torch.bool).contiguous()
        old = old_logps.reshape(-1).float().contiguous()
        ratio, kl, bad = _RatioKL.apply(pol, ref, ids, mask, old)
        if self.check_ids and int(bad.item()):
            raise ValueError(
                f"action_ids at active (unmasked) positions must be in [0, {v}); found out-of-range ids."
            )
        return ratio.reshape(lead), kl.reshape(lead)
