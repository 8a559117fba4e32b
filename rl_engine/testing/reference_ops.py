"""Plain fp32 reference math for RL quantities.

Parity: reference ``rl_engine/testing/reference_ops.py:15-142`` (same function names, argument
order and conventions — note ``compute_policy_ratio`` zeroes masked entries whereas the
``ratio_kl`` op yields 1 there; both conventions are kept on purpose).
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch


def _keep(mask: torch.Tensor, device: torch.device) -> torch.Tensor:
    return mask.to(device=device, dtype=torch.bool)


def selected_logprobs_reference(
    logits: torch.Tensor,
    token_ids: torch.Tensor,
    mask: Optional[torch.Tensor] = None,
    temperature: float = 1.0,
    output_dtype: torch.dtype = torch.float32,
) -> torch.Tensor:
    if temperature <= 0.0:
        raise ValueError("temperature must be greater than zero")
    if tuple(logits.shape[:-1]) != tuple(token_ids.shape):
        raise ValueError(
            f"logits leading shape {tuple(logits.shape[:-1])} must match token_ids shape {tuple(token_ids.shape)}"
        )
    if mask is not None and tuple(mask.shape) != tuple(token_ids.shape):
        raise ValueError(f"mask shape {tuple(mask.shape)} must match token_ids shape")
    ids = token_ids.long()
    keep = None
    if mask is not None:
        keep = _keep(mask, token_ids.device)
        ids = torch.where(keep, ids, torch.zeros_like(ids))
    logp = torch.log_softmax(logits.float() / float(temperature), dim=-1)
    picked = logp.gather(-1, ids.to(logp.device).unsqueeze(-1)).squeeze(-1)
    if keep is not None:
        picked = torch.where(keep.to(picked.device), picked, torch.zeros_like(picked))
    return picked.to(output_dtype)


def masked_sum(values: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    v = values.float()
    if mask is None:
        return v.sum()
    return torch.where(_keep(mask, v.device), v, torch.zeros_like(v)).sum()


def active_token_count(mask: Optional[torch.Tensor], values: Optional[torch.Tensor] = None) -> torch.Tensor:
    if mask is None:
        if values is None:
            raise ValueError("values must be provided when mask is None")
        return torch.tensor(float(values.numel()), device=values.device)
    return mask.to(torch.bool).sum().to(torch.float32)


def masked_mean(values: torch.Tensor, mask: Optional[torch.Tensor] = None, eps: float = 1e-8) -> torch.Tensor:
    return masked_sum(values, mask) / active_token_count(mask, values).clamp_min(eps)


def compute_policy_ratio(current_logps, old_logps, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    ratio = torch.exp(current_logps.float() - old_logps.float())
    if mask is not None:
        ratio = torch.where(_keep(mask, ratio.device), ratio, torch.zeros_like(ratio))
    return ratio


def compute_reference_kl(current_logps, ref_logps, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    d = ref_logps.float() - current_logps.float()
    kl = torch.exp(d) - d - 1.0
    if mask is not None:
        kl = torch.where(_keep(mask, kl.device), kl, torch.zeros_like(kl))
    return kl


def summarize_kernel_drift(candidate, reference, mask: Optional[torch.Tensor] = None) -> Dict[str, Any]:
    if candidate.shape != reference.shape:
        raise ValueError(
            f"candidate shape {tuple(candidate.shape)} must match reference shape {tuple(reference.shape)}"
        )
    err = (candidate.float() - reference.float()).abs()
    picked = err.reshape(-1) if mask is None else err[_keep(mask, err.device)]
    n = int(picked.numel())
    return {
        "max_abs_error": float(picked.max()) if n else 0.0,
        "mean_abs_error": float(picked.mean()) if n else 0.0,
        "active_count": n,
    }
