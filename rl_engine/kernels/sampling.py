"""Sampling front end: ``SamplerBackend.sample`` and ``SamplerBackend.compute_logp``.

Parity: reference ``rl_engine/kernels/sampling.py:11-102`` (same class, method names, argument
order and defaults; temperature applied exactly once; ``compute_logp`` returns ``[B, L]`` in the
logits dtype).  On a Blackwell GPU ``sample`` runs the fused sm_100a kernel and ``compute_logp``
the streaming log-prob kernel (constant extra memory: only the ``[B, L]`` output); on CPU both use
plain PyTorch.  ``deterministic`` is accepted for compatibility: the fused sampler is always a pure
function of ``(logits, seed, offset)``; the offset advances on every call.
"""

from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from rl_engine.platforms.constants import constants
from rl_engine.platforms.device import device_ctx
from rl_engine.utils.logger import logger


class SamplerBackend(nn.Module):
    def __init__(self, seed: int = 0) -> None:
        super().__init__()
        self.backend = self._detect_backend()
        self.seed = int(seed)
        self._offset = 0

    def _detect_backend(self) -> str:
        if device_ctx.is_blackwell:
            from rl_engine.kernels.ops.base import _EXT_AVAILABLE

            if _EXT_AVAILABLE:
                logger.info_once("Detected NVIDIA Blackwell GPU - using the fused sm_100a sampler")
                return constants.BackendLib.SM100.value
        return constants.BackendLib.NATIVE.value

    def manual_seed(self, seed: int) -> "SamplerBackend":
        self.seed, self._offset = int(seed), 0
        return self

    @torch.inference_mode()
    def sample(self, logits, top_k: Optional[int] = None, top_p: Optional[float] = None, temperature: float = 1.0,
               deterministic: bool = True):
        if temperature <= 0.0:
            raise ValueError("temperature must be greater than zero")
        if self.backend == constants.BackendLib.SM100.value and logits.is_cuda:
            from rl_engine.kernels.ops.sm100 import sampler as fused

            if top_k is None or top_k <= fused.TOPK_LIMIT or top_k >= logits.shape[-1]:
                offset = self._offset
                self._offset += 1
                ids, _ = fused.sample_topk_topp(
                    logits, top_k=top_k, top_p=top_p, temperature=temperature, seed=self.seed, offset=offset
                )
                return ids.view(-1)
        return self._sample_torch(logits, top_k, top_p, temperature)

    @staticmethod
    def _sample_torch(logits, top_k, top_p, temperature):
        if top_k is not None and int(top_k) <= 0:       # 0 is the usual spelling of "no top-k", as in the fused kernel
            top_k = None
        if top_p is not None and float(top_p) >= 1.0:
            top_p = None
        z = logits.float()
        if temperature != 1.0:
            z = z / temperature
        if top_k is not None:
            kth = torch.topk(z, min(int(top_k), z.shape[-1])).values[..., -1, None]
            z = torch.where(z < kth, torch.full_like(z, float("-inf")), z)
        if top_p is not None:
            sorted_z, order = torch.sort(z, descending=True)
            cum = torch.softmax(sorted_z, dim=-1).cumsum(-1)
            drop = cum > top_p
            drop[..., 1:] = drop[..., :-1].clone()
            drop[..., 0] = False
            z = z.masked_fill(torch.zeros_like(drop).scatter(-1, order, drop), float("-inf"))
        return torch.multinomial(torch.softmax(z, dim=-1), 1).view(-1)

    @torch.inference_mode()
    def compute_logp(self, logits, token_ids):
        """Selected-token log-probs ``[B, L]`` for ``logits`` ``[B, L, V]`` without a ``[B, L, V]`` temporary."""
        batch = logits.shape[0]
        if self.backend == constants.BackendLib.SM100.value and logits.is_cuda:
            from rl_engine.kernels.registry import kernel_registry

            return kernel_registry.get_op("logp").apply(logits, token_ids).view(batch, -1)
        out = torch.empty(logits.shape[:-1], dtype=logits.dtype, device=logits.device)
        step = 4096
        for i in range(0, batch, step):
            chunk = torch.log_softmax(logits[i : i + step], dim=-1)
            out[i : i + step] = chunk.gather(-1, token_ids[i : i + step].unsqueeze(-1)).squeeze(-1)
        return out.view(batch, -1)
