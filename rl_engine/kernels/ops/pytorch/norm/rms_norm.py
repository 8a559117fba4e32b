"""CPU/PyTorch oracle for RMSNorm.

Parity: reference ``rl_engine/kernels/ops/pytorch/norm/rms_norm.py:9-70``:
``x * rsqrt(mean(x^2) + eps) * weight`` in fp32 with eps inside the sqrt and a plain
(not ``1 + w``) weight; ``forward`` returns ``x.dtype``, ``forward_fp32`` returns fp32.
"""

from __future__ import annotations

import torch


class NativeRMSNormOp:
    def __call__(self, x: torch.Tensor, weight: torch.Tensor, *, eps: float = 1e-6) -> torch.Tensor:
        return self.forward(x, weight, eps=eps)

    def forward(self, x, weight, *, eps: float = 1e-6):
        return self._run(x, weight, eps).to(x.dtype)

    def forward_fp32(self, x, weight, *, eps: float = 1e-6):
        return self._run(x, weight, eps)

    @staticmethod
    def _run(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
        if weight.ndim != 1 or weight.shape[0] != x.shape[-1]:
            raise ValueError(
                f"weight must be 1-D of size x.shape[-1]={x.shape[-1]}, got tuple(weight.shape)={tuple(weight.shape)}"
            )
        xf = x.float()
        inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
        return xf * inv * weight.float()
