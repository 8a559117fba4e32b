"""CPU/PyTorch oracles for SiLU and SwiGLU.

Parity: reference ``rl_engine/kernels/ops/pytorch/activation/swiglu.py:10-86``: fp32 math,
``forward`` casts back to the input dtype, ``forward_fp32`` keeps fp32, shape guard on SwiGLU.
"""

from __future__ import annotations

import torch
from torch import nn


class NativeSiLUOp(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.forward_fp32(x).to(x.dtype)

    def forward_fp32(self, x: torch.Tensor) -> torch.Tensor:
        xf = x.float()
        return xf * torch.sigmoid(xf)


class NativeSwiGLUOp(nn.Module):
    def forward(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        return self.forward_fp32(gate, up).to(gate.dtype)

    def forward_fp32(self, gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
        if gate.shape != up.shape:
            raise ValueError(
                f"gate and up must share shape, got tuple(gate.shape)={tuple(gate.shape)} "
                f"vs tuple(up.shape)={tuple(up.shape)}"
            )
        gf = gate.float()
        return gf * torch.sigmoid(gf) * up.float()
