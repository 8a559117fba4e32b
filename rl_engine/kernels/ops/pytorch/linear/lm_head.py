"""CPU/PyTorch oracle for the LM head projection ``hidden @ weight.T (+ bias)``.

Parity: reference ``rl_engine/kernels/ops/pytorch/linear/lm_head.py:12-124``: weight in HF
``[vocab, hidden]`` layout; ``forward`` computes and returns in ``hidden.dtype``;
``forward_fp32`` upcasts and runs with autocast and TF32 disabled, restoring both afterwards.
"""

from __future__ import annotations

from contextlib import contextmanager
from typing import Optional

import torch


@contextmanager
def strict_fp32_matmul(device_type: str):
    saved = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        with torch.autocast(device_type=device_type, enabled=False):
            yield
    finally:
        torch.backends.cuda.matmul.allow_tf32 = saved


class NativeLMHeadOp:
    def __call__(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        return self.forward(hidden, weight, bias=bias)

    def forward(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        dt = hidden.dtype
        out = hidden @ weight.to(dt).t()
        return out if bias is None else out + bias.to(dt)

    def forward_fp32(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        with strict_fp32_matmul(hidden.device.type):
            out = hidden.float() @ weight.float().t()
        return out if bias is None else out + bias.float()

    _strict_fp32_matmul = staticmethod(strict_fp32_matmul)
