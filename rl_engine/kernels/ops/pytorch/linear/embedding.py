"""CPU/PyTorch oracle for token embedding (row gather).

Parity: reference ``rl_engine/kernels/ops/pytorch/linear/embedding.py:10-51``: argument order
``(token_ids, weight)``; gather in the table's dtype, ``forward_fp32`` upcasts only the result.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn


class NativeEmbeddingOp(nn.Module):
    def forward(self, token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return F.embedding(token_ids.long(), weight)

    def forward_fp32(self, token_ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        return F.embedding(token_ids.long(), weight).float()
