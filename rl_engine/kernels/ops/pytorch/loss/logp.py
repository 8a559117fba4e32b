"""CPU/PyTorch oracle for selected-token log-probabilities over materialised logits.

Parity: reference ``rl_engine/kernels/ops/pytorch/loss/logp.py:7-103`` — the nine-method
contract (``apply``, ``apply_fp32``, ``out``, ``indexed_out``, ``indexed_fp32`` and the four
``online_*`` aliases).  Semantics kept: ``indexed_out`` only writes the listed rows and leaves
all others untouched; ``indexed_fp32`` starts from zeros; out-of-range ``row_indices`` raise.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


class NativeLogpOp:
    def __call__(self, logits: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        return self.apply(logits, token_ids)

    # -- core -----------------------------------------------------------------------------
    @staticmethod
    def _check_lead(lead: torch.Size, other: torch.Tensor, what: str) -> None:
        if tuple(lead) != tuple(other.shape):
            raise ValueError(
                f"logits leading shape {tuple(lead)} must match {what} shape {tuple(other.shape)}"
            )

    def _gathered(self, logits: torch.Tensor, token_ids: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
        lead = logits.shape[:-1]
        self._check_lead(lead, token_ids, "token_ids")
        rows = logits.reshape(-1, logits.shape[-1]).float()
        ids = token_ids.reshape(-1, 1).to(device=logits.device, dtype=torch.long)
        picked = F.log_softmax(rows, dim=-1).gather(1, ids)
        return picked.reshape(lead).to(dtype)

    @staticmethod
    def _rows(row_indices: torch.Tensor, logits: torch.Tensor) -> torch.Tensor:
        n_rows = logits.numel() // max(logits.shape[-1], 1)
        flat = row_indices.reshape(-1).to(device=logits.device, dtype=torch.long)
        if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= n_rows):
            raise ValueError("row_indices contains an out-of-range row")
        return flat

    # -- dense ----------------------------------------------------------------------------
    def apply(self, logits, token_ids):
        return self._gathered(logits, token_ids, logits.dtype)

    def apply_fp32(self, logits, token_ids):
        return self._gathered(logits, token_ids, torch.float32)

    def out(self, logits, token_ids, output):
        self._check_lead(logits.shape[:-1], output, "output")
        output.copy_(self._gathered(logits, token_ids, output.dtype))
        return output

    # -- indexed (only the listed flat rows are produced) ---------------------------------
    def indexed_out(self, logits, token_ids, row_indices, output):
        self._check_lead(logits.shape[:-1], output, "output")
        rows = self._rows(row_indices, logits)
        if rows.numel():
            flat_logits = logits.reshape(-1, logits.shape[-1])[rows]
            flat_ids = token_ids.reshape(-1).to(logits.device)[rows]
            output.view(-1)[rows] = self._gathered(flat_logits, flat_ids, output.dtype)
        return output

    def indexed_fp32(self, logits, token_ids, row_indices):
        output = torch.zeros(logits.shape[:-1], dtype=torch.float32, device=logits.device)
        return self.indexed_out(logits, token_ids, row_indices, output)

    # -- "online" (single-sweep) variants: same math ---------------------------------------
    def online_out(self, logits, token_ids, output):
        return self.out(logits, token_ids, output)

    def online_fp32(self, logits, token_ids):
        return self.apply_fp32(logits, token_ids)

    def online_indexed_out(self, logits, token_ids, row_indices, output):
        return self.indexed_out(logits, token_ids, row_indices, output)

    def online_indexed_fp32(self, logits, token_ids, row_indices):
        return self.indexed_fp32(logits, token_ids, row_indices)
