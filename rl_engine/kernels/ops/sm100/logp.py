"""Selected-token log-prob over materialised logits on the sm_100a streaming kernel.

Parity: the nine-method contract of the reference CUDA wrapper
(``rl_engine/kernels/ops/cuda/loss/logp.py:92-205``): ``apply``, ``apply_fp32``, ``out``,
``indexed_out``, ``indexed_fp32`` and the ``online_*`` aliases.  One single-sweep kernel serves
all of them (``csrc/kernels/logp_rows.cu``).  CPU tensors go to the PyTorch oracle.
"""

from __future__ import annotations

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.logp import NativeLogpOp

_SUPPORTED = (torch.float32, torch.bfloat16, torch.float16)


class FusedLogpSM100Op:
    def __init__(self) -> None:
        self._native = NativeLogpOp()

    def __call__(self, logits, token_ids):
        return self.apply(logits, token_ids)

    # -- helpers ---------------------------------------------------------------------------
    @staticmethod
    def _flat(logits: torch.Tensor, token_ids: torch.Tensor):
        if tuple(logits.shape[:-1]) != tuple(token_ids.shape):
            raise ValueError(
                f"logits leading shape {tuple(logits.shape[:-1])} must match token_ids shape {tuple(token_ids.shape)}"
            )
        rows = logits.reshape(-1, logits.shape[-1])
        if rows.stride(1) != 1:
            rows = rows.contiguous()
        ids = token_ids.reshape(-1).to(device=logits.device, dtype=torch.long).contiguous()
        return rows, ids

    def _use_native(self, logits: torch.Tensor, out_dtype: torch.dtype) -> bool:
        return (not logits.is_cuda) or logits.dtype not in _SUPPORTED or out_dtype not in _SUPPORTED

    def _run(self, logits, token_ids, output, row_indices=None):
        rows, ids = self._flat(logits, token_ids)
        if tuple(output.shape) != tuple(logits.shape[:-1]):
            raise ValueError(
                f"output shape {tuple(output.shape)} must match logits leading shape {tuple(logits.shape[:-1])}"
            )
        target = output if output.is_contiguous() else torch.empty_like(output, memory_format=torch.contiguous_format)
        if target is not output:
            target.copy_(output)
        idx = None
        if row_indices is not None:
            idx = row_indices.reshape(-1).to(device=logits.device, dtype=torch.long).contiguous()
            if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= rows.shape[0]):
                raise ValueError("row_indices contains an out-of-range row")
        require_ext().logp_rows(rows, ids, idx, target.view(-1))
        if target is not output:
            output.copy_(target)
        return output

    # -- dense -----------------------------------------------------------------------------
    def apply(self, logits, token_ids):
        if self._use_native(logits, logits.dtype):
            return self._native.apply(logits, token_ids)
        return self._run(logits, token_ids, torch.empty(logits.shape[:-1], dtype=logits.dtype, device=logits.device))

    def apply_fp32(self, logits, token_ids):
        if self._use_native(logits, torch.float32):
            return self._native.apply_fp32(logits, token_ids)
        return self._run(logits, token_ids, torch.empty(logits.shape[:-1], dtype=torch.float32, device=logits.device))

    def out(self, logits, token_ids, output):
        if self._use_native(logits, output.dtype):
            return self._native.out(logits, token_ids, output)
        return self._run(logits, token_ids, output)

    # -- indexed ---------------------------------------------------------------------------
    def indexed_out(self, logits, token_ids, row_indices, output):
        if self._use_native(logits, output.dtype):
            return self._native.indexed_out(logits, token_ids, row_indices, output)
        return self._run(logits, token_ids, output, row_indices)

    def indexed_fp32(self, logits, token_ids, row_indices):
        if self._use_native(logits, torch.float32):
            return self._native.indexed_fp32(logits, token_ids, row_indices)
        output = torch.zeros(logits.shape[:-1], dtype=torch.float32, device=logits.device)
        return self._run(logits, token_ids, output, row_indices)

    # -- the kernel is already single-sweep ("online"), so these are aliases ------------------
    online_out = out
    online_fp32 = apply_fp32
    online_indexed_out = indexed_out
    online_indexed_fp32 = indexed_fp32
