"""fp8 (e4m3) GEMM with row-wise scales on the tcgen05 kernel (``kind::f8f6f4``, fp32 accumulation in TMEM).

``quantize_rows(x)`` turns bf16 rows into e4m3 codes plus one fp32 scale per row (``x ~= code * scale``, scale =
row amax / 448).  ``matmul_nt_fp8(x, w_q, w_scale)`` quantises the activations per token and multiplies them with
weights that were quantised per output channel once; ``Fp8Linear`` packages that for inference-side linears (rollout,
scoring), where the tensor cores run at twice their bf16 rate.  Not differentiable: training stays in bf16.

The reference has no reduced-precision GEMM (it serves in bf16: ``rl_engine/kernels/ops/pytorch/linear/lm_head.py``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext

E4M3_MAX = 448.0


def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x [rows, cols]`` (bf16, cols % 16 == 0) -> ``(codes uint8 [rows, cols], scale fp32 [rows])``."""
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(1) != 1:
        x2 = x2.contiguous()
    q, scale = require_ext().quantize_fp8_rows(x2)
    return q, scale


def quantize_rows_reference(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """PyTorch restatement of ``quantize_rows`` (codes as ``torch.float8_e4m3fn``)."""
    xf = x.float()
    amax = xf.abs().amax(dim=-1)
    # tensor / tensor is a true division (a Python-scalar divisor would be turned into a multiplication by 1 / 448)
    scale = torch.where(amax > 0, amax / torch.full_like(amax, E4M3_MAX), torch.ones_like(amax))
    inv = torch.ones_like(scale) / scale
    codes = (xf * inv[:, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return codes, scale


def gemm_fp8(a_q: torch.Tensor, scale_a: torch.Tensor, b_q: torch.Tensor, scale_b: torch.Tensor,
             pair: Optional[bool] = None) -> torch.Tensor:
    """``(a_q @ b_q.T) * scale_a[:, None] * scale_b[None, :]`` -> bf16 ``[M, N]``; codes are uint8 or float8_e4m3fn.
    ``pair``: 256 x 256 tiles on SM pairs (default for more than one row tile) or 128 x 256 tiles on single SMs."""
    as_u8 = lambda t: t.view(torch.uint8) if t.dtype != torch.uint8 else t
    flag = -1 if pair is None else int(bool(pair))
    return require_ext().gemm_fp8(as_u8(a_q), scale_a, as_u8(b_q), scale_b, flag)


def matmul_nt_fp8(x: torch.Tensor, w_q: torch.Tensor, w_scale: torch.Tensor) -> torch.Tensor:
    """``x[..., K] @ w[N, K].T`` with ``x`` quantised per token on the fly and ``w`` given as codes + per-channel scales."""
    x_q, x_scale = quantize_rows(x)
    return gemm_fp8(x_q, x_scale, w_q, w_scale).reshape(*x.shape[:-1], w_q.shape[0])


class Fp8Linear:
    """A linear layer whose weight ``[N, K]`` is stored as e4m3 codes with one scale per output channel."""

    def __init__(self, weight: torch.Tensor) -> None:
        self.w_q, self.w_scale = quantize_rows(weight.detach().to(torch.bfloat16))

    @torch.no_grad()
    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        return matmul_nt_fp8(x, self.w_q, self.w_scale)
