"""bf16 GEMM on the hand-written tcgen05 kernel, with autograd.

``matmul_nt(x, w)`` computes ``x @ w.T`` (the ``nn.Linear`` layout).  The backward products
``dx = dy @ w`` and ``dw = dy.T @ x`` run on the same kernel with MN-major operand descriptors, so
no transpose copies are made.  The reference has no GEMM of its own (torch.matmul / cuBLAS:
``rl_engine/kernels/ops/pytorch/linear/lm_head.py:104-113``).
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_engine.kernels.ops.base import require_ext


def _as_2d(t: torch.Tensor) -> torch.Tensor:
    t2 = t.reshape(-1, t.shape[-1])
    if t2.stride(1) != 1 or t2.stride(0) % 8 or t2.data_ptr() % 16:
        t2 = t2.contiguous()
    return t2


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    *,
    a_mn: bool = False,
    b_mn: bool = False,
    out: Optional[torch.Tensor] = None,
    out_dtype: torch.dtype = torch.bfloat16,
    accumulate: bool = False,
    alpha: float = 1.0,
    pair: Optional[bool] = None,
) -> torch.Tensor:
    """``D[M,N] = alpha * op(A) @ op(B).T (+ D)``; see ``csrc/kernels/kernels.h`` for layouts.

    ``pair`` selects the tile engine: ``True`` = 256 x 256 tiles on pairs of SMs (``tcgen05`` ``cta_group::2``),
    ``False`` = 128 x 256 tiles on single SMs, ``None`` = the library default (``RLK_GEMM_PAIR`` overrides it)."""
    flag = -1 if pair is None else int(bool(pair))
    return require_ext().gemm(a, b, a_mn, b_mn, out, out_dtype == torch.float32, accumulate, alpha, flag)


class _LinearNT(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        x2 = _as_2d(x)
        w2 = _as_2d(w)
        ctx.save_for_backward(x2, w2)
        ctx.x_shape = x.shape
        y = gemm(x2, w2)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy: torch.Tensor):
        x2, w2 = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx[M,K] = dy[M,N] @ w[N,K]: B operand is w read as [contraction N, K] -> MN-major
            dx = gemm(dy2, w2, b_mn=True).reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dw[N,K] = dy.T @ x: both operands are stored [contraction M, *] -> MN-major
            dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw


def matmul_nt(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x[..., K] @ w[N, K].T`` in bf16 with fp32 accumulation (differentiable)."""
    return _LinearNT.apply(x, w)
