"""Linear layers fused (at the autograd level) with the cheap op in front of them, so that the cheap op's output is
not kept for the backward pass but recomputed there.

``norm_linear(x, norm_weight, w)`` = ``rms_norm(x) @ w.T`` keeps ``x`` and the per-row ``rstd`` (``x`` is the residual
stream and alive anyway), not the normalised activations.  ``swiglu_linear(gate_up, w)`` = ``(silu(gate) * up) @ w.T``
keeps the packed ``[gate | up]`` GEMM output, not the activation.  For a Llama-3-8B layer that is 2 x 4096 + 14336
fewer elements per token out of 69632, paid for with three memory-bound kernels in the backward pass; the results are
the same bits as the unfused composition (same kernels, same order).

More layers keep their activations in the same memory (``rl_engine.models.activation_plan``), which saves whole layer
recomputations.  The reference has no counterpart (its models are Hugging Face modules).
"""

from __future__ import annotations

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.sm100.gemm import _as_2d, gemm


def _supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0
            and x.numel() > 0)


class _NormLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, norm_weight, w, eps):
        ext = require_ext()
        x2 = _as_2d(x)
        nw = norm_weight.contiguous()
        w2 = _as_2d(w)
        h, rstd = ext.rmsnorm_fwd(x2, nw, eps, False, True)
        ctx.save_for_backward(x2, nw, rstd, w2)
        ctx.eps, ctx.x_shape = eps, x.shape
        return gemm(h, w2).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        ext = require_ext()
        x2, nw, rstd, w2 = ctx.saved_tensors
        dy2 = _as_2d(dy)
        h, _ = ext.rmsnorm_fwd(x2, nw, ctx.eps, False, False)
        dw = gemm(dy2, h, a_mn=True, b_mn=True) if ctx.needs_input_grad[2] else None
        del h
        dx, dnw = ext.rmsnorm_bwd(x2, nw, gemm(dy2, w2, b_mn=True), rstd)
        return dx.reshape(ctx.x_shape), dnw, dw, None


class _SwiGLULinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up, w):
        gu2 = _as_2d(gate_up)
        w2 = _as_2d(w)
        ctx.save_for_backward(gu2, w2)
        ctx.gu_shape = gate_up.shape
        y = gemm(require_ext().swiglu_packed_fwd(gu2), w2)
        return y.reshape(*gate_up.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        ext = require_ext()
        gu2, w2 = ctx.saved_tensors
        dy2 = _as_2d(dy)
        dw = None
        if ctx.needs_input_grad[1]:
            act = ext.swiglu_packed_fwd(gu2)
            dw = gemm(dy2, act, a_mn=True, b_mn=True)
            del act
        dgu = ext.swiglu_packed_bwd(gu2, gemm(dy2, w2, b_mn=True))
        return dgu.reshape(ctx.gu_shape), dw


def norm_linear(x: torch.Tensor, norm_weight: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """``rms_norm(x, norm_weight) @ w.T``; the normalised activations are recomputed in the backward pass."""
    if _supported(x, w) and norm_weight.dtype == torch.bfloat16:
        return _NormLinear.apply(x, norm_weight, w, float(eps))
    from rl_engine.kernels.registry import kernel_registry

    return kernel_registry.get_op("rms_norm")(x, norm_weight, eps=eps) @ w.t()


def swiglu_linear(gate_up: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``(silu(gate) * up) @ w.T`` for packed ``[rows, 2F] = [gate | up]``; the activation is recomputed in backward."""
    f = gate_up.shape[-1] // 2
    if _supported(gate_up, w) and f % 8 == 0:
        return _SwiGLULinear.apply(gate_up, w)
    from rl_engine.kernels.registry import kernel_registry

    return kernel_registry.get_op("swiglu")(gate_up[..., :f], gate_up[..., f:]) @ w.t()
