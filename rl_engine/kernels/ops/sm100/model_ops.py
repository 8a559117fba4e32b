"""RMSNorm, SiLU/SwiGLU, RoPE, embedding and LM-head ops on sm_100a kernels, with autograd.

Each class keeps the ``forward`` / ``forward_fp32`` contract of the reference's PyTorch ops
(``rl_engine/kernels/ops/pytorch/norm/rms_norm.py:27-48``, ``activation/swiglu.py:23-67``,
``linear/embedding.py:23-33``, ``linear/lm_head.py:47-81``); CPU tensors and dtypes the kernels do
not cover are delegated to those oracles.  RoPE has no reference counterpart.
"""

from __future__ import annotations

from typing import Optional

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.activation.swiglu import NativeSiLUOp, NativeSwiGLUOp
from rl_engine.kernels.ops.pytorch.linear.embedding import NativeEmbeddingOp
from rl_engine.kernels.ops.pytorch.linear.lm_head import NativeLMHeadOp
from rl_engine.kernels.ops.pytorch.linear.rope import NativeRoPEOp, rope_cos_sin
from rl_engine.kernels.ops.pytorch.norm.rms_norm import NativeRMSNormOp

_KERNEL_DTYPES = (torch.float32, torch.bfloat16, torch.float16)


def _rows(x: torch.Tensor) -> torch.Tensor:
    x2 = x.reshape(-1, x.shape[-1])
    return x2 if x2.stride(1) == 1 else x2.contiguous()


def _ok(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype in _KERNEL_DTYPES and x.numel() > 0


# ------------------------------------------------------------------------------------ RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = _rows(x)
        w = weight.contiguous()
        y, rstd = require_ext().rmsnorm_fwd(x2, w, eps, False, True)
        ctx.save_for_backward(x2, w, rstd)
        ctx.shape = x.shape
        return y.reshape(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, w, rstd = ctx.saved_tensors
        dx, dw = require_ext().rmsnorm_bwd(x2, w, _rows(dy.to(x2.dtype)), rstd)
        return dx.reshape(ctx.shape), dw, None


class FusedRMSNormSM100Op:
    def __init__(self) -> None:
        self._native = NativeRMSNormOp()

    def __call__(self, x, weight, *, eps: float = 1e-6):
        return self.forward(x, weight, eps=eps)

    def _check(self, x, weight):
        if weight.ndim != 1 or weight.shape[0] != x.shape[-1]:
            raise ValueError(
                f"weight must be 1-D of size x.shape[-1]={x.shape[-1]}, got tuple(weight.shape)={tuple(weight.shape)}"
            )

    def forward(self, x, weight, *, eps: float = 1e-6):
        self._check(x, weight)
        if not (_ok(x) and weight.dtype in _KERNEL_DTYPES):
            return self._native.forward(x, weight, eps=eps)
        return _RMSNorm.apply(x, weight, float(eps))

    def forward_fp32(self, x, weight, *, eps: float = 1e-6):
        self._check(x, weight)
        if not (_ok(x) and weight.dtype in _KERNEL_DTYPES):
            return self._native.forward_fp32(x, weight, eps=eps)
        y, _ = require_ext().rmsnorm_fwd(_rows(x), weight.contiguous(), float(eps), True, False)
        return y.reshape(x.shape)


# ------------------------------------------------------------------------------ SiLU / SwiGLU
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate, up):
        g2 = _rows(gate)
        u2 = None if up is None else _rows(up)
        ctx.save_for_backward(g2, *(() if u2 is None else (u2,)))
        ctx.has_up = up is not None
        ctx.shape = gate.shape
        return require_ext().swiglu_fwd(g2, u2, False).reshape(gate.shape)

    @staticmethod
    def backward(ctx, dy):
        g2, *rest = ctx.saved_tensors
        u2 = rest[0] if ctx.has_up else None
        dg, du = require_ext().swiglu_bwd(g2, u2, _rows(dy.to(g2.dtype)))
        return dg.reshape(ctx.shape), (du.reshape(ctx.shape) if ctx.has_up else None)


class _SwiGLUPacked(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        return require_ext().swiglu_packed_fwd(gu)

    @staticmethod
    def backward(ctx, dy):
        (gu,) = ctx.saved_tensors
        dy2 = dy if (dy.stride(1) == 1 and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0) else dy.contiguous()
        return require_ext().swiglu_packed_bwd(gu, dy2)


def swiglu_packed(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for a packed ``[rows, 2F]`` tensor ``[gate | up]`` (the fused gate/up GEMM output).

    The backward produces the packed gradient in one kernel, so autograd never has to scatter two
    half-width gradients back into a zero-filled ``[rows, 2F]`` buffer."""
    f = gate_up.shape[-1] // 2
    gu2 = gate_up.reshape(-1, gate_up.shape[-1])
    ok = (gate_up.is_cuda and gate_up.dtype == torch.bfloat16 and f % 8 == 0 and gu2.stride(1) == 1
          and gu2.stride(0) % 8 == 0 and gu2.data_ptr() % 16 == 0 and gu2.numel() > 0)
    if not ok:
        from rl_engine.kernels.registry import kernel_registry

        return kernel_registry.get_op("swiglu")(gate_up[..., :f], gate_up[..., f:])
    return _SwiGLUPacked.apply(gu2).reshape(*gate_up.shape[:-1], f)


class FusedSiLUSM100Op(torch.nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self._native = NativeSiLUOp()

    def forward(self, x):
        return _SwiGLU.apply(x, None) if _ok(x) else self._native.forward(x)

    def forward_fp32(self, x):
        if not _ok(x):
            return self._native.forward_fp32(x)
        return require_ext().swiglu_fwd(_rows(x), None, True).reshape(x.shape)


class FusedSwiGLUSM100Op(torch.nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self._native = NativeSwiGLUOp()

    @staticmethod
    def _check(gate, up):
        if gate.shape != up.shape:
            raise ValueError(
                f"gate and up must share shape, got tuple(gate.shape)={tuple(gate.shape)} "
                f"vs tuple(up.shape)={tuple(up.shape)}"
            )

    def forward(self, gate, up):
        self._check(gate, up)
        if not (_ok(gate) and up.dtype == gate.dtype):
            return self._native.forward(gate, up)
        return _SwiGLU.apply(gate, up)

    def forward_fp32(self, gate, up):
        self._check(gate, up)
        if not (_ok(gate) and up.dtype == gate.dtype):
            return self._native.forward_fp32(gate, up)
        return require_ext().swiglu_fwd(_rows(gate), _rows(up), True).reshape(gate.shape)


# --------------------------------------------------------------------------------------- RoPE
class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, cos_t, sin_t):
        ctx.save_for_backward(positions, cos_t, sin_t)
        return require_ext().rope(x, positions, cos_t, sin_t, False)

    @staticmethod
    def backward(ctx, dy):
        positions, cos_t, sin_t = ctx.saved_tensors
        return require_ext().rope(dy.contiguous(), positions, cos_t, sin_t, True), None, None, None


class FusedRoPESM100Op:
    """``x`` ``[..., seq, heads, head_dim]``, ``positions`` ``[..., seq]``; half-split rotation."""

    def __init__(self) -> None:
        self._native = NativeRoPEOp()
        self._tables = {}

    def tables(self, max_pos: int, head_dim: int, theta: float, device, scaling=None) -> tuple:
        key = (int(max_pos), head_dim, float(theta), str(device), scaling)
        hit = self._tables.get(key)
        if hit is None:
            cos, sin = rope_cos_sin(torch.arange(max_pos, device=device), head_dim, theta, scaling)
            hit = self._tables[key] = (cos.contiguous(), sin.contiguous())
        return hit

    def __call__(self, x, positions, *, theta: float = 10000.0, tables=None, scaling=None):
        return self.forward(x, positions, theta=theta, tables=tables, scaling=scaling)

    def forward(self, x, positions, *, theta: float = 10000.0, tables=None, scaling=None):
        """``scaling``: context-extension rule of the rotary frequencies (``scaled_inv_freq``), ``None`` for none."""
        if not _ok(x):
            return self._native.forward(x, positions, theta=theta, scaling=scaling)
        heads, d = x.shape[-2], x.shape[-1]
        x3 = x.reshape(-1, heads, d).contiguous()
        pos = positions.reshape(-1).to(torch.long).contiguous()
        if tables is None:
            # table length rounded up to a power of two so it is built at most log(max_pos) times
            need = int(pos.max()) + 1 if pos.numel() else 1
            tables = self.tables(1 << max(need - 1, 1).bit_length(), d, theta, x.device, scaling)
        return _RoPE.apply(x3, pos, tables[0], tables[1]).reshape(x.shape)

    def forward_fp32(self, x, positions, *, theta: float = 10000.0, scaling=None):
        return self._native.forward_fp32(x, positions, theta=theta, scaling=scaling)


# ---------------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        flat = ids.reshape(-1).to(torch.long).contiguous()
        ctx.save_for_backward(flat)
        ctx.w_shape = weight.shape
        ctx.w_dtype = weight.dtype
        out = require_ext().embedding_fwd(flat, weight if weight.stride(1) == 1 else weight.contiguous())
        return out.reshape(*ids.shape, weight.shape[1])

    @staticmethod
    def backward(ctx, dy):
        (flat,) = ctx.saved_tensors
        d = ctx.w_shape[1]
        dy2 = dy.reshape(-1, d).contiguous()
        # stable sort + run-length encoding fix the summation order: no atomics, bitwise reproducible
        sorted_ids, order = torch.sort(flat, stable=True)
        seg_ids, counts = torch.unique_consecutive(sorted_ids, return_counts=True)
        seg_start = torch.zeros(seg_ids.numel() + 1, dtype=torch.long, device=flat.device)
        seg_start[1:] = counts.cumsum(0)
        keep = (seg_ids >= 0) & (seg_ids < ctx.w_shape[0])
        dtable = torch.zeros(ctx.w_shape, dtype=ctx.w_dtype, device=dy.device)
        if bool(keep.all()):
            require_ext().embedding_bwd(seg_ids, seg_start, order, dy2, dtable)
        else:
            raise ValueError("embedding backward saw out-of-range token ids")
        return None, dtable


class FusedEmbeddingSM100Op(torch.nn.Module):
    def __init__(self) -> None:
        super().__init__()
        self._native = NativeEmbeddingOp()

    def forward(self, token_ids, weight):
        if not (_ok(weight) and token_ids.is_cuda):
            return self._native.forward(token_ids, weight)
        return _Embedding.apply(token_ids, weight)

    def forward_fp32(self, token_ids, weight):
        return self.forward(token_ids, weight).float()


# ------------------------------------------------------------------------------------ LM head
class FusedLMHeadSM100Op:
    """``hidden @ weight.T (+ bias)`` on the tcgen05 GEMM for bf16; fp32 ground truth stays in PyTorch."""

    def __init__(self) -> None:
        self._native = NativeLMHeadOp()

    def __call__(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        return self.forward(hidden, weight, bias=bias)

    def forward(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        if not (hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
                and hidden.shape[-1] % 8 == 0 and hidden.numel() > 0):
            return self._native.forward(hidden, weight, bias=bias)
        from rl_engine.kernels.ops.sm100.gemm import matmul_nt

        out = matmul_nt(hidden, weight)
        return out if bias is None else out + bias.to(out.dtype)

    def forward_fp32(self, hidden, weight, *, bias: Optional[torch.Tensor] = None):
        return self._native.forward_fp32(hidden, weight, bias=bias)
