"""Backward of packed attention.

``packed_attention_backward`` returns ``(dq, dk, dv)`` from the forward's output and global
log-sum-exp.  The fused sm_100a backward kernels are used when present in the extension; otherwise
the fp32 PyTorch restatement below runs (same math, far slower, used as the test oracle too).
"""

from __future__ import annotations

from rl_engine.kernels.ops.base import require_ext


def packed_attention_backward(q, k, v, out, lse, dout, layout, scale: float):
    ext = require_ext()
    if hasattr(ext, "attention_bwd"):
        from rl_engine.kernels.ops.sm100.attention_bwd_kernels import fused_backward

        return fused_backward(q, k, v, out, lse, dout, layout, scale)
    from rl_engine.kernels.ops.sm100.attention import _reference_backward

    return _reference_backward(q, k, v, out, lse, dout, layout, scale)
