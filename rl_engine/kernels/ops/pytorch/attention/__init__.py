"""CPU/PyTorch attention oracles.

Parity: reference ``rl_engine/kernels/ops/pytorch/attention/__init__.py:8-46``:
``NativeAttentionOp`` takes FlashAttention layout ``(batch, seq, heads, head_dim)``, repeats K/V
heads for GQA/MQA and calls SDPA.

``NativePrefixSharedAttentionOp`` is the oracle for the prefix-shared kernel
(``csrc/cuda/attention/prefix_shared_attention.cu:85-311`` in the reference computes the
non-causal, shared-K/V form only); here it also covers what a GRPO step needs: G completions
attend a shared prompt K/V *and* causally their own completion K/V, with GQA and an LSE output.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


class NativeAttentionOp:
    def __call__(self, q, k, v, dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False):
        qh, kh, vh = (t.transpose(1, 2) for t in (q, k, v))
        if kh.shape[1] != vh.shape[1]:
            raise ValueError("k and v must have the same number of heads")
        if qh.shape[1] != kh.shape[1]:
            if qh.shape[1] % kh.shape[1]:
                raise ValueError("q heads must be divisible by k/v heads for GQA/MQA")
            rep = qh.shape[1] // kh.shape[1]
            kh, vh = kh.repeat_interleave(rep, 1), vh.repeat_interleave(rep, 1)
        out = F.scaled_dot_product_attention(qh, kh, vh, dropout_p=dropout_p, is_causal=causal, scale=softmax_scale)
        return out.transpose(1, 2)


class NativePrefixSharedAttentionOp:
    """``q`` ``[bs, G, Lq, D]`` attends shared ``k``/``v`` ``[bs, Lkv, D]`` with no mask."""

    def __call__(self, q, k, v, softmax_scale: Optional[float] = None):
        scale = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else softmax_scale
        s = torch.einsum("bgqd,bkd->bgqk", q.float(), k.float()) * scale
        return torch.einsum("bgqk,bkd->bgqd", torch.softmax(s, dim=-1), v.float()).to(q.dtype)


def grouped_prefix_causal_attention_reference(
    q: torch.Tensor, k_prefix: torch.Tensor, v_prefix: torch.Tensor, k_suffix: torch.Tensor, v_suffix: torch.Tensor,
    softmax_scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 oracle for one prompt group.

    ``q`` ``[G, Lq, Hq, D]`` (completion queries), ``k_prefix``/``v_prefix`` ``[P, Hkv, D]`` (the
    shared prompt), ``k_suffix``/``v_suffix`` ``[G, Lq, Hkv, D]`` (each completion's own K/V).
    Query ``i`` of completion ``g`` sees all P prompt keys and suffix keys ``0..i`` of ``g``.
    Returns ``(out [G, Lq, Hq, D] fp32, lse [G, Hq, Lq] fp32)``.
    """
    g, lq, hq, d = q.shape
    hkv = k_prefix.shape[1]
    rep = hq // hkv
    scale = 1.0 / math.sqrt(d) if softmax_scale is None else softmax_scale
    qf = q.float().permute(0, 2, 1, 3)  # G,Hq,Lq,D
    kp = k_prefix.float().permute(1, 0, 2).repeat_interleave(rep, 0)  # Hq,P,D
    vp = v_prefix.float().permute(1, 0, 2).repeat_interleave(rep, 0)
    ks = k_suffix.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)  # G,Hq,Lq,D
    vs = v_suffix.float().permute(0, 2, 1, 3).repeat_interleave(rep, 1)
    s_p = torch.einsum("ghqd,hkd->ghqk", qf, kp) * scale
    s_s = torch.einsum("ghqd,ghkd->ghqk", qf, ks) * scale
    tri = torch.ones(lq, lq, dtype=torch.bool, device=q.device).tril()
    s_s = s_s.masked_fill(~tri, float("-inf"))
    s = torch.cat([s_p, s_s], dim=-1)
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse[..., None])
    out = torch.einsum("ghqk,hkd->ghqd", p[..., : kp.shape[1]], vp) + torch.einsum(
        "ghqk,ghkd->ghqd", p[..., kp.shape[1] :], vs
    )
    return out.permute(0, 2, 1, 3).contiguous(), lse


__all__ = ["NativeAttentionOp", "NativePrefixSharedAttentionOp", "grouped_prefix_causal_attention_reference"]
