"""Attention on the tcgen05 flash kernel: packed tokens, shared prefix + causal suffix, GQA, LSE.

Three front ends over one kernel (``csrc/kernels/attention_fwd.cu``):

* ``FlashAttentionSM100Op`` — the registry's ``attn`` op with the reference call signature
  ``op(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False)`` on ``(batch, seq, heads, dim)``
  tensors (reference: ``rl_engine/kernels/ops/cuda/attention/flash_attn.py:10-57`` wraps the
  flash_attn library).
* ``PrefixSharedAttentionSM100Op`` — ``op(q [bs, G, Lq, D], k [bs, Lkv, D], v)``, the non-causal
  shared-K/V form of the reference kernel (``ops/cuda/attention/prefix_shared_attn.py:11-70``).
* ``grouped_prefix_attention`` — what a GRPO training step needs and the reference lacks: a packed
  batch ``[prompt | completion_0 | ... | completion_{G-1}]`` where every completion attends the
  prompt K/V (stored once) and, causally, its own K/V; differentiable.

Head dim must be 128 and tensors bf16 for the kernel; other cases go to the PyTorch oracle.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.attention import NativeAttentionOp, NativePrefixSharedAttentionOp

TILE = 128


@dataclass(frozen=True)
class PackedLayout:
    """Device tables describing which key ranges each packed sequence attends."""

    seqs: torch.Tensor   # int32 [S, 8]: q_start, q_len, pk_start, pk_len, sk_start, sk_len, 0, 0
    tiles: torch.Tensor  # int32 [n_tiles, 2]: (sequence, first query row in the sequence)
    host_seqs: Tuple[Tuple[int, ...], ...]
    causal: bool


_LAYOUT_CACHE: Dict[Tuple, PackedLayout] = {}


def make_layout(seqs: Sequence[Sequence[int]], causal: bool, device) -> PackedLayout:
    """``seqs``: tuples ``(q_start, q_len, pk_start, pk_len, sk_start, sk_len)``."""
    key = (tuple(tuple(int(x) for x in s) for s in seqs), bool(causal), str(device))
    hit = _LAYOUT_CACHE.get(key)
    if hit is not None:
        return hit
    rows: List[List[int]] = []
    tiles: List[List[int]] = []
    for idx, s in enumerate(key[0]):
        q_start, q_len, pk_start, pk_len, sk_start, sk_len = s
        if causal and sk_len and sk_len != q_len:
            raise ValueError("causal attention needs self key length == query length for every sequence")
        rows.append([q_start, q_len, pk_start, pk_len, sk_start, sk_len, 0, 0])
        tiles.extend([idx, q0] for q0 in range(0, q_len, TILE))
    layout = PackedLayout(
        seqs=torch.tensor(rows, dtype=torch.int32, device=device).reshape(-1, 8),
        tiles=torch.tensor(tiles, dtype=torch.int32, device=device).reshape(-1, 2),
        host_seqs=key[0],
        causal=bool(causal),
    )
    if len(_LAYOUT_CACHE) > 64:
        _LAYOUT_CACHE.clear()
    _LAYOUT_CACHE[key] = layout
    return layout


def grpo_group_layout(prompt_len: int, num_completions: int, completion_len: int, device, base: int = 0) -> PackedLayout:
    """Packed ``[prompt | G completions]``: the prompt is causal on itself; completion g sees the whole prompt
    plus its own tokens causally."""
    seqs = [(base, prompt_len, 0, 0, base, prompt_len)]
    for g in range(num_completions):
        start = base + prompt_len + g * completion_len
        seqs.append((start, completion_len, base, prompt_len, start, completion_len))
    return make_layout(seqs, True, device)


def _kernel_ok(q: torch.Tensor, k: torch.Tensor) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 128


def _packed(t: torch.Tensor) -> torch.Tensor:
    t = t if (t.stride(2) == 1 and t.stride(1) == 128 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()
    return t


def packed_attention_forward(q, k, v, layout: PackedLayout, softmax_scale: Optional[float] = None, want_lse: bool = True):
    """``q [Tq, Hq, 128]``, ``k``/``v`` ``[Tkv, Hkv, 128]`` -> ``(out [Tq, Hq, 128], lse [Hq, Tq])``."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else float(softmax_scale)
    out, lse = require_ext().attention_fwd(
        _packed(q), _packed(k), _packed(v), layout.seqs, layout.tiles, layout.causal, scale, want_lse
    )
    return out, lse


def _reference_backward(q, k, v, out, lse, dout, layout: PackedLayout, scale: float):
    """Interim fp32 PyTorch backward (per sequence) using the saved global LSE."""
    hq, hkv = q.shape[1], k.shape[1]
    rep = hq // hkv
    dq = torch.zeros_like(q, dtype=torch.float32)
    dk = torch.zeros_like(k, dtype=torch.float32)
    dv = torch.zeros_like(v, dtype=torch.float32)
    delta = (dout.float() * out.float()).sum(-1)  # [Tq, Hq]
    for (q_start, q_len, pk_start, pk_len, sk_start, sk_len) in layout.host_seqs:
        qs = slice(q_start, q_start + q_len)
        qf = q[qs].float().transpose(0, 1)            # Hq, Lq, D
        dof = dout[qs].float().transpose(0, 1)
        lse_s = lse[:, qs]                             # Hq, Lq
        dl = delta[qs].transpose(0, 1)                 # Hq, Lq
        for (k0, klen, masked) in ((pk_start, pk_len, False), (sk_start, sk_len, layout.causal)):
            if klen == 0:
                continue
            ks = slice(k0, k0 + klen)
            kf = k[ks].float().transpose(0, 1).repeat_interleave(rep, 0)  # Hq, Lk, D
            vf = v[ks].float().transpose(0, 1).repeat_interleave(rep, 0)
            s = torch.einsum("hqd,hkd->hqk", qf, kf) * scale
            if masked:
                tri = torch.ones(q_len, klen, dtype=torch.bool, device=q.device).tril()
                s = s.masked_fill(~tri, float("-inf"))
            p = torch.exp(s - lse_s[..., None])
            dp = torch.einsum("hqd,hkd->hqk", dof, vf)
            ds = p * (dp - dl[..., None]) * scale
            dq[qs] += torch.einsum("hqk,hkd->hqd", ds, kf).transpose(0, 1)
            dk_h = torch.einsum("hqk,hqd->hkd", ds, qf)
            dv_h = torch.einsum("hqk,hqd->hkd", p, dof)
            dk[ks] += dk_h.reshape(hkv, rep, klen, -1).sum(1).transpose(0, 1)
            dv[ks] += dv_h.reshape(hkv, rep, klen, -1).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


class _PackedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, layout, scale):
        out, lse = packed_attention_forward(q, k, v, layout, scale, True)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.layout = layout
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        from rl_engine.kernels.ops.sm100 import attention_bwd

        dq, dk, dv = attention_bwd.packed_attention_backward(q, k, v, out, lse, dout.contiguous(), ctx.layout, ctx.scale)
        return dq, dk, dv, None, None


def packed_attention(q, k, v, layout: PackedLayout, softmax_scale: Optional[float] = None) -> torch.Tensor:
    """Differentiable packed attention (see module docstring)."""
    scale = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else float(softmax_scale)
    return _PackedAttention.apply(q, k, v, layout, scale)


def grouped_prefix_attention(q, k, v, prompt_len: int, num_completions: int, completion_len: int,
                             softmax_scale: Optional[float] = None) -> torch.Tensor:
    layout = grpo_group_layout(prompt_len, num_completions, completion_len, q.device)
    return packed_attention(q, k, v, layout, softmax_scale)


class FlashAttentionSM100Op:
    def __init__(self) -> None:
        self._native = NativeAttentionOp()

    def __call__(self, q, k, v, dropout_p: float = 0.0, softmax_scale: Optional[float] = None, causal: bool = False):
        b, sq, hq, d = q.shape
        sk = k.shape[1]
        if dropout_p or not _kernel_ok(q, k) or (causal and sq != sk):
            return self._native(q, k, v, dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal)
        if causal:
            seqs = [(i * sq, sq, 0, 0, i * sk, sk) for i in range(b)]
        else:
            seqs = [(i * sq, sq, i * sk, sk, 0, 0) for i in range(b)]
        layout = make_layout(seqs, causal, q.device)
        out = packed_attention(
            q.reshape(b * sq, hq, d), k.reshape(b * sk, k.shape[2], d), v.reshape(b * sk, v.shape[2], d), layout, softmax_scale
        )
        return out.reshape(b, sq, hq, d)


class PrefixSharedAttentionSM100Op:
    def __init__(self) -> None:
        self._native = NativePrefixSharedAttentionOp()

    def __call__(self, q, k, v, softmax_scale: Optional[float] = None):
        if q.ndim != 4 or k.ndim != 3 or k.shape != v.shape or q.shape[0] != k.shape[0] or q.shape[-1] != k.shape[-1]:
            raise ValueError("expected q [bs, G, len_q, D] and k, v [bs, len_kv, D]")
        if not _kernel_ok(q, k):
            return self._native(q, k, v, softmax_scale)
        bs, g, lq, d = q.shape
        lkv = k.shape[1]
        seqs = [((b * g + i) * lq, lq, b * lkv, lkv, 0, 0) for b in range(bs) for i in range(g)]
        layout = make_layout(seqs, False, q.device)
        out = packed_attention(
            q.reshape(bs * g * lq, 1, d), k.reshape(bs * lkv, 1, d), v.reshape(bs * lkv, 1, d), layout, softmax_scale
        )
        return out.reshape(bs, g, lq, d)
