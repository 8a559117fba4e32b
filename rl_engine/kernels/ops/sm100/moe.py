"""Mixture-of-experts FFN on sm_100a kernels: top-k routing, dispatch, grouped expert GEMMs, combine.

Layout: assignments ``(token, j)`` are grouped expert by expert into "slots"; every expert's block is
padded to a multiple of 128 rows (at least one block), so a 128-row GEMM tile never straddles two
experts and the per-expert weight gradient contracts over whole 64-row blocks.  The slot order inside
an expert is the assignment order (token-major), which fixes every summation order: forward, backward
and the weight gradients are bitwise reproducible.

    xs   = gather_rows(x, src_row)                        dispatch            [S, H]
    h1   = grouped_gemm(xs, W1)  -> swiglu -> grouped_gemm(., W2) = y         [S, H]
    out  = combine(y, slot, weight)                        weighted gather-sum [T, H]

The expert GEMMs run on the shared tcgen05 mainloop in its grouped modes (``csrc/common/gemm_sm100.cuh``).
With expert parallelism (``rl_engine.parallel.expert_parallel``) the same gather / combine kernels take
peer pointers: dispatch stores rows straight into the owning rank's slot buffer over NVLink and combine
reads the expert outputs back from the peers -- no NCCL all-to-all.

The reference has no MoE operator; ``NativeMoEOp`` below is the PyTorch oracle used by the tests.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import torch

from rl_engine.kernels.ops.base import require_ext

BLOCK = 128


class _RouteTopK(torch.autograd.Function):
    """Softmax over all experts, top-k, renormalisation in ONE kernel; the backward kernel writes the logits' gradient
    row (the renormalised weights are a softmax over the selected logits)."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, k: int):
        idx, weights = require_ext().moe_topk(logits.contiguous(), int(k))
        ctx.save_for_backward(idx, weights)
        ctx.experts = logits.shape[1]
        ctx.mark_non_differentiable(idx)
        return idx, weights

    @staticmethod
    def backward(ctx, _didx, dweights):
        idx, weights = ctx.saved_tensors
        return require_ext().moe_topk_bwd(idx, weights, dweights.float().contiguous(), ctx.experts), None


def route_topk(router_logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """(expert ids int32 [T, k], renormalised weights fp32 [T, k]); differentiable w.r.t. the logits.

    On the GPU selection and weights come from the ``moe_topk`` kernel (ties -> lower expert id) and the gradient from
    ``moe_topk_bwd``; the portable path below spells the same function with PyTorch ops."""
    logits = router_logits.float()
    if logits.is_cuda:
        return _RouteTopK.apply(logits, int(k))
    probs = torch.softmax(logits.detach(), dim=-1)
    # stable descending sort reproduces the kernel's tie rule
    idx = torch.sort(probs, dim=-1, descending=True, stable=True).indices[:, :k].to(torch.int32)
    probs = torch.softmax(logits, dim=-1)
    picked = probs.gather(1, idx.long())
    return idx, picked / picked.sum(dim=-1, keepdim=True)


@dataclass
class DispatchPlan:
    slot: torch.Tensor          # int32 [T, k]   slot of every assignment
    src_row: torch.Tensor       # int32 [S]      token feeding each slot, -1 for padding
    tile_group: torch.Tensor    # int32 [S/128]  expert of every 128-row tile
    offsets: torch.Tensor       # int32 [E + 1]  padded slot offsets per expert
    counts: torch.Tensor        # int64 [E]      real assignments per expert
    num_slots: int              # S (static upper bound, multiple of 128)


def build_dispatch_plan(expert_idx: torch.Tensor, num_experts: int) -> DispatchPlan:
    """Index plumbing (no host synchronisation): slot tables for ``expert_idx`` int32 ``[T, k]``.

    On the GPU three small kernels (``moe_build_plan``: chunk histograms, per-expert prefix + padded offsets, placement)
    replace the dozen framework index ops of the portable path below; both produce identical tables."""
    t, k = expert_idx.shape
    dev = expert_idx.device
    if expert_idx.is_cuda and expert_idx.dtype == torch.int32 and t * k > 0:
        num_slots = (t * k + num_experts * BLOCK + BLOCK - 1) // BLOCK * BLOCK
        slot, src_row, tile_group, offsets, counts = require_ext().moe_build_plan(
            expert_idx.contiguous(), int(num_experts), int(num_slots), int(num_experts - 1))
        return DispatchPlan(slot, src_row, tile_group, offsets, counts.long(), num_slots)
    flat = expert_idx.reshape(-1).long()
    order = torch.argsort(flat, stable=True)                 # assignments by (expert, assignment id)
    counts = torch.bincount(flat, minlength=num_experts)
    padded = torch.clamp((counts + BLOCK - 1) // BLOCK, min=1) * BLOCK
    offsets = torch.zeros(num_experts + 1, dtype=torch.long, device=dev)
    offsets[1:] = padded.cumsum(0)
    starts = counts.cumsum(0) - counts
    expert_sorted = flat[order]
    rank_in_expert = torch.arange(t * k, device=dev) - starts[expert_sorted]
    slot_sorted = offsets[expert_sorted] + rank_in_expert
    num_slots = (t * k + num_experts * BLOCK + BLOCK - 1) // BLOCK * BLOCK  # static bound: no .item()
    slot = torch.empty(t * k, dtype=torch.int32, device=dev)
    slot[order] = slot_sorted.to(torch.int32)
    src_row = torch.full((num_slots,), -1, dtype=torch.int32, device=dev)
    src_row[slot_sorted] = (order // k).to(torch.int32)
    tile_start = torch.arange(num_slots // BLOCK, device=dev) * BLOCK
    tile_group = (torch.searchsorted(offsets[1:].contiguous(), tile_start, right=True)).clamp_(max=num_experts - 1)
    return DispatchPlan(slot.view(t, k), src_row, tile_group.to(torch.int32), offsets.to(torch.int32), counts, num_slots)


class _ExpertFFN(torch.autograd.Function):
    """x [T, H], weights [T, k], plan, W1 [E*2F, H], W2 [E*H, F] -> out [T, H]."""

    @staticmethod
    def forward(ctx, x, weights, w1, w2, plan: DispatchPlan, num_experts: int):
        ext = require_ext()
        xs = ext.moe_gather_rows(x, plan.src_row)
        h1 = ext.grouped_gemm(xs, w1, 1, plan.tile_group, num_experts, False, False)
        act = ext.swiglu_packed_fwd(h1)
        y = ext.grouped_gemm(act, w2, 1, plan.tile_group, num_experts, False, False)
        out = ext.moe_combine(y, 0, 0, 0, plan.slot, weights.detach())
        ctx.save_for_backward(xs, h1, act, y, weights.detach(), w1, w2)
        ctx.plan, ctx.num_experts = plan, num_experts
        return out

    @staticmethod
    def backward(ctx, dout):
        ext = require_ext()
        xs, h1, act, y, weights, w1, w2 = ctx.saved_tensors
        plan, e = ctx.plan, ctx.num_experts
        dout = dout.contiguous()
        # weight of the assignment living in each slot (padding slots: src_row = -1, never read)
        slot_weight = torch.zeros(plan.num_slots, dtype=torch.float32, device=dout.device)
        slot_weight[plan.slot.reshape(-1).long()] = weights.reshape(-1)
        dweights = ext.moe_rowdot(dout, y, plan.slot)
        dy = ext.moe_gather_rows(dout, plan.src_row, slot_weight)
        dact = ext.grouped_gemm(dy, w2, 1, plan.tile_group, e, True, False)
        dw2 = ext.grouped_gemm(dy, act, 2, plan.offsets, e, True, False)
        dh1 = ext.swiglu_packed_bwd(h1, dact)
        dxs = ext.grouped_gemm(dh1, w1, 1, plan.tile_group, e, True, False)
        dw1 = ext.grouped_gemm(dh1, xs, 2, plan.offsets, e, True, False)
        dx = ext.moe_combine(dxs, 0, 0, 0, plan.slot, None)
        return dx, dweights, dw1, dw2, None, None


def _fusable(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, num_experts: int) -> bool:
    h = x.shape[-1]
    f2 = w1.shape[0] // num_experts
    return (x.is_cuda and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and w2.dtype == torch.bfloat16
            and h % 128 == 0 and f2 % 128 == 0 and (f2 // 2) % 64 == 0 and x.numel() > 0)


class FusedMoESM100Op:
    """``op(x, router_weight [E, H], w_gate_up [E*2F, H], w_down [E*H, F], top_k)`` -> ``[..., H]``."""

    def __init__(self) -> None:
        self._native = NativeMoEOp()

    def __call__(self, x, router_weight, w_gate_up, w_down, top_k: int):
        e = router_weight.shape[0]
        if not _fusable(x, w_gate_up, w_down, e):
            return self._native(x, router_weight, w_gate_up, w_down, top_k)
        from rl_engine.kernels.ops.sm100.gemm import gemm

        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
            x2 = x2.contiguous()
        logits = _RouterLogits.apply(x2, router_weight)
        idx, weights = route_topk(logits, top_k)
        plan = build_dispatch_plan(idx, e)
        out = _ExpertFFN.apply(x2, weights, w_gate_up, w_down, plan, e)
        return out.reshape(x.shape)


class _RouterLogits(torch.autograd.Function):
    """fp32 router logits on the tcgen05 GEMM (bf16 operands, fp32 accumulate and output)."""

    @staticmethod
    def forward(ctx, x2, router_weight):
        from rl_engine.kernels.ops.sm100.gemm import gemm

        ctx.save_for_backward(x2, router_weight)
        return gemm(x2, router_weight.contiguous(), out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dlogits):
        from rl_engine.kernels.ops.sm100.gemm import gemm

        x2, rw = ctx.saved_tensors
        d = dlogits.to(torch.bfloat16).contiguous()
        e = d.shape[1]
        if e % 8:
            return (d.float() @ rw.float()).to(x2.dtype), (d.float().t() @ x2.float()).to(rw.dtype)
        return gemm(d, rw.contiguous(), b_mn=True), gemm(d, x2, a_mn=True, b_mn=True)


class NativeMoEOp:
    """PyTorch oracle: same routing rule, dense loop over experts, fp32 math."""

    def __call__(self, x, router_weight, w_gate_up, w_down, top_k: int):
        e = router_weight.shape[0]
        h = x.shape[-1]
        f2 = w_gate_up.shape[0] // e
        x2 = x.reshape(-1, h)
        logits = x2.float() @ router_weight.float().t()
        idx, weights = route_topk(logits, top_k)
        out = torch.zeros(x2.shape, dtype=torch.float32, device=x.device)
        w1 = w_gate_up.float().view(e, f2, h)
        w2 = w_down.float().view(e, h, f2 // 2)
        for expert in range(e):
            hit = idx.long() == expert
            rows = hit.any(dim=1).nonzero().squeeze(-1)
            if rows.numel() == 0:
                continue
            gate_w = (weights * hit).sum(dim=1)[rows]
            xe = x2[rows].float()
            gu = xe @ w1[expert].t()
            act = torch.nn.functional.silu(gu[:, : f2 // 2]) * gu[:, f2 // 2 :]
            out.index_add_(0, rows, (act @ w2[expert].t()) * gate_w[:, None])
        return out.to(x.dtype).reshape(x.shape)
