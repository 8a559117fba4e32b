"""Context parallelism for causal attention over long sequences.

The sequence of ``S = 2 * W * C`` tokens is cut into ``2 W`` chunks of ``C`` tokens; rank ``r`` owns
chunks ``r`` and ``2 W - 1 - r`` (zig-zag), which gives every rank the same amount of causal work.

Forward: every rank stores its K/V chunks straight into all peers' gathered K/V buffers in symmetric
memory (one peer-store kernel per tensor; no NCCL, no ring of dependent hops: behind NVSwitch every
peer is one hop away), then runs the tcgen05 flash kernel on its local queries against the gathered
keys.  In the kernel's layout table the keys that precede a chunk are a non-causal "prefix" range and the
chunk itself is the causal "self" range, so no masking work is spent on fully visible blocks.

Backward: K/V are gathered again (cheaper than keeping ``S`` keys alive per layer), the local
queries produce gradient contributions for every key they saw, the contributions are published in
symmetric memory and every rank sums, in fixed rank order, the ``W`` contributions to the chunks it
owns (``peer_sum``): deterministic, no atomics.

The reference has no context-parallel or ring attention; the oracle is the single-GPU packed attention
(and through it the fp32 PyTorch attention) over the whole sequence.
"""

from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.parallel.symmetric import SymmetricMemory


def zigzag_chunks(rank: int, world: int) -> Tuple[int, int]:
    """The two chunk ids (of ``2 * world``) owned by ``rank``."""
    return rank, 2 * world - 1 - rank


def shard_sequence(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rows of ``x [S, ...]`` owned by ``rank``: its two chunks, lower chunk first."""
    s = x.shape[0]
    if s % (2 * world):
        raise ValueError(f"sequence length {s} is not a multiple of 2 * world = {2 * world}")
    c = s // (2 * world)
    a, b = zigzag_chunks(rank, world)
    return torch.cat([x[a * c:(a + 1) * c], x[b * c:(b + 1) * c]], dim=0)


def unshard_sequence(parts: List[torch.Tensor]) -> torch.Tensor:
    """Inverse of ``shard_sequence`` given every rank's shard (rank order)."""
    world = len(parts)
    c = parts[0].shape[0] // 2
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = zigzag_chunks(r, world)
        chunks[a], chunks[b] = p[:c], p[c:]
    return torch.cat(chunks, dim=0)  # type: ignore[arg-type]


def local_layout_rows(rank: int, world: int, chunk: int) -> List[Tuple[int, int, int, int, int, int]]:
    """Layout rows ``(q_start, q_len, prefix_start, prefix_len, self_start, self_len)`` for the two local
    query chunks against the gathered keys."""
    rows = []
    for i, cid in enumerate(zigzag_chunks(rank, world)):
        rows.append((i * chunk, chunk, 0, cid * chunk, cid * chunk, chunk))
    return rows


class ContextParallelAttention:
    """``op(q [2C, Hq, 128], k [2C, Hkv, 128], v)`` on this rank's zig-zag shard -> ``out [2C, Hq, 128]``."""

    def __init__(self, seq_len: int, kv_heads: int, head_dim: int = 128, group=None,
                 mem: Optional[SymmetricMemory] = None, device: Optional[torch.device] = None) -> None:
        import torch.distributed as dist

        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if seq_len % (2 * self.world):
            raise ValueError(f"sequence length {seq_len} is not a multiple of 2 * world = {2 * self.world}")
        self.seq_len, self.kv_heads, self.head_dim = seq_len, kv_heads, head_dim
        self.chunk = seq_len // (2 * self.world)
        self.row = kv_heads * head_dim
        nbytes = 4 * seq_len * self.row * 2 + (1 << 20)
        self.mem = mem if mem is not None else SymmetricMemory(nbytes, group=group, device=device)
        shape = (seq_len, kv_heads, head_dim)
        self.k_all = self.mem.alloc(shape, torch.bfloat16)
        self.v_all = self.mem.alloc(shape, torch.bfloat16)
        self.dk_all = self.mem.alloc(shape, torch.bfloat16)
        self.dv_all = self.mem.alloc(shape, torch.bfloat16)
        self._layout = None

    # -- pieces -------------------------------------------------------------------------------------
    def layout(self, device):
        from rl_engine.kernels.ops.sm100.attention import make_layout

        if self._layout is None:
            self._layout = make_layout(local_layout_rows(self.rank, self.world, self.chunk), True, device)
        return self._layout

    def gather_kv(self, k: torch.Tensor, v: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Push the local K/V chunks into every rank's gathered buffers; returns the local gathered views."""
        ext = require_ext()
        c = self.chunk
        self.mem.barrier()  # nobody still reads the buffers' previous contents
        for buf, src in ((self.k_all, k), (self.v_all, v)):
            src = src.contiguous()
            for i, cid in enumerate(zigzag_chunks(self.rank, self.world)):
                off = cid * c * self.row * 2
                ext.cast_broadcast(src[i * c:(i + 1) * c], [p + off for p in buf.ptrs], 1)
        self.mem.barrier()  # every chunk has landed everywhere
        return self.k_all.local, self.v_all.local

    def reduce_dkv(self, dk_full: torch.Tensor, dv_full: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Sum the ranks' contributions to the K/V chunks owned here (fixed rank order)."""
        ext = require_ext()
        c = self.chunk
        self.mem.barrier()  # the previous reduction's readers are done
        self.dk_all.local.copy_(dk_full)
        self.dv_all.local.copy_(dv_full)
        self.mem.barrier()
        outs = []
        for buf in (self.dk_all, self.dv_all):
            out = torch.empty(2 * c, self.kv_heads, self.head_dim, dtype=torch.bfloat16, device=dk_full.device)
            for i, cid in enumerate(zigzag_chunks(self.rank, self.world)):
                off = cid * c * self.row * 2
                ext.peer_sum([p + off for p in buf.ptrs], c * self.row, False, out[i * c:(i + 1) * c])
            outs.append(out)
        return outs[0], outs[1]

    def __call__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: Optional[float] = None):
        if q.shape[0] != 2 * self.chunk or k.shape[0] != 2 * self.chunk:
            raise ValueError(f"expected {2 * self.chunk} local tokens, got q {q.shape[0]} and k {k.shape[0]}")
        scale = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else float(softmax_scale)
        return _CPAttention.apply(q, k, v, self, scale)


class _CPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cp: ContextParallelAttention, scale: float):
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        k_all, v_all = cp.gather_kv(k, v)
        out, lse = packed_attention_forward(q, k_all, v_all, cp.layout(q.device), scale, True)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.cp, ctx.scale = cp, scale
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_engine.kernels.ops.sm100.attention_bwd_kernels import fused_backward

        q, k, v, out, lse = ctx.saved_tensors
        cp = ctx.cp
        k_all, v_all = cp.gather_kv(k, v)
        dq, dk_full, dv_full = fused_backward(q, k_all, v_all, out, lse, dout.contiguous(), cp.layout(q.device), ctx.scale)
        dk, dv = cp.reduce_dkv(dk_full, dv_full)
        return dq, dk, dv, None, None


class SharedRow:
    """``share(row [1, n])``: the ``owner`` rank's row on every rank of ``mem``'s group, differentiable.

    Forward: the owner stores its row into every peer's buffer (one peer-store kernel); the other ranks' inputs are
    ignored.  Backward: every rank publishes the gradient it holds, the owner sums them in rank order (``peer_sum``)
    and the other ranks get zeros.  Calls must be issued by all ranks in the same order."""

    def __init__(self, mem: SymmetricMemory, n: int, owner: int = 0) -> None:
        self.mem, self.n, self.owner = mem, int(n), int(owner)
        self.value = mem.alloc((self.n,), torch.bfloat16)
        self.grad = mem.alloc((self.n,), torch.bfloat16)

    def __call__(self, row: torch.Tensor) -> torch.Tensor:
        if row.numel() != self.n or row.dtype != torch.bfloat16:
            raise ValueError(f"expected a bfloat16 row of {self.n} elements")
        return _ShareRow.apply(row, self)


class _ShareRow(torch.autograd.Function):
    @staticmethod
    def forward(ctx, row, shared: SharedRow):
        mem = shared.mem
        mem.barrier()  # the previous value's readers are done
        if mem.rank == shared.owner:
            require_ext().cast_broadcast(row.contiguous().view(-1), list(shared.value.ptrs), 1)
        mem.barrier()
        ctx.shared = shared
        return shared.value.local.clone().view_as(row)

    @staticmethod
    def backward(ctx, grad):
        shared = ctx.shared
        mem = shared.mem
        mem.barrier()  # the previous reduction's readers are done
        shared.grad.local.copy_(grad.reshape(-1))
        mem.barrier()
        if mem.rank == shared.owner:
            out = torch.empty(shared.n, dtype=torch.bfloat16, device=grad.device)
            require_ext().peer_sum(list(shared.grad.ptrs), shared.n, False, out)
        else:
            out = torch.zeros(shared.n, dtype=torch.bfloat16, device=grad.device)
        return out.view_as(grad).to(grad.dtype), None
