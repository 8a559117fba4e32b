"""Vocab-parallel fused linear -> log-prob: the cross-rank merge happens INSIDE the GEMM kernel.

Each rank holds ``lm_head_weight[v0:v1]``.  The forward kernel of rank r pushes, for every finished
(row tile, vocab split), a 16-byte record ``(max, sum-exp, sum-exp*z, target-logit)`` per row into
every peer's record buffer with plain NVLink stores and bumps a per-row-tile arrival counter on each
peer; whoever sees a row tile complete merges its records in fixed (rank, split) order.  All ranks
therefore produce bitwise identical log-probs, with no collective call: 16 bytes per row per split
cross NVLink instead of the reference's three ``[N]`` all-reduces plus five validation collectives
(``rl_engine/kernels/ops/cuda/loss/linear_logp.py:141-171``).

Backward: per token chunk each rank forms ``dz`` for its shard and ``dz @ W_shard`` into a symmetric
bf16 buffer; after one device-side barrier every rank sums the partial ``grad_hidden`` rows of all
ranks in rank order (``peer_sum``).  ``grad_weight`` is local to the shard.

Shards may be uneven but must tile ``[0, V)``; that is verified once per (group, shard) with a host
collective and cached.
"""

from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.linear_logp import check_linear_logp_args
from rl_engine.parallel.symmetric import SymmetricMemory

_PARTITIONS: Dict[Tuple, Tuple] = {}
_WORKSPACES: Dict[Tuple, "_TPWorkspace"] = {}


def _partition(tp_group, v_start: int, v_local: int, v_global: Optional[int]):
    """-> (global vocab, per-rank (start, size) list); raises like the reference's validators."""
    import torch.distributed as dist

    key = (id(tp_group), v_start, v_local, v_global)
    hit = _PARTITIONS.get(key)
    if hit is not None:
        return hit
    world = dist.get_world_size(tp_group)
    table = [None] * world
    dist.all_gather_object(table, (int(v_start), int(v_local), v_global), group=tp_group)
    spans = sorted((s, s + n) for s, n, _ in table)
    cursor = 0
    for start, end in spans:
        if end <= start:
            raise ValueError(f"invalid TP vocab shard range [{start}, {end}).")
        if start != cursor:
            raise ValueError(f"TP vocab shards must form a contiguous [0, V) partition; got ranges={spans}.")
        cursor = end
    for _s, _n, g in table:
        if g is not None and int(g) != cursor:
            raise ValueError(f"global_vocab_size must match the TP vocab partition size: got {g}, covered {cursor}.")
    hit = _PARTITIONS[key] = (cursor, [(s, n) for s, n, _ in table])
    return hit


class _TPWorkspace:
    def __init__(self, tp_group, device, records: int, n_pad: int, tiles_m: int, chunk: int, hidden_dim: int) -> None:
        self.records, self.n_pad, self.cap = records, n_pad, max(1024, 2 * tiles_m)
        self.chunk, self.hidden_dim = chunk, hidden_dim
        nbytes = 2 * records * n_pad * 16 + 2 * self.cap * 4 + 2 * chunk * hidden_dim * 2 + (1 << 16)
        self.mem = SymmetricMemory(nbytes, group=tp_group, device=device)
        self.partials = [self.mem.alloc((records * n_pad * 4,), torch.float32) for _ in range(2)]
        self.counters = [self.mem.alloc((self.cap,), torch.int32) for _ in range(2)]
        self.gh_part = [self.mem.alloc((chunk, hidden_dim), torch.bfloat16) for _ in range(2)]
        self.calls = 0
        self.chunk_calls = 0
        self.mem.barrier()

    def fits(self, records, n_pad, tiles_m, chunk, hidden_dim) -> bool:
        return (records <= self.records and n_pad <= self.n_pad and tiles_m <= self.cap and chunk <= self.chunk
                and hidden_dim == self.hidden_dim)


def _workspace(tp_group, device, records, n_pad, tiles_m, chunk, hidden_dim) -> _TPWorkspace:
    key = (id(tp_group), device.index or 0)
    ws = _WORKSPACES.get(key)
    if ws is None or not ws.fits(records, n_pad, tiles_m, chunk, hidden_dim):
        if ws is not None:
            ws.mem.close()
        ws = _WORKSPACES[key] = _TPWorkspace(tp_group, device, records, n_pad, tiles_m, chunk, hidden_dim)
    return ws


class _TPLinearLogp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, bias, target, v_start, tp_group, shards, chunk_tokens, want_entropy,
                check_vocab=0):
        import torch.distributed as dist

        ext = require_ext()
        rank, world = dist.get_rank(tp_group), dist.get_world_size(tp_group)
        h2 = hidden.reshape(-1, hidden.shape[-1])
        if h2.stride(1) != 1 or h2.stride(0) % 8 or h2.data_ptr() % 16:
            h2 = h2.contiguous()
        w = weight if (weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0) else weight.contiguous()
        t = target.reshape(-1).to(device=h2.device, dtype=torch.long).contiguous()
        n, d = h2.shape
        per_rank_items = []
        n_pad = tiles_m = 0
        for (_s, size) in shards:
            items, n_pad, tiles_m = ext.linear_logp_workspace_shape(n, size, world)
            per_rank_items.append(items)
        chunk = max(128, min(chunk_tokens, (n + 127) // 128 * 128))
        ws = _workspace(tp_group, h2.device, sum(per_rank_items), n_pad, tiles_m, chunk, d)
        parity = ws.calls % 2
        ws.calls += 1
        logp, lse, ent = ext.linear_logp_fwd(
            h2, w, t, bias, v_start, rank, world, sum(per_rank_items[:rank]), sum(per_rank_items),
            ws.partials[parity].ptrs, ws.counters[parity].ptrs, ws.counters[1 - parity].local.data_ptr(), ws.cap,
            True, bool(want_entropy), ws.mem.wait_limit_ms, int(check_vocab),
        )
        ctx.save_for_backward(h2, w, t, lse, *(() if bias is None else (bias,)))
        ctx.meta = (bias is not None, hidden.shape, v_start, tp_group, chunk)
        lead = hidden.shape[:-1]
        if want_entropy:
            ctx.mark_non_differentiable(ent)
            return logp.reshape(lead), ent.reshape(lead)
        return logp.reshape(lead), None

    @staticmethod
    def backward(ctx, grad_logp, _grad_ent):
        from rl_engine.kernels.ops.sm100.linear_logp import _dz_workspace

        ext = require_ext()
        has_bias, hidden_shape, v_start, tp_group, chunk = ctx.meta
        h2, w, t, lse, *rest = ctx.saved_tensors
        bias = rest[0] if has_bias else None
        n, d = h2.shape
        v = w.shape[0]
        ws = _WORKSPACES[(id(tp_group), h2.device.index or 0)]
        g = grad_logp.reshape(-1).float().contiguous()
        dz_buf = _dz_workspace(h2.device, chunk, v)
        grad_h = torch.empty(n, d, dtype=h2.dtype, device=h2.device)
        grad_w = torch.zeros(v, d, dtype=torch.float32, device=w.device) if ctx.needs_input_grad[1] else None
        grad_b = torch.zeros(v, dtype=torch.float32, device=w.device) if has_bias else None
        for i0 in range(0, n, chunk):
            i1 = min(i0 + chunk, n)
            rows = i1 - i0
            dz = dz_buf[:rows, :v]
            ext.linear_logp_dz(h2[i0:i1], w, t[i0:i1], bias, lse[i0:i1], g[i0:i1], v_start, dz)
            part = ws.gh_part[ws.chunk_calls % 2]
            ws.chunk_calls += 1
            ext.gemm(dz, w, False, True, part.local[:rows], False, False, 1.0)
            ws.mem.barrier()
            ext.peer_sum(part.ptrs, rows * d, False, grad_h[i0:i1])
            if grad_w is not None:
                ext.gemm(dz, h2[i0:i1], True, True, grad_w, True, True, 1.0)
            if grad_b is not None:
                grad_b += dz.float().sum(0)
        return (
            grad_h.reshape(hidden_shape), None if grad_w is None else grad_w.to(w.dtype),
            None if grad_b is None else grad_b.to(bias.dtype), None, None, None, None, None, None, None,
        )


def tensor_parallel_linear_logp_fused(
    hidden, lm_head_weight, target_ids, bias=None, *, tp_group: Any, vocab_start_index: int = 0,
    global_vocab_size: Optional[int] = None, check_targets="device", chunk_tokens: int = 4096,
    with_entropy: bool = False,
):
    """``check_targets``: ``"device"`` (the kernel flags out-of-range ids in the error word), ``"sync"`` (host check,
    raises at once) or ``"off"``; booleans mean ``"device"`` / ``"off"``."""
    from rl_engine.kernels.ops.sm100.linear_logp import target_check_mode

    mode = target_check_mode(check_targets)
    check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
    v_global, shards = _partition(tp_group, int(vocab_start_index), lm_head_weight.shape[0], global_vocab_size)
    if mode == "sync" and target_ids.numel():
        lo, hi = (int(x) for x in torch.aminmax(target_ids))
        if lo < 0 or hi >= v_global:
            raise ValueError(
                f"target_ids out of range: expected [0, {v_global - 1}], got [{lo}, {hi}]. "
                "Mask or filter padding / ignore-index values (e.g. -100) before this op."
            )
    logp, ent = _TPLinearLogp.apply(
        hidden, lm_head_weight, bias, target_ids, int(vocab_start_index), tp_group, tuple(shards), int(chunk_tokens),
        bool(with_entropy), int(v_global) if mode == "device" else 0,
    )
    return (logp, ent) if with_entropy else logp
