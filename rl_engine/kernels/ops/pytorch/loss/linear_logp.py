"""CPU/PyTorch oracle for fused linear -> selected-token log-prob, incl. vocab-parallel TP.

Parity: reference ``rl_engine/kernels/ops/pytorch/loss/linear_logp.py``:
* ``NativeLinearLogpOp`` (``:442-520``): materialising ``F.linear + log_softmax + gather`` oracle,
  fp32 output, kwargs ``tp_group / vocab_start_index / global_vocab_size``.
* ``should_use_tensor_parallel_linear_logp`` (``:58-83``) decision rules and error messages.
* TP autograd function (``:217-335``): per-rank online (max, sum-exp, target-logit, owner) stats
  over the local vocab shard, cross-rank merge, chunked recompute backward with an fp32
  all-reduce of ``grad_hidden``.  Shards may be uneven but must tile ``[0, V)``.
* ``chunked_linear_logp_backward`` (``:383-439``): the no-``[N,V]`` backward used on one rank.

This module is the *oracle and CPU path*: it uses ``torch.distributed`` collectives (Gloo on CPU).
The GPU path (``ops/sm100/linear_logp.py``) does the same merge inside the kernel over NVLink
peer memory with a fixed rank order.
"""

from __future__ import annotations

from typing import Any, Optional, Tuple

import torch
import torch.nn.functional as F

BWD_CHUNK_ELEMS = 1 << 24
_HALF = (torch.float16, torch.bfloat16)


def _dist():
    import torch.distributed as dist

    if not dist.is_available():
        raise RuntimeError("tensor-parallel linear_logp requires torch.distributed.")
    if not dist.is_initialized():
        raise RuntimeError("tensor-parallel linear_logp requires an initialized process group.")
    return dist


def _tp_world(tp_group: Any) -> int:
    return 1 if tp_group is None else _dist().get_world_size(group=tp_group)


def should_use_tensor_parallel_linear_logp(
    tp_group: Any, vocab_start_index: int, global_vocab_size: Optional[int], local_vocab_size: int
) -> bool:
    explicit = tp_group is not None or vocab_start_index != 0 or global_vocab_size is not None
    if not explicit:
        if local_vocab_size <= 0:
            raise ValueError("lm_head_weight must contain at least one vocab row.")
        return False
    world = _tp_world(tp_group)
    if world > 1:
        return True
    if local_vocab_size <= 0:
        raise ValueError("lm_head_weight must contain at least one vocab row.")
    if vocab_start_index != 0:
        raise ValueError("vocab_start_index requires a tensor-parallel group.")
    if global_vocab_size is not None and int(global_vocab_size) != local_vocab_size:
        raise ValueError(
            "global_vocab_size differs from the local vocab size, but no multi-rank "
            "tensor-parallel group was provided."
        )
    return False


def check_linear_logp_args(hidden, weight, target_ids, bias) -> None:
    if tuple(hidden.shape[:-1]) != tuple(target_ids.shape):
        raise ValueError(
            f"hidden leading shape {tuple(hidden.shape[:-1])} must match "
            f"target_ids shape {tuple(target_ids.shape)}"
        )
    if weight.shape[-1] != hidden.shape[-1]:
        raise ValueError(f"hidden dim {hidden.shape[-1]} must match lm_head_weight dim {weight.shape[-1]}")
    if weight.device != hidden.device:
        raise ValueError(f"lm_head_weight device {weight.device} must match hidden device {hidden.device}")
    if bias is not None:
        if bias.ndim != 1 or bias.numel() != weight.shape[0]:
            raise ValueError(
                f"bias must be 1-D with local V={weight.shape[0]} elements, got shape {tuple(bias.shape)}"
            )
        if bias.device != hidden.device:
            raise ValueError(f"bias device {bias.device} must match hidden device {hidden.device}")


def validate_tp_vocab_partition(
    *, tp_group: Any, device: torch.device, vocab_start_index: int, local_vocab_size: int,
    global_vocab_size: Optional[int],
) -> int:
    """All ranks agree that the shards tile ``[0, V)``; returns V."""
    dist = _dist()
    world = dist.get_world_size(tp_group)
    mine = torch.tensor(
        [vocab_start_index, vocab_start_index + local_vocab_size,
         0 if global_vocab_size is None else 1, 0 if global_vocab_size is None else int(global_vocab_size)],
        dtype=torch.long, device=device,
    )
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=tp_group)
    table = torch.stack(gathered).cpu().tolist()
    spans = sorted((row[0], row[1]) for row in table)
    cursor = 0
    for start, end in spans:
        if end <= start:
            raise ValueError(f"invalid TP vocab shard range [{start}, {end}).")
        if start != cursor:
            raise ValueError(f"TP vocab shards must form a contiguous [0, V) partition; got ranges={spans}.")
        cursor = end
    for row in table:
        if row[2] and row[3] != cursor:
            raise ValueError(
                f"global_vocab_size must match the TP vocab partition size: got {row[3]}, covered {cursor}."
            )
    return cursor if global_vocab_size is None else int(global_vocab_size)


def validate_global_targets(target_1d: torch.Tensor, global_vocab_size: int, tp_group: Any = None) -> None:
    if target_1d.numel():
        lo, hi = int(target_1d.min()), int(target_1d.max())
    else:
        lo, hi = global_vocab_size, -1
    if tp_group is not None:
        dist = _dist()
        span = torch.tensor([-lo, hi], dtype=torch.long, device=target_1d.device)
        dist.all_reduce(span, op=dist.ReduceOp.MAX, group=tp_group)
        lo, hi = -int(span[0]), int(span[1])
    if hi >= lo and (lo < 0 or hi >= global_vocab_size):
        raise ValueError(
            f"target_ids out of range: expected [0, {global_vocab_size - 1}], got [{lo}, {hi}]. "
            "Mask or filter padding / ignore-index values (e.g. -100) before this op."
        )


def _logits(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """fp32 logits; half inputs are upcast so the oracle never accumulates in half."""
    if x.dtype in _HALF or w.dtype in _HALF:
        z = x.float() @ w.float().t()
        return z if b is None else z + b.float()
    z = x @ w.t()
    z = z if b is None else z + b
    return z.float()


def local_linear_logp_stats(
    hidden_2d: torch.Tensor, weight: torch.Tensor, target_1d: torch.Tensor, bias: Optional[torch.Tensor],
    *, vocab_start_index: int, chunk_elems: int = BWD_CHUNK_ELEMS,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Online (max, sum-exp, target-logit, owner-count) over this rank's vocab rows."""
    n, v_local = hidden_2d.shape[0], weight.shape[0]
    dev = hidden_2d.device
    run_max = torch.full((n,), float("-inf"), device=dev)
    run_sum = torch.zeros(n, device=dev)
    tgt = torch.zeros(n, device=dev)
    owners = torch.zeros(n, dtype=torch.int32, device=dev)
    step = max(1, min(v_local, chunk_elems // max(n, 1)))
    for v0 in range(0, v_local, step):
        v1 = min(v0 + step, v_local)
        z = _logits(hidden_2d, weight[v0:v1], None if bias is None else bias[v0:v1])
        new_max = torch.maximum(run_max, z.max(dim=-1).values)
        run_sum = run_sum * torch.exp(run_max - new_max) + torch.exp(z - new_max[:, None]).sum(-1)
        run_max = new_max
        local = target_1d - (vocab_start_index + v0)
        mine = (local >= 0) & (local < v1 - v0)
        picked = z.gather(1, local.clamp(0, v1 - v0 - 1)[:, None]).squeeze(1)
        tgt = torch.where(mine, picked, tgt)
        owners = owners + mine.to(torch.int32)
    return run_max, run_sum, tgt, owners


def _recompute_grads(
    g: torch.Tensor, hidden_2d: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
    target_local: torch.Tensor, lse: Optional[torch.Tensor], chunk_elems: int,
):
    """Token-chunked ``dz = g * (onehot - softmax)`` and its three products, never ``[N, V]``.

    ``lse`` given: softmax is ``exp(z - lse)`` (global normaliser, TP).  ``lse`` None: recompute a
    self-normalising softmax per chunk (single rank).
    """
    n, d = hidden_2d.shape
    v = weight.shape[0]
    half = hidden_2d.dtype in _HALF or weight.dtype in _HALF
    grad_h = torch.empty(n, d, dtype=torch.float32, device=hidden_2d.device)
    grad_w = torch.zeros(v, d, dtype=torch.float32, device=weight.device)
    grad_b = None if bias is None else torch.zeros(v, dtype=torch.float32, device=weight.device)
    step = max(1, min(n, chunk_elems // max(v, 1)))
    for i0 in range(0, n, step):
        i1 = min(i0 + step, n)
        x = hidden_2d[i0:i1]
        z = _logits(x, weight, bias)
        dz = -(torch.softmax(z, dim=-1) if lse is None else torch.exp(z - lse[i0:i1, None]))
        t = target_local[i0:i1]
        mine = (t >= 0) & (t < v)
        dz[torch.arange(i1 - i0, device=dz.device)[mine], t[mine]] += 1.0
        dz *= g[i0:i1, None]
        if half:
            grad_h[i0:i1] = dz @ weight.float()
            grad_w += dz.t() @ x.float()
        else:
            dzc = dz.to(weight.dtype)
            grad_h[i0:i1] = (dzc @ weight).float()
            grad_w += (dzc.t() @ x).float()
        if grad_b is not None:
            grad_b += dz.sum(0)
    return grad_h, grad_w, grad_b


def chunked_linear_logp_backward(
    grad_logp, hidden_2d, weight, target_1d, bias_t, *, has_bias, lead_shape, hidden_dtype, weight_dtype,
    bias_dtype, chunk_elems: int = BWD_CHUNK_ELEMS,
):
    g = grad_logp.reshape(-1).float()
    gh, gw, gb = _recompute_grads(
        g, hidden_2d, weight, bias_t if has_bias else None, target_1d.long(), None, chunk_elems
    )
    return (
        gh.to(hidden_dtype).reshape(tuple(lead_shape) + (hidden_2d.shape[1],)),
        gw.to(weight_dtype),
        None if gb is None else gb.to(bias_dtype),
    )


class _VocabParallelLinearLogp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, bias, target_ids, vocab_start_index, global_vocab_size, tp_group):
        dist = _dist()
        x = hidden.reshape(-1, hidden.shape[-1]).contiguous()
        w = weight.contiguous()
        t = target_ids.reshape(-1).to(device=x.device, dtype=torch.long)
        v_total = validate_tp_vocab_partition(
            tp_group=tp_group, device=x.device, vocab_start_index=vocab_start_index,
            local_vocab_size=w.shape[0], global_vocab_size=global_vocab_size,
        )
        validate_global_targets(t, v_total, tp_group)
        m_loc, s_loc, z_t, owners = local_linear_logp_stats(x, w, t, bias, vocab_start_index=vocab_start_index)
        m = m_loc.clone()
        dist.all_reduce(m, op=dist.ReduceOp.MAX, group=tp_group)
        packed = torch.stack([s_loc * torch.exp(m_loc - m), z_t, owners.float()])
        dist.all_reduce(packed, op=dist.ReduceOp.SUM, group=tp_group)
        if bool((packed[2] != 1).any()):
            raise ValueError(
                "target_ids must be covered by exactly one TP vocab shard; check "
                "vocab_start_index and global_vocab_size."
            )
        lse = m + torch.log(packed[0])
        ctx.save_for_backward(x, w, t, lse, *(() if bias is None else (bias,)))
        ctx.meta = (bias is not None, hidden.shape, hidden.dtype, weight.dtype,
                    None if bias is None else bias.dtype, vocab_start_index, tp_group)
        return (packed[1] - lse).reshape(hidden.shape[:-1])

    @staticmethod
    def backward(ctx, grad_logp):
        dist = _dist()
        has_bias, shape, h_dt, w_dt, b_dt, v0, group = ctx.meta
        x, w, t, lse, *rest = ctx.saved_tensors
        bias = rest[0] if has_bias else None
        gh, gw, gb = _recompute_grads(grad_logp.reshape(-1).float(), x, w, bias, t - v0, lse, BWD_CHUNK_ELEMS)
        dist.all_reduce(gh, op=dist.ReduceOp.SUM, group=group)
        return gh.to(h_dt).reshape(shape), gw.to(w_dt), None if gb is None else gb.to(b_dt), None, None, None, None


def tensor_parallel_linear_logp(
    hidden, lm_head_weight, target_ids, bias=None, *, tp_group: Any, vocab_start_index: int = 0,
    global_vocab_size: Optional[int] = None,
) -> torch.Tensor:
    check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
    return _VocabParallelLinearLogp.apply(
        hidden, lm_head_weight, bias, target_ids, int(vocab_start_index),
        None if global_vocab_size is None else int(global_vocab_size), tp_group,
    )


class NativeLinearLogpOp:
    def __call__(self, hidden, lm_head_weight, target_ids, bias=None, **kw) -> torch.Tensor:
        return self.apply(hidden, lm_head_weight, target_ids, bias, **kw)

    def apply(
        self, hidden, lm_head_weight, target_ids, bias=None, *, tp_group: Any = None,
        vocab_start_index: int = 0, global_vocab_size: Optional[int] = None,
    ) -> torch.Tensor:
        """Selected-token log-prob ``z[t] - logsumexp(z)`` in float32."""
        check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
        if should_use_tensor_parallel_linear_logp(
            tp_group, int(vocab_start_index), global_vocab_size, lm_head_weight.shape[0]
        ):
            return tensor_parallel_linear_logp(
                hidden, lm_head_weight, target_ids, bias, tp_group=tp_group,
                vocab_start_index=vocab_start_index, global_vocab_size=global_vocab_size,
            )
        z = F.linear(hidden.reshape(-1, hidden.shape[-1]), lm_head_weight, bias).float()
        ids = target_ids.reshape(-1, 1).to(device=z.device, dtype=torch.long)
        return torch.log_softmax(z, dim=-1).gather(1, ids).reshape(hidden.shape[:-1])

    def with_entropy(self, hidden, lm_head_weight, target_ids, bias=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(logp, entropy) oracle: entropy of the full softmax per token, fp32."""
        check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
        z = F.linear(hidden.reshape(-1, hidden.shape[-1]), lm_head_weight, bias).float()
        logp_all = torch.log_softmax(z, dim=-1)
        ids = target_ids.reshape(-1, 1).to(device=z.device, dtype=torch.long)
        ent = -(logp_all.exp() * logp_all).sum(-1)
        lead = hidden.shape[:-1]
        return logp_all.gather(1, ids).reshape(lead), ent.reshape(lead)
