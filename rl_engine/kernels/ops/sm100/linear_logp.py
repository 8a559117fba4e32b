"""Fused linear -> selected-token log-prob (+ entropy) on the tcgen05 kernel, with autograd.

Parity: ``FusedLinearLogpSM90Op`` (``rl_engine/kernels/ops/cuda/loss/linear_logp.py:58-359``):
same call signature ``op(hidden, lm_head_weight, target_ids, bias=None, *, tp_group=None,
vocab_start_index=0, global_vocab_size=None)`` returning float32 log-probs shaped like
``target_ids``; out-of-range (unmasked) targets raise.  Differences:

* forward is ONE kernel including the split/rank merge (the reference launches a GEMM kernel, a
  combine kernel and, under tensor parallelism, three NCCL all-reduces);
* backward never calls a library GEMM: per token chunk a recompute kernel writes
  ``dz = g * (onehot - softmax)`` as bf16 into a pre-allocated chunk workspace, then two tcgen05
  GEMMs form ``grad_hidden`` and accumulate ``grad_weight`` in fp32 in fixed chunk order.  Extra
  memory is constant in the number of tokens: ``chunk * V`` bf16 plus the fp32 ``grad_weight``;
* ``with_entropy`` also returns the softmax entropy per token from the same sweep.

Inputs must be bf16 on a CUDA device for the fused path; anything else goes to the PyTorch oracle.
"""

from __future__ import annotations

import os
from typing import Any, Dict, Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.kernels.ops.pytorch.loss.linear_logp import (
    NativeLinearLogpOp,
    check_linear_logp_args,
    should_use_tensor_parallel_linear_logp,
)

DEFAULT_BWD_CHUNK_TOKENS = 4096


class _LocalWorkspace:
    """Per-device scratch of the forward kernel: split records and two arrival-counter sets.

    The kernel of call ``k`` counts arrivals in set ``k % 2`` and zeroes set ``(k + 1) % 2``, so no
    memset is ever needed between calls (stream order makes this race free on one GPU; the
    tensor-parallel variant in ``rl_engine.parallel`` explains why it also is across ranks).
    """

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.partials: Optional[torch.Tensor] = None
        self.counters: Optional[torch.Tensor] = None
        self.calls = 0

    def ensure(self, records: int, n_pad: int, tiles_m: int) -> None:
        need = records * n_pad * 4
        if self.partials is None or self.partials.numel() < need:
            self.partials = torch.empty(need, dtype=torch.float32, device=self.device)
        if self.counters is None or self.counters.shape[1] < tiles_m:
            cap = max(1024, 2 * tiles_m)
            self.counters = torch.zeros(2, cap, dtype=torch.int32, device=self.device)
            self.calls = 0

    def next_sets(self) -> Tuple[int, int, int]:
        cur = self.calls % 2
        self.calls += 1
        c = self.counters
        return c[cur].data_ptr(), c[1 - cur].data_ptr(), c.shape[1]


_WORKSPACES: Dict[Tuple[int, int], _LocalWorkspace] = {}


def _workspace(device: torch.device) -> _LocalWorkspace:
    # one workspace per (device, stream): launches on different streams must not share counters
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = _WORKSPACES[key] = _LocalWorkspace(device)
    return ws


def _forward_local(hidden2d, weight, target, bias, want_lse: bool, want_entropy: bool, check_vocab: int = 0):
    """``check_vocab`` > 0: the kernel flags target ids outside ``[0, check_vocab)`` in the device error word."""
    ext = require_ext()
    items, n_pad, tiles_m = ext.linear_logp_workspace_shape(hidden2d.shape[0], weight.shape[0], 1)
    ws = _workspace(hidden2d.device)
    ws.ensure(items, n_pad, tiles_m)
    cur, nxt, cap = ws.next_sets()
    return ext.linear_logp_fwd(
        hidden2d, weight, target, bias, 0, 0, 1, 0, items, [ws.partials.data_ptr()], [cur], nxt, cap, want_lse, want_entropy, 0.0,
        int(check_vocab),
    )


_DZ_CACHE: Dict[Tuple[int, int, int], torch.Tensor] = {}


def _dz_workspace(device: torch.device, chunk: int, v_local: int) -> torch.Tensor:
    v_pad = (v_local + 7) // 8 * 8
    key = (device.index or 0, chunk, v_pad)
    buf = _DZ_CACHE.get(key)
    if buf is None:
        buf = _DZ_CACHE[key] = torch.empty(chunk, v_pad, dtype=torch.bfloat16, device=device)
    return buf


def linear_logp_backward_local(
    grad_logp: torch.Tensor, hidden2d: torch.Tensor, weight: torch.Tensor, target: torch.Tensor,
    bias: Optional[torch.Tensor], lse: torch.Tensor, *, vocab_start: int = 0, need_hidden: bool = True,
    need_weight: bool = True, chunk_tokens: int = DEFAULT_BWD_CHUNK_TOKENS, grad_hidden_dtype=torch.bfloat16,
):
    """Chunked recompute backward on one rank's vocab shard.  Returns (grad_h, grad_w fp32, grad_b fp32)."""
    ext = require_ext()
    n, d = hidden2d.shape
    v = weight.shape[0]
    g = grad_logp.reshape(-1).float().contiguous()
    chunk = max(128, min(chunk_tokens, (n + 127) // 128 * 128))
    dz_buf = _dz_workspace(hidden2d.device, chunk, v)
    grad_h = torch.empty(n, d, dtype=grad_hidden_dtype, device=hidden2d.device) if need_hidden else None
    grad_w = torch.zeros(v, d, dtype=torch.float32, device=weight.device) if need_weight else None
    grad_b = torch.zeros(v, dtype=torch.float32, device=weight.device) if bias is not None else None
    for i0 in range(0, n, chunk):
        i1 = min(i0 + chunk, n)
        rows = i1 - i0
        dz = dz_buf[:rows, :v]
        ext.linear_logp_dz(hidden2d[i0:i1], weight, target[i0:i1], bias, lse[i0:i1], g[i0:i1], vocab_start, dz)
        if need_hidden:
            ext.gemm(dz, weight, False, True, grad_h[i0:i1], grad_hidden_dtype == torch.float32, False, 1.0)
        if need_weight:
            ext.gemm(dz, hidden2d[i0:i1], True, True, grad_w, True, True, 1.0)
        if grad_b is not None:
            grad_b += dz.float().sum(0)
    return grad_h, grad_w, grad_b


class _LinearLogp(torch.autograd.Function):
    @staticmethod
    def forward(ctx, hidden, weight, bias, target, want_entropy, chunk_tokens, check_vocab=0):
        h2 = hidden.reshape(-1, hidden.shape[-1])
        if h2.stride(1) != 1 or h2.stride(0) % 8 or h2.data_ptr() % 16:
            h2 = h2.contiguous()
        w = weight if (weight.stride(1) == 1 and weight.stride(0) % 8 == 0 and weight.data_ptr() % 16 == 0) else weight.contiguous()
        t = target.reshape(-1).to(device=h2.device, dtype=torch.long).contiguous()
        logp, lse, ent = _forward_local(h2, w, t, bias, True, bool(want_entropy), check_vocab)
        ctx.save_for_backward(h2, w, t, lse, *(() if bias is None else (bias,)))
        ctx.has_bias = bias is not None
        ctx.hidden_shape = hidden.shape
        ctx.chunk_tokens = chunk_tokens
        lead = hidden.shape[:-1]
        if want_entropy:
            ctx.mark_non_differentiable(ent)
            return logp.reshape(lead), ent.reshape(lead)
        return logp.reshape(lead), None

    @staticmethod
    def backward(ctx, grad_logp, _grad_ent):
        h2, w, t, lse, *rest = ctx.saved_tensors
        bias = rest[0] if ctx.has_bias else None
        gh, gw, gb = linear_logp_backward_local(
            grad_logp, h2, w, t, bias, lse, need_hidden=ctx.needs_input_grad[0], need_weight=ctx.needs_input_grad[1],
            chunk_tokens=ctx.chunk_tokens,
        )
        return (
            None if gh is None else gh.reshape(ctx.hidden_shape),
            None if gw is None else gw.to(w.dtype),
            None if gb is None else gb.to(bias.dtype),
            None, None, None, None,
        )


def target_check_mode(check_targets=None) -> str:
    """``"device"`` (default), ``"sync"`` or ``"off"``, from the argument or ``RL_KERNEL_CHECK_TARGETS``
    (``1`` / ``device``, ``sync``, ``0``)."""
    if check_targets is None:
        check_targets = os.environ.get("RL_KERNEL_CHECK_TARGETS", "device")
    if check_targets in (True, "1", "device", "true", "True"):
        return "device"
    if check_targets in (False, "0", "off", "false", "False"):
        return "off"
    if check_targets == "sync":
        return "sync"
    raise ValueError(f"check_targets must be 'device', 'sync' or 'off', got {check_targets!r}")


class FusedLinearLogpSM100Op:
    """``check_targets``: how unmasked target ids outside ``[0, V)`` are caught.  ``"device"`` (default): the forward
    kernel itself tests every id, makes that row's log-prob NaN and records a bad-argument error that the next
    ``check_device_errors()`` raises -- no host round trip per call (the reference reads ``min`` / ``max`` back on every
    call: ``rl_engine/kernels/ops/cuda/loss/linear_logp.py:353-358``).  ``"sync"``: that host check, raising
    ``ValueError`` at once.  ``"off"``: no check."""

    def __init__(self, *, check_targets=None, bwd_chunk_tokens: int = DEFAULT_BWD_CHUNK_TOKENS) -> None:
        self._native = NativeLinearLogpOp()
        self.check_targets = target_check_mode(check_targets)
        self.bwd_chunk_tokens = bwd_chunk_tokens

    def __call__(self, hidden, lm_head_weight, target_ids, bias=None, **kw):
        return self.apply(hidden, lm_head_weight, target_ids, bias, **kw)

    @staticmethod
    def _fusable(hidden: torch.Tensor, weight: torch.Tensor) -> bool:
        return (
            hidden.is_cuda and hidden.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16
            and hidden.shape[-1] % 8 == 0 and hidden.numel() > 0
        )

    def _validate_targets(self, target_ids: torch.Tensor, vocab: int) -> None:
        if self.check_targets == "sync" and target_ids.numel():
            lo, hi = torch.aminmax(target_ids)
            lo, hi = int(lo), int(hi)  # one host sync, like the reference (ops/cuda/loss/linear_logp.py:353-358)
            if lo < 0 or hi >= vocab:
                raise ValueError(
                    f"target_ids out of range: expected [0, {vocab - 1}], got [{lo}, {hi}]. "
                    "Mask or filter padding / ignore-index values (e.g. -100) before this op."
                )

    def apply(
        self, hidden, lm_head_weight, target_ids, bias=None, *, tp_group: Any = None, vocab_start_index: int = 0,
        global_vocab_size: Optional[int] = None,
    ) -> torch.Tensor:
        check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
        if should_use_tensor_parallel_linear_logp(
            tp_group, int(vocab_start_index), global_vocab_size, lm_head_weight.shape[0]
        ):
            if self._fusable(hidden, lm_head_weight):
                from rl_engine.parallel.tp_linear_logp import tensor_parallel_linear_logp_fused

                return tensor_parallel_linear_logp_fused(
                    hidden, lm_head_weight, target_ids, bias, tp_group=tp_group,
                    vocab_start_index=int(vocab_start_index), global_vocab_size=global_vocab_size,
                    check_targets=self.check_targets, chunk_tokens=self.bwd_chunk_tokens,
                )
            return self._native.apply(
                hidden, lm_head_weight, target_ids, bias, tp_group=tp_group, vocab_start_index=vocab_start_index,
                global_vocab_size=global_vocab_size,
            )
        if not self._fusable(hidden, lm_head_weight):
            return self._native.apply(hidden, lm_head_weight, target_ids, bias)
        self._validate_targets(target_ids, lm_head_weight.shape[0])
        logp, _ = _LinearLogp.apply(hidden, lm_head_weight, bias, target_ids, False, self.bwd_chunk_tokens,
                                    self._device_check(lm_head_weight.shape[0]))
        return logp

    def _device_check(self, vocab: int) -> int:
        return int(vocab) if self.check_targets == "device" else 0

    def with_entropy(self, hidden, lm_head_weight, target_ids, bias=None) -> Tuple[torch.Tensor, torch.Tensor]:
        check_linear_logp_args(hidden, lm_head_weight, target_ids, bias)
        if not self._fusable(hidden, lm_head_weight):
            return self._native.with_entropy(hidden, lm_head_weight, target_ids, bias)
        self._validate_targets(target_ids, lm_head_weight.shape[0])
        return _LinearLogp.apply(hidden, lm_head_weight, bias, target_ids, True, self.bwd_chunk_tokens,
                                 self._device_check(lm_head_weight.shape[0]))
