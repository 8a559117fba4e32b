"""Sequence-parallel tensor-parallel linears with the collective fused into the GEMM kernel.

Activations between the two linears of a block are sharded by rows (tokens) over the ``W`` ranks:

    column_parallel(x_local [M/W, K], w_local [N/W, K]) -> y [M, N/W]      all-gather  -> GEMM
    row_parallel(x [M, K/W],      w_local [N, K/W])     -> y_local [M/W, N]  GEMM -> reduce-scatter

Forward and the activation gradients run on the two fused kernels of ``csrc/kernels/tp_linear.cu``:
``tp_ag_gemm`` (copy warps push this rank's rows to every peer while the tensor cores already work on the
tiles that have landed) and ``tp_gemm_rs`` (the epilogue stores partial tiles into the owner's slab over
NVLink; the owner sums the ``W`` partials in rank order).  The backward of one is the other:

    column_parallel:  dx_local = reduce_scatter(dy @ w_local)        -> tp_gemm_rs (B as [K, N] operand)
    row_parallel:     dx       = all_gather(dy_local) @ w_local      -> tp_ag_gemm

Weight gradients contract over the gathered token axis on the plain tcgen05 GEMM; ``row_parallel`` reuses
the rows that ``tp_ag_gemm`` has just gathered, ``column_parallel`` gathers ``x`` again with a peer-store
copy (cheaper than keeping ``M x K`` alive per layer).

Buffers live in symmetric memory, one set per problem shape, double-buffered by call parity; arrival
counters are monotonic, so no reset pass or extra barrier is needed between calls.  All summation orders
are fixed: results are run-to-run reproducible.

The reference has no tensor-parallel linear layers (its TP support is the vocab-parallel log-prob,
``rl_engine/kernels/ops/pytorch/loss/linear_logp.py:176-377``).
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext
from rl_engine.parallel.symmetric import SymmetricMemory

TILE_M = 128
TILE_N = 256


def pick_chunks(rows_local: int, k: int, sm_count: int = 148) -> int:
    """Column chunks per 128-row tile for the gather copy: enough (tile, chunk) units to occupy the copy
    warps of every CTA, each unit at least 64 sixteen-byte vectors wide."""
    tiles = max(rows_local // TILE_M, 1)
    want = min(32, max(1, -(-sm_count // tiles)))
    vec = k // 8
    chunks = 1
    while chunks * 2 <= want and vec % (chunks * 2) == 0 and vec // (chunks * 2) >= 64:
        chunks *= 2
    return chunks


class _BufferSet:
    """Two parities of (data buffer, counter array) in a symmetric heap of its own."""

    def __init__(self, group, device, data_shape: Tuple[int, ...], counters: int) -> None:
        numel = 1
        for d in data_shape:
            numel *= d
        nbytes = 2 * (numel * 2 + 256) + 2 * (counters * 4 + 256) + (1 << 16)
        self.mem = SymmetricMemory(nbytes, group=group, device=device)
        self.data = [self.mem.alloc(data_shape, torch.bfloat16) for _ in range(2)]
        self.counters = [self.mem.alloc((counters,), torch.int32) for _ in range(2)]
        for c in self.counters:
            c.local.zero_()
        self.mem.barrier()  # no arrival may precede the zeroing
        self.calls = 0

    def next(self):
        """(data SymmetricTensor, counter SymmetricTensor, 1-based use count of that parity)."""
        parity = self.calls & 1
        use = self.calls // 2 + 1
        self.calls += 1
        return self.data[parity], self.counters[parity], use


class TensorParallelLinears:
    def __init__(self, group=None, device: Optional[torch.device] = None, wait_ms: float = 2000.0) -> None:
        import torch.distributed as dist

        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.wait_ms = float(wait_ms)
        self._ag: Dict[Tuple[int, int], _BufferSet] = {}
        self._rs: Dict[Tuple[int, int], _BufferSet] = {}
        self._plain: Dict[Tuple[int, int], _BufferSet] = {}

    # -- fused kernels --------------------------------------------------------------------------------
    def ag_gemm(self, x_local: torch.Tensor, b: torch.Tensor, b_mn: bool = False):
        """``(allgather_rows(x_local) @ B^T  [M, N], gathered rows [M, K])``; ``b`` is ``[N, K]`` or, with ``b_mn``, ``[K, N]``."""
        rows, k = x_local.shape
        m = rows * self.world
        key = (m, k)
        if key not in self._ag:
            self._ag[key] = _BufferSet(self.group, self.device, (m, k), m // TILE_M)
        data, ready, use = self._ag[key].next()
        out = require_ext().tp_ag_gemm(x_local, b, bool(b_mn), self.rank, data.ptrs, ready.ptrs, use,
                                       pick_chunks(rows, k), self.wait_ms)
        return out, data.local

    def gemm_rs(self, a: torch.Tensor, b: torch.Tensor, b_mn: bool = False) -> torch.Tensor:
        """``reduce_scatter_rows(a @ B^T)  [M / W, N]``."""
        m = a.shape[0]
        n = b.shape[1] if b_mn else b.shape[0]
        key = (m, n)
        if key not in self._rs:
            tiles = (m // self.world // TILE_M) * (-(-n // TILE_N))
            self._rs[key] = _BufferSet(self.group, self.device, (self.world, m // self.world, n), tiles)
        data, counters, use = self._rs[key].next()
        return require_ext().tp_gemm_rs(a, b, bool(b_mn), self.rank, data.ptrs, counters.ptrs, use * self.world, self.wait_ms)

    def all_gather_rows(self, x_local: torch.Tensor) -> torch.Tensor:
        """Plain gather by peer stores (two device barriers); the result is valid until the next call with this shape."""
        rows, k = x_local.shape
        key = (rows * self.world, k)
        if key not in self._plain:
            self._plain[key] = _BufferSet(self.group, self.device, (rows * self.world, k), 1)
        bufs = self._plain[key]
        buf = bufs.data[0]
        bufs.mem.barrier()
        off = self.rank * rows * k * 2
        require_ext().cast_broadcast(x_local.contiguous(), [p + off for p in buf.ptrs], 1)
        bufs.mem.barrier()
        return buf.local

    def process_group(self):
        """The ``torch.distributed`` group of this instance (``None`` on a single rank), for ops that take ``tp_group``."""
        if self.world == 1:
            return None
        import torch.distributed as dist

        return self.group if self.group is not None else dist.group.WORLD

    def supports(self, rows_local: int, k: int, n: int) -> bool:
        return rows_local > 0 and rows_local % TILE_M == 0 and k % 8 == 0 and n % 8 == 0

    # -- differentiable layers ------------------------------------------------------------------------
    def column_parallel(self, x_local: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        return _ColumnParallel.apply(x_local, w_local, self)

    def row_parallel(self, x: torch.Tensor, w_local: torch.Tensor) -> torch.Tensor:
        return _RowParallel.apply(x, w_local, self)

    def check(self) -> None:
        from rl_engine.kernels.ops.base import check_device_errors

        check_device_errors(self.device.index or 0)


def _rows_ok(t: torch.Tensor) -> torch.Tensor:
    return t if (t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0) else t.contiguous()


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w_local, tp: TensorParallelLinears):
        x_local, w_local = _rows_ok(x_local), _rows_ok(w_local)
        out, _ = tp.ag_gemm(x_local, w_local)
        ctx.save_for_backward(x_local, w_local)
        ctx.tp = tp
        return out

    @staticmethod
    def backward(ctx, dy):
        from rl_engine.kernels.ops.sm100.gemm import gemm

        x_local, w_local = ctx.saved_tensors
        tp = ctx.tp
        dy = _rows_ok(dy)
        dx_local = tp.gemm_rs(dy, w_local, b_mn=True)          # [M, Nl] @ [Nl, K] -> rows scattered
        x_all = tp.all_gather_rows(x_local)
        dw = gemm(dy, x_all, a_mn=True, b_mn=True)             # dy^T @ x  [Nl, K]
        return dx_local, dw, None


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_local, tp: TensorParallelLinears):
        x, w_local = _rows_ok(x), _rows_ok(w_local)
        ctx.save_for_backward(x, w_local)
        ctx.tp = tp
        return tp.gemm_rs(x, w_local)

    @staticmethod
    def backward(ctx, dy_local):
        from rl_engine.kernels.ops.sm100.gemm import gemm

        x, w_local = ctx.saved_tensors
        tp = ctx.tp
        dx, dy_all = tp.ag_gemm(_rows_ok(dy_local), w_local, b_mn=True)   # gather(dy) [M, N] @ [N, Kl]
        dw = gemm(dy_all, x, a_mn=True, b_mn=True)                         # dy^T @ x  [N, Kl]
        return dx, dw, None
