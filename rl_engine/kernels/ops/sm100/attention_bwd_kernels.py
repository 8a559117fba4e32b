"""Host-side work lists for the fused attention backward kernels.

The dQ kernel reuses the forward's query-tile table.  The dK/dV kernel needs, for every 128-key
tile of every distinct key range, the list of 64-query blocks that can see it; long lists (a shared
prompt is seen by every completion) are split into items whose partial sums are reduced in slot
order, which keeps the result bitwise reproducible.  Lists depend only on the packed layout and are
cached with it.
"""

from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext

KEY_TILE = 128
Q_BLOCK = 64
MAX_BLOCKS_PER_ITEM = 64

_PLAN_CACHE: Dict[int, tuple] = {}


def build_plan(layout) -> tuple:
    hit = _PLAN_CACHE.get(id(layout))
    if hit is not None and hit[0] is layout:
        return hit[1]
    # key range -> [(q_start, q_len, causal)]
    ranges: Dict[Tuple[int, int], List[Tuple[int, int, int]]] = {}
    for (q_start, q_len, pk_start, pk_len, sk_start, sk_len) in layout.host_seqs:
        if pk_len:
            ranges.setdefault((pk_start, pk_len), []).append((q_start, q_len, 0))
        if sk_len:
            ranges.setdefault((sk_start, sk_len), []).append((q_start, q_len, 1 if layout.causal else 0))
    q_blocks: List[List[int]] = []
    items: List[List[int]] = []
    jobs: List[List[int]] = []
    slots = 0
    for (k_start, k_len), readers in sorted(ranges.items()):
        for k_pos in range(0, k_len, KEY_TILE):
            begin = len(q_blocks)
            for (q_start, q_len, causal) in readers:
                for q_pos in range(0, q_len, Q_BLOCK):
                    n_rows = min(Q_BLOCK, q_len - q_pos)
                    if causal and q_pos + n_rows - 1 < k_pos:
                        continue  # every query of the block precedes the tile's first key
                    q_blocks.append([q_start + q_pos, n_rows, q_pos, causal])
            end = len(q_blocks)
            if end == begin:
                continue
            tile_len = min(KEY_TILE, k_len - k_pos)
            pieces = [(b, min(b + MAX_BLOCKS_PER_ITEM, end)) for b in range(begin, end, MAX_BLOCKS_PER_ITEM)]
            if len(pieces) == 1:
                items.append([k_start + k_pos, tile_len, k_pos, begin, end, -1, 0, 0])
            else:
                jobs.append([k_start + k_pos, tile_len, slots, slots + len(pieces)])
                for (b, e) in pieces:
                    items.append([k_start + k_pos, tile_len, k_pos, b, e, slots, 0, 0])
                    slots += 1
    items.sort(key=lambda it: it[3] - it[4])  # longest lists first
    dev = layout.seqs.device
    as_t = lambda rows, w: torch.tensor(rows, dtype=torch.int32, device=dev).reshape(-1, w)
    plan = (as_t(items, 8), as_t(q_blocks, 4), as_t(jobs, 4), slots)
    if len(_PLAN_CACHE) > 64:
        _PLAN_CACHE.clear()
    _PLAN_CACHE[id(layout)] = (layout, plan)
    return plan


def _aligned(t: torch.Tensor) -> torch.Tensor:
    ok = t.stride(2) == 1 and t.stride(1) == 128 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0
    return t if ok else t.contiguous()


def fused_backward(q, k, v, out, lse, dout, layout, scale: float):
    items, q_blocks, jobs, slots = build_plan(layout)
    dout = _aligned(dout)
    out = _aligned(out)
    if out.stride(0) != dout.stride(0):
        out, dout = out.contiguous(), dout.contiguous()
    dq, dk, dv = require_ext().attention_bwd(
        _aligned(q), _aligned(k), _aligned(v), out, dout, lse, layout.seqs, layout.tiles, items, q_blocks, jobs, slots,
        layout.causal, float(scale),
    )
    return dq, dk, dv
