"""Host-side work lists for the fused attention backward kernels.

The dQ kernel reuses the forward's query-tile table.  The dK/dV kernel needs, for every 128-key
tile of the key axis, the list of 64-query blocks that can see it; long lists (a shared
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
    # readers: (k_start, k_len, q_start, q_len, causal).  Key ranges of different sequences may be equal
    # (a prompt shared by a group), disjoint, or overlap partly (context-parallel shards whose "prefix"
    # covers another shard's "self" keys), so the key axis is cut at every range boundary and each
    # elementary interval is tiled on its own: one key tile is then written by exactly one job.
    readers: List[Tuple[int, int, int, int, int]] = []
    for (q_start, q_len, pk_start, pk_len, sk_start, sk_len) in layout.host_seqs:
        if pk_len:
            readers.append((pk_start, pk_len, q_start, q_len, 0))
        if sk_len:
            readers.append((sk_start, sk_len, q_start, q_len, 1 if layout.causal else 0))
    cuts = sorted({r[0] for r in readers} | {r[0] + r[1] for r in readers})
    q_blocks: List[List[int]] = []
    items: List[List[int]] = []
    jobs: List[List[int]] = []
    slots = 0
    for lo, hi in zip(cuts[:-1], cuts[1:]):
        covering = [r for r in readers if r[0] <= lo and hi <= r[0] + r[1]]
        if not covering:
            continue
        for k_abs in range(lo, hi, KEY_TILE):
            begin = len(q_blocks)
            for (k_start, _k_len, q_start, q_len, causal) in covering:
                k_pos = k_abs - k_start  # index of the tile's first key inside this reader's range
                for q_pos in range(0, q_len, Q_BLOCK):
                    n_rows = min(Q_BLOCK, q_len - q_pos)
                    if causal and q_pos + n_rows - 1 < k_pos:
                        continue  # every query of the block precedes the tile's first key
                    # the kernel's causal test only uses (item k_pos - block q_pos): fold k_pos in here
                    q_blocks.append([q_start + q_pos, n_rows, q_pos - k_pos, causal])
            end = len(q_blocks)
            if end == begin:
                continue
            tile_len = min(KEY_TILE, hi - k_abs)
            pieces = [(b, min(b + MAX_BLOCKS_PER_ITEM, end)) for b in range(begin, end, MAX_BLOCKS_PER_ITEM)]
            if len(pieces) == 1:
                items.append([k_abs, tile_len, 0, begin, end, -1, 0, 0])
            else:
                jobs.append([k_abs, tile_len, slots, slots + len(pieces)])
                for (b, e) in pieces:
                    items.append([k_abs, tile_len, 0, b, e, slots, 0, 0])
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
