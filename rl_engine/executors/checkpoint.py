"""Trainer checkpoint: save and resume weights, optimizer state, weight version and sampler stream.

The reference has no checkpoint writer or resume path (its ``CheckpointFormat`` enum is unused and the
weight-update manifest is its only serialised model-state format: ``rl_engine/executors/bridge.py:
1359-1405``).  This module keeps that manifest as the checkpoint's description of the weights -- the
packed 256-byte-aligned blob + JSON manifest written by the ``file`` transport -- and adds what a
resume needs beside it: AdamW moments / master weights, the step count, the last published weight
version and the sampler's (seed, offset).
"""

from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch

from rl_engine.executors.bridge import FileBlobBridge


def _optimizer_file(directory: str, rank: int, world: int) -> str:
    """One file per rank when the optimizer state is sharded (``optimizer.rank3of8.pt``), else ``optimizer.pt``."""
    return os.path.join(directory, "optimizer.pt" if world <= 1 else f"optimizer.rank{rank}of{world}.pt")


def _plain(value: Any) -> Any:
    """Optimizer state as tensors (on the CPU), numbers, strings, ``None`` and lists / dicts of those: what
    ``torch.load(..., weights_only=True)`` accepts, so that loading a checkpoint never unpickles code."""
    if torch.is_tensor(value):
        return value.detach().cpu()
    if isinstance(value, dict):
        return {str(k): _plain(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [_plain(v) for v in value]
    if value is None or isinstance(value, (bool, int, float, str)):
        return value
    raise TypeError(f"optimizer state holds a {type(value).__name__}, which a checkpoint cannot carry")


class OptimizerShardReader:
    """The flat optimizer vectors of a checkpoint, whatever number of ranks wrote it.

    A job that lost a rank (or gained GPUs) resumes with another world size: the new ranks' slices of the flat
    parameter vector are cut differently from the saved ones.  The reader maps every saved shard into the flat index
    space (a shard of ``ShardedFusedAdamW`` carries its ``slices``; the state of ``FlatAdamW`` is one slice
    ``[0, n)``) and hands out any range ``[lo, hi)`` of a vector by gathering from the shards that overlap it, so no
    rank ever assembles a whole vector.  Shards are memory-mapped when the files allow it."""

    def __init__(self, shards) -> None:
        self._pieces = []                      # (lo, hi, offset into the shard's vectors, shard)
        steps = set()
        for shard in shards:
            steps.add(int(shard["steps"]))
            slices = shard.get("slices")
            if slices is None:
                slices = [[0, int(shard["m"].numel())]]
            off = 0
            for lo, hi in slices:
                lo, hi = int(lo), int(hi)
                if hi > lo:
                    self._pieces.append((lo, hi, off, shard))
                off += hi - lo
        if len(steps) != 1:
            raise ValueError(f"optimizer shards disagree on the step count: {sorted(steps)}")
        self.steps = steps.pop()
        self._pieces.sort(key=lambda piece: piece[0])
        for (_, hi_a, _, _), (lo_b, _, _, _) in zip(self._pieces, self._pieces[1:]):
            if lo_b < hi_a:
                raise ValueError("optimizer shards overlap: not the shards of one checkpoint")
        self.numel = self._pieces[-1][1] if self._pieces else 0

    @classmethod
    def from_directory(cls, directory: str, saved_world: int) -> "OptimizerShardReader":
        shards = []
        for r in range(max(1, int(saved_world))):
            path = _optimizer_file(directory, r, saved_world)
            if not os.path.exists(path):
                raise FileNotFoundError(f"checkpoint has no optimizer state for rank {r} of {saved_world}: {path}")
            try:
                shards.append(torch.load(path, map_location="cpu", weights_only=True, mmap=True))
            except (RuntimeError, ValueError):         # a file that cannot be mapped is read the plain way
                shards.append(torch.load(path, map_location="cpu", weights_only=True))
        return cls(shards)

    def has(self, name: str) -> bool:
        """Whether every shard holds vector ``name`` (``"m"``, ``"v"``, ``"master"``, ``"master_residual"``)."""
        return bool(self._pieces) and all(shard.get(name) is not None for _, _, _, shard in self._pieces)

    def read(self, name: str, lo: int, hi: int) -> torch.Tensor:
        """Elements ``[lo, hi)`` of vector ``name`` on the CPU, zeros where no shard covers (padding past the end)."""
        dtype = next((shard[name].dtype for _, _, _, shard in self._pieces if shard.get(name) is not None), torch.float32)
        out = torch.zeros(max(0, hi - lo), dtype=dtype)
        for p_lo, p_hi, off, shard in self._pieces:
            a, b = max(lo, p_lo), min(hi, p_hi)
            if b > a:
                out[a - lo : b - lo] = shard[name][off + a - p_lo : off + b - p_lo]
        return out


def save_checkpoint(directory: str, model: Any, optimizer: Any = None, *, weight_version: int = 0,
                    sampler: Any = None, extra: Optional[Dict[str, Any]] = None, rank: int = 0,
                    world: int = 1) -> Optional[str]:
    """Write ``weights.{blob,json}``, the optimizer state and ``state.json`` under ``directory``.

    With data-parallel ranks (``world`` > 1) every rank calls this with its ``rank``: rank 0 writes the weights and
    ``state.json`` (all ranks hold the same weights), every rank writes its own optimizer shard.  Returns the update
    id on the rank that wrote the weights, ``None`` elsewhere."""
    os.makedirs(directory, exist_ok=True)
    if optimizer is not None:
        torch.save(_plain(optimizer.state_dict()), _optimizer_file(directory, rank, world))
    if rank != 0:
        return None
    bridge = FileBlobBridge(directory, source_worker="checkpoint")
    bridge._latest_published_weight_version = int(weight_version) - 1
    source = model.state_dict_views() if hasattr(model, "state_dict_views") else model
    manifest = bridge.publish(source, weight_version=int(weight_version), metadata={"checkpoint": True})
    state = {
        "update_id": manifest.update_id,
        "weight_version": int(weight_version),
        "world": int(world),
        "sampler": None if sampler is None else {"seed": int(sampler.seed), "offset": int(sampler._offset)},
        "extra": dict(extra or {}),
    }
    with open(os.path.join(directory, "state.json"), "w") as f:
        json.dump(state, f)
    return manifest.update_id


@torch.no_grad()
def load_checkpoint(directory: str, model: Any, optimizer: Any = None, *, sampler: Any = None, rank: int = 0,
                    world: int = 1) -> Dict[str, Any]:
    """Restores weights (validated against the manifest), then the optimizer state of this ``rank`` (the optimizer's
    ``load_state_dict`` runs after the weights are in place, so it can re-derive master weights from them), then the
    sampler's stream position.  Returns ``state.json``.

    ``world`` may differ from the number of ranks that saved (a job that resumes after losing a rank, or on more
    GPUs): the weights are replicated, and an optimizer with ``accepts_resharded_state`` (``FlatAdamW``,
    ``ShardedFusedAdamW``) gets an ``OptimizerShardReader`` over all saved shards and picks its new slices."""
    with open(os.path.join(directory, "state.json")) as f:
        state = json.load(f)
    saved_world = int(state.get("world", 1))
    resharded = saved_world != int(world)
    if resharded and optimizer is not None and not getattr(optimizer, "accepts_resharded_state", False):
        raise ValueError(f"checkpoint was written by {saved_world} rank(s), resuming with {world}: "
                         f"{type(optimizer).__name__} cannot take a re-cut optimizer state")
    bridge = FileBlobBridge(directory, source_worker="checkpoint")
    manifest = bridge.load_manifest(state["update_id"])
    tensors = bridge.import_update(manifest)
    targets = model.named_views() if hasattr(model, "named_views") else dict(model.state_dict())
    missing = sorted(set(targets) - set(tensors))
    if missing:
        raise KeyError(f"checkpoint lacks tensors for: {missing[:5]}")
    for name, dst in targets.items():
        dst.copy_(tensors[name].to(device=dst.device, dtype=dst.dtype))
    bridge.acknowledge(manifest.update_id)
    opt_path = _optimizer_file(directory, rank, world)
    if optimizer is not None and resharded:
        # another world size than the one that saved: every rank reads its new slices out of all the saved shards
        optimizer.load_state_dict(OptimizerShardReader.from_directory(directory, saved_world))
    elif optimizer is not None:
        if not os.path.exists(opt_path):
            raise FileNotFoundError(f"checkpoint has no optimizer state for rank {rank} of {world}: {opt_path}")
        optimizer.load_state_dict(torch.load(opt_path, map_location="cpu", weights_only=True))
    if sampler is not None and state.get("sampler"):
        sampler.seed, sampler._offset = state["sampler"]["seed"], state["sampler"]["offset"]
    return state
