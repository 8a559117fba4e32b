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


def save_checkpoint(directory: str, model: Any, optimizer: Any = None, *, weight_version: int = 0,
                    sampler: Any = None, extra: Optional[Dict[str, Any]] = None) -> str:
    """Write ``weights.{blob,json}``, ``optimizer.pt`` and ``state.json`` under ``directory``; returns the update id."""
    os.makedirs(directory, exist_ok=True)
    bridge = FileBlobBridge(directory, source_worker="checkpoint")
    bridge._latest_published_weight_version = int(weight_version) - 1
    source = model.state_dict_views() if hasattr(model, "state_dict_views") else model
    manifest = bridge.publish(source, weight_version=int(weight_version), metadata={"checkpoint": True})
    if optimizer is not None:
        torch.save(optimizer.state_dict(), os.path.join(directory, "optimizer.pt"))
    state = {
        "update_id": manifest.update_id,
        "weight_version": int(weight_version),
        "sampler": None if sampler is None else {"seed": int(sampler.seed), "offset": int(sampler._offset)},
        "extra": dict(extra or {}),
    }
    with open(os.path.join(directory, "state.json"), "w") as f:
        json.dump(state, f)
    return manifest.update_id


@torch.no_grad()
def load_checkpoint(directory: str, model: Any, optimizer: Any = None, *, sampler: Any = None) -> Dict[str, Any]:
    with open(os.path.join(directory, "state.json")) as f:
        state = json.load(f)
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
    opt_path = os.path.join(directory, "optimizer.pt")
    if optimizer is not None and os.path.exists(opt_path):
        optimizer.load_state_dict(torch.load(opt_path, map_location="cpu", weights_only=False))
    if sampler is not None and state.get("sampler"):
        sampler.seed, sampler._offset = state["sampler"]["seed"], state["sampler"]["offset"]
    return state
