"""DeepSpeed-backed training worker (optional).

Parity: ``rl_engine/executors/deepspeed_trainer.py:41-693`` of the reference:
``DeepSpeedTrainingConfig`` (ZeRO stage, config deep-merged over defaults), ``deepspeed.initialize``
with an AdamW optimizer, ``engine.backward`` / ``engine.step``, ZeRO-3 ``GatheredParameters`` around
the LM head for the fused log-prob, ZeRO-3 publication from rank 0 through a gathered clone of the full
state (``:204-286,644-675``), ``CUDA_HOME`` discovery for CUDA toolkits that came as Python wheels
(``:332-391``), ``DeepSpeedUnavailableError`` when the package is missing.  The objective is the one
function shared with ``NativeTrainingWorker`` (``clipped_ratio_objective``); DeepSpeed is looked up in
``sys.modules`` / imported lazily so tests can install a fake module.  This build's own data-parallel
path does not need DeepSpeed (see ``rl_engine.parallel.data_parallel``).
"""

from __future__ import annotations

import contextlib
import importlib
import os
import sysconfig
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Mapping, Optional

import torch

from rl_engine.executors.bridge import WeightBridgeUnavailableError
from rl_engine.executors.hidden_states import extract_hidden_states
from rl_engine.executors.trainer import (
    NativeTrainingConfig, NativeTrainingWorker, advantage_metrics, clipped_ratio_objective, safe_token_ids,
    validate_model_input_token_ids,
)
from rl_engine.executors.training_contract import RolloutStageResult, TrainingStageResult


class DeepSpeedUnavailableError(RuntimeError):
    """DeepSpeed is not installed and no module was injected."""


def _deep_merge(base: Mapping[str, Any], override: Mapping[str, Any]) -> Dict[str, Any]:
    out = dict(base)
    for key, value in override.items():
        if isinstance(value, Mapping) and isinstance(out.get(key), Mapping):
            out[key] = _deep_merge(out[key], value)
        else:
            out[key] = value
    return out


@dataclass(frozen=True)
class DeepSpeedTrainingConfig(NativeTrainingConfig):
    zero_stage: int = 0
    train_micro_batch_size_per_gpu: int = 1
    deepspeed_config: Mapping[str, Any] = field(default_factory=dict)
    initialize_kwargs: Mapping[str, Any] = field(default_factory=dict)     # extra keywords for ``deepspeed.initialize``

    def resolved_deepspeed_config(self) -> Dict[str, Any]:
        defaults = {
            "train_micro_batch_size_per_gpu": self.train_micro_batch_size_per_gpu,
            "gradient_accumulation_steps": 1,
            "zero_optimization": {"stage": self.zero_stage},
            "bf16": {"enabled": self.dtype == torch.bfloat16},
            "fp16": {"enabled": self.dtype == torch.float16},
        }
        return _deep_merge(defaults, self.deepspeed_config)


def cuda_home_candidates() -> List[Path]:
    """Places a CUDA toolkit may live when it was installed as Python wheels (``site-packages/nvidia/cu*``, newest
    first), followed by the toolkit torch's extension builder already knows."""
    roots = {Path(p) for key in ("purelib", "platlib") if (p := sysconfig.get_paths().get(key))}
    found: List[Path] = []
    for root in sorted(roots):
        if (root / "nvidia").is_dir():
            found += sorted((root / "nvidia").glob("cu*"), reverse=True)
    try:
        from torch.utils.cpp_extension import CUDA_HOME
    except Exception:  # noqa: BLE001 - torch without the extension builder
        CUDA_HOME = None
    if CUDA_HOME:
        found.append(Path(str(CUDA_HOME)))
    return found


def configure_cuda_home(environ: Optional[Dict[str, str]] = None) -> Optional[str]:
    """DeepSpeed compiles its ops at import and needs ``CUDA_HOME`` to hold ``bin/nvcc`` and ``include/cuda.h``.  An
    explicit ``CUDA_HOME`` wins (torch's extension builder is pointed at it); otherwise the first candidate that
    looks like a toolkit is exported, with its ``bin`` on ``PATH`` and ``lib64`` / ``lib`` on ``LD_LIBRARY_PATH``.
    Returns the toolkit root that is in effect, or ``None``."""
    env = os.environ if environ is None else environ

    def tell_torch(path: str) -> None:
        try:
            import torch.utils.cpp_extension as ext

            ext.CUDA_HOME = path
        except Exception:  # noqa: BLE001
            pass

    def prepend(key: str, value: str) -> None:
        parts = [p for p in env.get(key, "").split(os.pathsep) if p]
        if value not in parts:
            env[key] = os.pathsep.join([value] + parts)

    if env.get("CUDA_HOME"):
        tell_torch(env["CUDA_HOME"])
        return env["CUDA_HOME"]
    for root in cuda_home_candidates():
        if (root / "bin" / "nvcc").is_file() and (root / "include" / "cuda.h").is_file():
            env["CUDA_HOME"] = str(root)
            tell_torch(str(root))
            prepend("PATH", str(root / "bin"))
            for lib in ("lib64", "lib"):
                if (root / lib).is_dir():
                    prepend("LD_LIBRARY_PATH", str(root / lib))
            return str(root)
    return None


def _load_deepspeed(module: Any = None) -> Any:
    if module is not None:
        return module
    configure_cuda_home()
    try:
        return importlib.import_module("deepspeed")
    except ImportError as exc:
        raise DeepSpeedUnavailableError(
            "DeepSpeed is not installed; use NativeTrainingWorker / GRPOTrainingWorker or install deepspeed."
        ) from exc
    except Exception as exc:  # noqa: BLE001 - installed, but its import-time op build failed
        raise DeepSpeedUnavailableError(
            "DeepSpeed is installed but failed to import here. If CUDA came as Python wheels, point CUDA_HOME at the "
            "toolkit root that holds bin/nvcc and include/cuda.h."
        ) from exc


class FullStateSnapshot(torch.nn.Module):
    """A detached full copy of a state dict, presented as a module so that a weight bridge can publish it."""

    def __init__(self, state: Mapping[str, torch.Tensor]) -> None:
        super().__init__()
        self._state = {name: t.detach().clone() for name, t in state.items()}

    def state_dict(self, *args: Any, **kwargs: Any) -> Dict[str, torch.Tensor]:  # noqa: D401 - nn.Module signature
        return dict(self._state)


class DeepSpeedTrainingWorker(NativeTrainingWorker):
    def __init__(self, config: Optional[DeepSpeedTrainingConfig] = None, *, model=None, weight_bridge=None,
                 weight_transport: Optional[str] = None, deepspeed_module: Any = None) -> None:
        """``weight_transport``: name for ``make_weight_bridge`` when no ``weight_bridge`` is given (default: the
        configuration's)."""
        config = config or DeepSpeedTrainingConfig()
        if weight_bridge is None and weight_transport is not None:
            from rl_engine.executors.bridge import make_weight_bridge

            weight_bridge = make_weight_bridge(weight_transport, source_worker="deepspeed-training")
        super().__init__(config, model=model, weight_bridge=weight_bridge, source_worker="deepspeed-training")
        self._deepspeed = _load_deepspeed(deepspeed_module)
        ds_config = self.config.resolved_deepspeed_config()
        self._zero_stage = int(ds_config.get("zero_optimization", {}).get("stage", 0))
        self.engine, self.optimizer, _, _ = self._deepspeed.initialize(
            model=self.model, optimizer=self.optimizer, config=ds_config, **dict(self.config.initialize_kwargs)
        )

    def _gathered(self):
        if self._zero_stage < 3:
            return contextlib.nullcontext()
        gather = getattr(getattr(self._deepspeed, "zero", None), "GatheredParameters", None)
        if not callable(gather):
            raise WeightBridgeUnavailableError(
                "DeepSpeed ZeRO-3 linear_logp training requires deepspeed.zero.GatheredParameters "
                "or an equivalent full-parameter gather API."
            )
        head = self.model.lm_head
        params = [head.weight] + ([head.bias] if getattr(head, "bias", None) is not None else [])
        return gather(params, modifier_rank=None)

    def _current_logps(self, batch) -> torch.Tensor:
        """The forward pass goes through the ENGINE (``engine(token_ids)``), not the bare module: DeepSpeed's
        ``backward`` / ``step`` book-keeping and the ZeRO-3 parameter hooks hang on the engine's forward
        (reference: ``rl_engine/executors/deepspeed_trainer.py:146-151,618-641``)."""
        head = self.model.lm_head
        hidden = extract_hidden_states(self.engine(batch.token_ids.long()), hidden_dim=head.weight.shape[1])
        targets = safe_token_ids(batch.token_ids.to(hidden.device), batch.completion_mask)
        logps = self._linear_logp(hidden, head.weight, targets, getattr(head, "bias", None))
        keep = batch.completion_mask.to(device=logps.device, dtype=torch.bool)
        return torch.where(keep, logps, torch.zeros_like(logps)).float()

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        t0 = time.perf_counter()
        cfg = self.config
        batch, payload_metrics = self._batch_from_rollout_or_synthetic(rollout)
        validate_model_input_token_ids(batch.token_ids, vocab_size=self.model.lm_head.weight.shape[0])
        zero = getattr(self.engine, "zero_grad", None)
        if callable(zero):
            zero()
        with self._gathered():
            loss = clipped_ratio_objective(self._current_logps(batch), batch, cfg)
            self.engine.backward(loss)
        self.engine.step()
        return TrainingStageResult(
            iteration=rollout.iteration, consumed_weight_version=rollout.weight_version,
            published_weight_version=self._next_published_weight_version(rollout.weight_version),
            metrics={
                "loss": float(loss.detach()), "active_tokens": int(batch.completion_mask.sum()),
                "payload_type": type(rollout.payload).__name__, "training_backend": "deepspeed",
                "training_device": str(self.device), "deepspeed_engine": type(self.engine).__name__,
                "deepspeed_zero_stage": self._zero_stage, "current_logp_path": "linear_logp",
                "current_logp_backend": type(self._linear_logp).__name__,
                **advantage_metrics(batch),
                **payload_metrics,
            },
            started_at=t0, finished_at=time.perf_counter(),
        )

    def _engine_attr(self, names, default: int) -> int:
        for name in names:
            value = getattr(self.engine, name, None)
            if value is not None:
                return int(value)
        return default

    def publish_weights(self, weight_version=None, metadata=None):
        """Publishes the COMPLETE model state.  Under ZeRO-3 every rank holds a slice of each parameter, so rank 0
        clones the full state inside DeepSpeed's gather context and publishes that clone; a runtime that cannot
        gather fails loudly rather than publishing a shard, and so does any rank but 0."""
        rank = self._engine_attr(("global_rank", "rank", "local_rank"), 0)
        world = self._engine_attr(("world_size", "dp_world_size"), 1)
        meta = dict(metadata or {})
        layout = {"kind": "full-state", "zero_stage": self._zero_stage, "world_size": world, "rank": rank}
        layout.update(dict(meta.get("layout", {})))
        meta["layout"] = layout
        if self._zero_stage < 3:
            return super().publish_weights(weight_version, meta)
        if rank != 0:
            raise WeightBridgeUnavailableError("DeepSpeed ZeRO-3 full-state publish is only supported from rank 0")
        module = getattr(self.engine, "module", None)
        module = module if isinstance(module, torch.nn.Module) else self.model
        gather = getattr(getattr(self._deepspeed, "zero", None), "GatheredParameters", None)
        if callable(gather):
            with gather(list(module.parameters()), modifier_rank=0):
                snapshot = FullStateSnapshot(module.state_dict())
            how = "deepspeed.zero.GatheredParameters"
        elif world == 1:
            snapshot = FullStateSnapshot(module.state_dict())
            how = "single-rank-state-dict"
        else:
            raise WeightBridgeUnavailableError(
                "DeepSpeed ZeRO-3 publish requires deepspeed.zero.GatheredParameters or an equivalent full-state export"
            )
        state = snapshot.state_dict()
        if not state:
            raise WeightBridgeUnavailableError("DeepSpeed ZeRO-3 full-state export produced no tensors")
        meta["deepspeed_zero3_full_state_export"] = {"method": how, "rank": rank, "world_size": world,
                                                     "tensor_count": len(state)}
        live, self.model = self.model, snapshot
        try:
            return super().publish_weights(weight_version, meta)
        finally:
            self.model = live
