"""DeepSpeed-backed training worker (optional).

Parity: ``rl_engine/executors/deepspeed_trainer.py:41-693`` of the reference:
``DeepSpeedTrainingConfig`` (ZeRO stage, config deep-merged over defaults), ``deepspeed.initialize``
with an AdamW optimizer, ``engine.backward`` / ``engine.step``, ZeRO-3 ``GatheredParameters`` around
the LM head for the fused log-prob, rank-0 gathered publish, ``DeepSpeedUnavailableError`` when the
package is missing.  The step math is inherited from ``NativeTrainingWorker``; DeepSpeed is looked up
in ``sys.modules`` / imported lazily so tests can install a fake module.  This build's own
data-parallel path does not need DeepSpeed (see ``rl_engine.parallel.data_parallel``).
"""

from __future__ import annotations

import contextlib
import importlib
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional

import torch

from rl_engine.executors.bridge import WeightBridgeUnavailableError
from rl_engine.executors.trainer import NativeTrainingConfig, NativeTrainingWorker, validate_model_input_token_ids
from rl_engine.executors.training_contract import RolloutStageResult, TrainingStageResult, objective_reference_logps
from rl_engine.testing import compute_policy_ratio, compute_reference_kl, masked_mean


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

    def resolved_deepspeed_config(self) -> Dict[str, Any]:
        defaults = {
            "train_micro_batch_size_per_gpu": self.train_micro_batch_size_per_gpu,
            "gradient_accumulation_steps": 1,
            "zero_optimization": {"stage": self.zero_stage},
            "bf16": {"enabled": self.dtype == torch.bfloat16},
            "fp16": {"enabled": self.dtype == torch.float16},
        }
        return _deep_merge(defaults, self.deepspeed_config)


def _load_deepspeed(module: Any = None) -> Any:
    if module is not None:
        return module
    try:
        return importlib.import_module("deepspeed")
    except ImportError as exc:
        raise DeepSpeedUnavailableError(
            "DeepSpeed is not installed; use NativeTrainingWorker or install deepspeed."
        ) from exc


class DeepSpeedTrainingWorker(NativeTrainingWorker):
    def __init__(self, config: Optional[DeepSpeedTrainingConfig] = None, *, model=None, weight_bridge=None,
                 deepspeed_module: Any = None) -> None:
        super().__init__(config or DeepSpeedTrainingConfig(), model=model, weight_bridge=weight_bridge,
                         source_worker="deepspeed-training")
        self._deepspeed = _load_deepspeed(deepspeed_module)
        ds_config = self.config.resolved_deepspeed_config()
        self._zero_stage = int(ds_config.get("zero_optimization", {}).get("stage", 0))
        self.engine, self.optimizer, _, _ = self._deepspeed.initialize(
            model=self.model, optimizer=self.optimizer, config=ds_config
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

    def train(self, rollout: RolloutStageResult) -> TrainingStageResult:
        t0 = time.perf_counter()
        cfg = self.config
        batch, payload_metrics = self._batch_from_rollout_or_synthetic(rollout)
        validate_model_input_token_ids(batch.token_ids, vocab_size=self.model.lm_head.weight.shape[0])
        zero = getattr(self.engine, "zero_grad", None)
        if callable(zero):
            zero()
        with self._gathered():
            cur = self._current_logps(batch)
            old = cur.detach() - cfg.old_logp_offset
            ref = objective_reference_logps(cur, batch)
            adv = batch.advantages.float()
            ratio = compute_policy_ratio(cur, old, batch.completion_mask)
            policy = -torch.minimum(ratio * adv, torch.clamp(ratio, cfg.clip_low, cfg.clip_high) * adv)
            kl = compute_reference_kl(cur, ref, batch.completion_mask)
            loss = masked_mean(policy + cfg.kl_beta * kl, batch.completion_mask)
            self.engine.backward(loss)
        self.engine.step()
        active = adv[batch.completion_mask]
        return TrainingStageResult(
            iteration=rollout.iteration, consumed_weight_version=rollout.weight_version,
            published_weight_version=self._next_published_weight_version(rollout.weight_version),
            metrics={
                "loss": float(loss.detach()), "active_tokens": int(batch.completion_mask.sum()),
                "payload_type": type(rollout.payload).__name__, "training_backend": "deepspeed",
                "training_device": str(self.device), "deepspeed_engine": type(self.engine).__name__,
                "deepspeed_zero_stage": self._zero_stage, "current_logp_path": "linear_logp",
                "current_logp_backend": type(self._linear_logp).__name__,
                "active_advantage_mean_global": float(active.mean()) if active.numel() else 0.0,
                "active_advantage_std_global": float(active.std(unbiased=False)) if active.numel() else 0.0,
                **payload_metrics,
            },
            started_at=t0, finished_at=time.perf_counter(),
        )

    def publish_weights(self, weight_version=None, metadata=None):
        meta = dict(metadata or {})
        layout = dict(meta.get("layout", {}))
        layout.setdefault("zero_stage", self._zero_stage)
        meta["layout"] = layout
        if self._zero_stage >= 3:
            gather = getattr(getattr(self._deepspeed, "zero", None), "GatheredParameters", None)
            if not callable(gather):
                raise WeightBridgeUnavailableError("ZeRO-3 publish needs deepspeed.zero.GatheredParameters")
            with gather(list(self.model.parameters()), modifier_rank=None):
                return super().publish_weights(weight_version, meta)
        return super().publish_weights(weight_version, meta)
