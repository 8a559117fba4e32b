"""Stateless (no KV cache) reference / reward scoring over full sequences.

Parity: ``rl_engine/executors/stateless_executor.py:22-637`` of the reference — the config and
result dataclasses, ``StatelessForwardExecutor.score``, ``score_reference_logprobs`` (next-token
shift aligned to ``[B, S]`` masks), ``score_rewards`` / ``default_reward_adapter``, KV-cache output
rejection, temporary ``use_cache=False`` / attention-backend configuration with restore, the
flash->eager fallback on attention-import-like errors, and the metrics dictionary.

Difference: selected log-probs come from the registry's streaming ``logp`` operator (one pass over
the logits, no ``[B, S, V]`` fp32 log-softmax temporary) instead of ``log_softmax`` + ``gather``.
"""

from __future__ import annotations

import inspect
import time
from contextlib import contextmanager
from dataclasses import dataclass, replace
from typing import Any, Callable, Dict, Iterator, Mapping, Optional

import torch

from rl_engine.testing import selected_logprobs_reference

_BACKENDS = {"flash_attention_2", "sdpa", "eager", "model_default"}
_KV_KEYS = ("past_key_values", "kv_cache", "key_value_cache", "present_key_values", "presents")


@dataclass(frozen=True)
class StatelessForwardConfig:
    mode: str = "both"
    use_cache: bool = False
    attention_backend: str = "flash_attention_2"
    reject_kv_cache_outputs: bool = True
    detach_outputs: bool = True
    return_token_scores: bool = False
    max_batch_size: Optional[int] = None
    temperature: float = 1.0
    output_dtype: torch.dtype = torch.float32

    def __post_init__(self) -> None:
        if self.mode not in {"reference", "reward", "both"}:
            raise ValueError("mode must be 'reference', 'reward', or 'both'")
        if self.use_cache:
            raise ValueError("StatelessForwardConfig.use_cache must be False")
        if self.attention_backend not in _BACKENDS:
            raise ValueError("attention_backend must be 'flash_attention_2', 'sdpa', 'eager', or 'model_default'")
        if self.max_batch_size is not None and self.max_batch_size <= 0:
            raise ValueError("max_batch_size must be greater than zero")
        if self.temperature <= 0.0:
            raise ValueError("temperature must be greater than zero")


@dataclass(frozen=True)
class StatelessForwardInputs:
    input_ids: torch.Tensor
    attention_mask: torch.Tensor
    completion_mask: torch.Tensor
    labels: Optional[torch.Tensor] = None


@dataclass(frozen=True)
class StatelessForwardOutputs:
    raw: Any
    logits: Optional[torch.Tensor]
    kv_cache: Optional[Any] = None


@dataclass(frozen=True)
class StatelessForwardResult:
    reference_logps: Optional[torch.Tensor]
    rewards: Optional[torch.Tensor]
    token_scores: Optional[torch.Tensor]
    metrics: Mapping[str, Any]


@dataclass(frozen=True)
class TensorTreeSummary:
    tensor_count: int
    total_bytes: int

    @property
    def total_mb(self) -> float:
        return self.total_bytes / 1_048_576.0


RewardAdapter = Callable[[StatelessForwardOutputs, StatelessForwardInputs], torch.Tensor]


# ---------------------------------------------------------------------------------- tree helpers
def summarize_tensor_tree(value: Any) -> TensorTreeSummary:
    count = total = 0
    stack = [value]
    while stack:
        node = stack.pop()
        if isinstance(node, torch.Tensor):
            count += 1
            total += node.numel() * node.element_size()
        elif isinstance(node, Mapping):
            stack.extend(node.values())
        elif isinstance(node, (list, tuple)):
            stack.extend(node)
        elif node is not None and hasattr(node, "__dict__") and not isinstance(node, (str, bytes)):
            for attr in ("key_cache", "value_cache", "layers"):
                if hasattr(node, attr):
                    stack.append(getattr(node, attr))
    return TensorTreeSummary(count, total)


def extract_kv_cache_outputs(raw_outputs: Any) -> Optional[Any]:
    raw = raw_outputs
    for key in _KV_KEYS:
        value = raw.get(key) if isinstance(raw, Mapping) else getattr(raw, key, None)
        if value is not None and summarize_tensor_tree(value).tensor_count > 0:
            return value
    return None


def _named_tensor(raw: Any, names) -> Optional[torch.Tensor]:
    for name in names:
        value = raw.get(name) if isinstance(raw, Mapping) else getattr(raw, name, None)
        if isinstance(value, torch.Tensor):
            return value
    return None


def _logits_of(raw: Any) -> Optional[torch.Tensor]:
    if isinstance(raw, torch.Tensor):
        return raw
    found = _named_tensor(raw, ("logits",))
    if found is not None:
        return found
    if isinstance(raw, (tuple, list)):
        for item in raw:
            if isinstance(item, torch.Tensor) and item.ndim >= 2:
                return item
    return None


def _accepts(model: torch.nn.Module, keyword: str) -> bool:
    try:
        params = inspect.signature(model.forward).parameters
    except (TypeError, ValueError):
        return False
    return keyword in params or any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values())


# ------------------------------------------------------------------------- model configuration
_ABSENT = object()


class _ConfigEdits:
    """Applies the no-cache scoring policy to ``model.config`` / ``model.generation_config`` and remembers what was
    there, so that a temporary application can be undone exactly (attributes that did not exist are removed again).

    Hugging Face models pick their attention kernels from configuration attributes, not from forward arguments, so the
    backend is written to ``attn_implementation`` and ``_attn_implementation`` of every configuration object, whether
    or not it had them (reference: ``rl_engine/executors/stateless_executor.py:335-366,583-627``)."""

    def __init__(self, model: torch.nn.Module, config: StatelessForwardConfig) -> None:
        self._undo = []
        cache_targets = backend_targets = 0
        owners = []
        for name in ("config", "generation_config"):
            owner = getattr(model, name, None)
            if owner is not None and all(owner is not seen for seen in owners):
                owners.append(owner)
        for owner in owners:
            if hasattr(owner, "use_cache"):
                self._set(owner, "use_cache", False)
                cache_targets += 1
            if config.attention_backend != "model_default":
                try:
                    self._set(owner, "attn_implementation", config.attention_backend)
                    self._set(owner, "_attn_implementation", config.attention_backend)
                    backend_targets += 1
                except Exception:            # a configuration class that refuses the attribute: leave it alone
                    pass
        self.policy: Dict[str, Any] = {
            "attention_backend": config.attention_backend,
            "attention_backend_configured": backend_targets > 0,
            "attention_backend_config_targets": backend_targets,
            "model_config_use_cache_disabled": cache_targets > 0,
            "model_config_use_cache_targets": cache_targets,
            "reject_kv_cache_outputs": config.reject_kv_cache_outputs,
        }

    def _set(self, owner: Any, attr: str, value: Any) -> None:
        before = getattr(owner, attr, _ABSENT)
        setattr(owner, attr, value)
        self._undo.append((owner, attr, before))

    def undo(self) -> None:
        for owner, attr, before in reversed(self._undo):
            try:
                if before is _ABSENT:
                    if hasattr(owner, attr):
                        delattr(owner, attr)
                else:
                    setattr(owner, attr, before)
            except Exception:
                pass
        self._undo.clear()


@contextmanager
def _stateless_model_policy(model: torch.nn.Module, config: StatelessForwardConfig) -> Iterator[Dict[str, Any]]:
    """Temporarily force ``use_cache=False`` and the requested attention backend; restore on exit."""
    edits = _ConfigEdits(model, config)
    was_training = model.training
    model.eval()
    try:
        yield edits.policy
    finally:
        edits.undo()
        model.train(was_training)


def configure_stateless_model(model: torch.nn.Module, config: Optional[StatelessForwardConfig] = None) -> Dict[str, Any]:
    """Permanently apply the no-cache policy (same fields as the temporary context manager)."""
    return _ConfigEdits(model, config or StatelessForwardConfig()).policy


def _raised_inside_flash_attention(exc: BaseException) -> bool:
    """True if any frame of the exception's traceback belongs to a flash-attention code path (the ``flash_attn``
    package or a library's ``flash_attention`` integration module)."""
    tb = exc.__traceback__
    while tb is not None:
        name = tb.tb_frame.f_code.co_filename.replace("\\", "/").lower()
        if "flash_att" in name or "flash-att" in name:
            return True
        tb = tb.tb_next
    return False


def _attention_import_like(exc: Exception, config: StatelessForwardConfig) -> bool:
    """Should a failed forward be retried with eager attention?  Only when flash attention was requested, and the
    failure says so: a missing / unusable kernel package (ImportError, NotImplementedError), an error message that
    names flash attention or ``attn_implementation``, or ANY error raised from inside a flash-attention code path --
    libraries fail there in untyped ways, e.g. a bare ``StopIteration`` while probing an fp32 model's dtype (the
    reference special-cases that type: ``rl_engine/executors/stateless_executor.py:496-513``)."""
    if config.attention_backend != "flash_attention_2":
        return False
    if isinstance(exc, (ImportError, NotImplementedError, StopIteration)):
        return True
    text = f"{type(exc).__name__}: {exc}".lower()
    if any(key in text for key in ("flash_attn", "flash attention", "flashattention", "flash-attn", "attn_implementation")):
        return True
    return _raised_inside_flash_attention(exc)


def _forward_no_cache(model: torch.nn.Module, inputs: StatelessForwardInputs):
    kwargs: Dict[str, Any] = {}
    if _accepts(model, "attention_mask"):
        kwargs["attention_mask"] = inputs.attention_mask
    passed = _accepts(model, "use_cache")
    if passed:
        kwargs["use_cache"] = False
    return model(inputs.input_ids, **kwargs), passed


# ----------------------------------------------------------------------------------- scoring
def _validate(inputs: StatelessForwardInputs, config: StatelessForwardConfig) -> None:
    """Shape, device and mask rules of a scoring call (reference: ``rl_engine/executors/stateless_executor.py:440-471``)."""
    ids = inputs.input_ids
    if ids.ndim != 2:
        raise ValueError(f"input_ids must have shape [B, S], got {tuple(ids.shape)}")
    companions = {"attention_mask": inputs.attention_mask, "completion_mask": inputs.completion_mask}
    if inputs.labels is not None:
        companions["labels"] = inputs.labels
    for rule, bad in (("shape", lambda t: t.shape != ids.shape), ("device", lambda t: t.device != ids.device)):
        for name, tensor in companions.items():
            if bad(tensor):
                raise ValueError(f"{name} {rule} must match input_ids {rule}")
    if config.max_batch_size is not None and ids.shape[0] > config.max_batch_size:
        raise ValueError(f"batch size {ids.shape[0]} exceeds max_batch_size {config.max_batch_size}")
    keep = inputs.completion_mask.to(torch.bool)
    if config.mode in ("reference", "both"):
        if ids.shape[1] < 2:
            raise ValueError("reference scoring requires sequence_len >= 2")
        if bool(keep[:, 0].any()):
            raise ValueError("completion_mask[:, 0] must be False; completions cannot start at position 0")
    if not bool(keep.any()):
        raise ValueError("completion_mask must contain at least one active token")


def score_reference_logprobs(logits, inputs: StatelessForwardInputs, *, temperature: float = 1.0,
                             output_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    if logits.ndim != 3:
        raise ValueError(f"reference logits must have shape [B, S, V], got {tuple(logits.shape)}")
    if tuple(logits.shape[:2]) != tuple(inputs.input_ids.shape):
        raise ValueError(
            "reference logits leading shape must match input_ids shape, got "
            f"{tuple(logits.shape[:2])} and {tuple(inputs.input_ids.shape)}"
        )
    labels = inputs.input_ids if inputs.labels is None else inputs.labels
    if labels.shape != inputs.input_ids.shape:
        raise ValueError("labels shape must match input_ids shape")
    keep = inputs.completion_mask.to(device=logits.device, dtype=torch.bool)
    if bool(keep[:, 0].any()):
        raise ValueError("completion_mask[:, 0] must be False; completions cannot start at position 0")
    nxt_logits, nxt_labels, nxt_keep = logits[:, :-1], labels[:, 1:].to(logits.device), keep[:, 1:]
    if logits.is_cuda and temperature == 1.0:
        from rl_engine.kernels.registry import kernel_registry

        ids = torch.where(nxt_keep, nxt_labels, torch.zeros_like(nxt_labels))
        picked = kernel_registry.get_op("logp").apply_fp32(nxt_logits, ids)
        picked = torch.where(nxt_keep, picked, torch.zeros_like(picked)).to(output_dtype)
    else:
        picked = selected_logprobs_reference(nxt_logits, nxt_labels, mask=nxt_keep, temperature=temperature,
                                             output_dtype=output_dtype)
    out = torch.zeros(inputs.input_ids.shape, dtype=output_dtype, device=logits.device)
    out[:, 1:] = picked
    return out


def default_reward_adapter(outputs: StatelessForwardOutputs, inputs: StatelessForwardInputs) -> torch.Tensor:
    found = _named_tensor(outputs.raw, ("rewards", "reward", "scores", "score"))
    if found is None:
        found = outputs.logits
    if found is None:
        raise ValueError("reward mode requires scalar logits or a reward_adapter")
    if found.ndim == 2 and found.shape[1] == 1:
        found = found[:, 0]
    if found.ndim != 1:
        raise ValueError(f"reward tensor must have shape [B] or [B, 1], got {tuple(found.shape)}")
    return found


def score_rewards(outputs, inputs, *, reward_adapter: RewardAdapter, output_dtype=torch.float32) -> torch.Tensor:
    rewards = reward_adapter(outputs, inputs)
    if not isinstance(rewards, torch.Tensor):
        raise TypeError("reward_adapter must return a torch.Tensor")
    if rewards.ndim != 1:
        raise ValueError(f"reward_adapter must return shape [B], got {tuple(rewards.shape)}")
    if rewards.shape[0] != inputs.input_ids.shape[0]:
        raise ValueError(
            f"reward_adapter batch size {rewards.shape[0]} must match input batch size {inputs.input_ids.shape[0]}"
        )
    return rewards.to(device=inputs.input_ids.device, dtype=output_dtype)


def collect_stateless_metrics(inputs, *, mode, elapsed_seconds, use_cache_passed, detached_outputs, cuda_tracking,
                              no_cache_policy, kv_cache_summary: TensorTreeSummary) -> Dict[str, Any]:
    ids = inputs.input_ids
    metrics: Dict[str, Any] = {
        "mode": mode,
        "batch_size": int(ids.shape[0]),
        "sequence_len": int(ids.shape[1]),
        "active_completion_tokens": int(inputs.completion_mask.to(torch.bool).sum()),
        "device": str(ids.device),
        "dtype": str(ids.dtype).replace("torch.", ""),
        "elapsed_ms": elapsed_seconds * 1000.0,
        "use_cache": False,
        "use_cache_passed": bool(use_cache_passed),
        "detached_outputs": bool(detached_outputs),
        "zero_kv_cache": kv_cache_summary.tensor_count == 0,
        "kv_cache_output_present": kv_cache_summary.tensor_count > 0,
        "kv_cache_output_tensors": kv_cache_summary.tensor_count,
        "kv_cache_output_bytes": kv_cache_summary.total_bytes,
        "kv_cache_output_mb": kv_cache_summary.total_mb,
        **dict(no_cache_policy),
    }
    if cuda_tracking:
        metrics["peak_allocated_mb"] = torch.cuda.max_memory_allocated(ids.device) / 1_048_576.0
        metrics["peak_reserved_mb"] = torch.cuda.max_memory_reserved(ids.device) / 1_048_576.0
    return metrics


class StatelessForwardExecutor:
    def __init__(self, model: torch.nn.Module, config: Optional[StatelessForwardConfig] = None, *,
                 reward_adapter: Optional[RewardAdapter] = None) -> None:
        self.model = model
        self.config = config or StatelessForwardConfig()
        self.reward_adapter = reward_adapter or default_reward_adapter

    def score(self, inputs: StatelessForwardInputs) -> StatelessForwardResult:
        cfg = self.config
        _validate(inputs, cfg)
        device = inputs.input_ids.device
        tracking = device.type == "cuda" and torch.cuda.is_available()
        if tracking:
            torch.cuda.reset_peak_memory_stats(device)
            torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        with _stateless_model_policy(self.model, cfg) as policy, torch.no_grad():
            try:
                raw, passed = _forward_no_cache(self.model, inputs)
                policy["attention_backend_fallback"] = False
            except Exception as exc:
                if not _attention_import_like(exc, cfg):
                    raise
                with _stateless_model_policy(self.model, replace(cfg, attention_backend="eager")) as fallback:
                    raw, passed = _forward_no_cache(self.model, inputs)
                policy.update(fallback)
                policy.update(attention_backend_requested=cfg.attention_backend, attention_backend_fallback=True,
                              attention_backend_fallback_reason=f"{type(exc).__name__}: {str(exc)[:200]}")
            kv = extract_kv_cache_outputs(raw)
            kv_summary = summarize_tensor_tree(kv)
            if cfg.reject_kv_cache_outputs and kv is not None:
                raise ValueError(
                    "stateless scoring received KV-cache outputs despite use_cache=False "
                    f"({kv_summary.tensor_count} tensors, {kv_summary.total_mb:.4f} MiB)."
                )
            outputs = StatelessForwardOutputs(raw=raw, logits=_logits_of(raw), kv_cache=kv)
            ref = rewards = tokens = None
            if cfg.mode in {"reference", "both"}:
                if outputs.logits is None:
                    raise ValueError("reference mode requires model outputs to expose logits")
                ref = score_reference_logprobs(outputs.logits, inputs, temperature=cfg.temperature,
                                               output_dtype=cfg.output_dtype)
                tokens = ref if cfg.return_token_scores else None
            if cfg.mode in {"reward", "both"}:
                rewards = score_rewards(outputs, inputs, reward_adapter=self.reward_adapter, output_dtype=cfg.output_dtype)
            if cfg.detach_outputs:
                ref, rewards, tokens = (None if t is None else t.detach() for t in (ref, rewards, tokens))
        if tracking:
            torch.cuda.synchronize(device)
        metrics = collect_stateless_metrics(
            inputs, mode=cfg.mode, elapsed_seconds=time.perf_counter() - t0, use_cache_passed=passed,
            detached_outputs=cfg.detach_outputs, cuda_tracking=tracking, no_cache_policy=policy, kv_cache_summary=kv_summary,
        )
        return StatelessForwardResult(reference_logps=ref, rewards=rewards, token_scores=tokens, metrics=metrics)
