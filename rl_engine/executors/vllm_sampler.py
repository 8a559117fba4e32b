"""Shared-prefix rollout sampling through a vLLM-shaped engine (lazy, injectable).

Parity: ``rl_engine/executors/vllm_sampler.py:11-303`` of the reference — ``VLLMSamplerConfig``
(``from_model_config`` merges ``vllm`` < ``sampler`` < top-level keys), prompts repeated
``num_generations`` times back to back so the engine's prefix cache hits, outputs regrouped per
prompt, and ``NormalizedRolloutCandidate`` records.  vLLM is imported only when an engine has to be
built; tests inject ``llm_cls`` / ``sampling_params_cls`` or a ready engine.
"""

from __future__ import annotations

import importlib
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Union

Prompt = Union[str, Mapping[str, Any]]


@dataclass(frozen=True)
class VLLMSamplerConfig:
    model: Optional[str] = None
    num_generations: int = 1
    enable_prefix_caching: bool = True
    sampling_params: Mapping[str, Any] = field(default_factory=dict)
    engine_kwargs: Mapping[str, Any] = field(default_factory=dict)
    backend: str = "vllm"

    def __post_init__(self) -> None:
        if self.num_generations < 1:
            raise ValueError("num_generations must be >= 1")
        if self.backend != "vllm":
            raise ValueError(f"Unsupported rollout sampler backend: {self.backend}")

    @classmethod
    def from_model_config(cls, model_config: Optional[Mapping[str, Any]]) -> "VLLMSamplerConfig":
        raw = dict(model_config or {})
        merged: Dict[str, Any] = {}
        for layer in (raw.get("vllm", {}), raw.get("sampler", {}),
                      {k: v for k, v in raw.items() if k not in {"sampler", "vllm"}}):
            merged.update(dict(layer))
        return cls(
            model=merged.get("model"),
            num_generations=int(merged.get("num_generations", 1)),
            enable_prefix_caching=bool(merged.get("enable_prefix_caching", True)),
            sampling_params=dict(merged.get("sampling_params", {})),
            engine_kwargs=dict(merged.get("engine_kwargs", {})),
            backend=merged.get("backend", "vllm"),
        )


@dataclass(frozen=True)
class NormalizedRolloutCandidate:
    prompt_index: int
    candidate_index: int
    request_id: Optional[str]
    prompt_token_ids: Optional[List[int]]
    token_ids: List[int]
    text: str
    finish_reason: Optional[str]
    cumulative_logprob: Optional[float]
    logprobs: Optional[Any] = None
    raw_output: Optional[Any] = field(default=None, repr=False, compare=False)

    def to_dict(self, *, include_raw: bool = False) -> Dict[str, Any]:
        data = asdict(self)
        if not include_raw:
            data.pop("raw_output", None)
        return data


def _is_seq(v: Any) -> bool:
    return isinstance(v, Sequence) and not isinstance(v, (str, bytes))


def _field(node: Any, name: str) -> Any:
    if node is None:
        return None
    return node.get(name) if isinstance(node, Mapping) else getattr(node, name, None)


def _int_list(v: Any) -> Optional[List[int]]:
    if v is None:
        return None
    try:
        return [int(x) for x in v]
    except TypeError:
        return None


def _opt_float(v: Any) -> Optional[float]:
    try:
        return None if v is None else float(v)
    except (TypeError, ValueError):
        return None


def normalize_output_candidate(raw_output: Any, *, prompt_index: int, candidate_index: int) -> NormalizedRolloutCandidate:
    inner = _field(raw_output, "outputs")
    body = inner[0] if _is_seq(inner) and len(inner) else raw_output
    pick = lambda name: _field(body, name) if _field(body, name) is not None else _field(raw_output, name)
    return NormalizedRolloutCandidate(
        prompt_index=prompt_index,
        candidate_index=candidate_index,
        request_id=_field(raw_output, "request_id"),
        prompt_token_ids=_int_list(_field(raw_output, "prompt_token_ids")),
        token_ids=_int_list(_field(body, "token_ids")) or [],
        text=str(pick("text") or ""),
        finish_reason=pick("finish_reason"),
        cumulative_logprob=_opt_float(pick("cumulative_logprob")),
        logprobs=pick("logprobs"),
        raw_output=raw_output,
    )


def normalize_grouped_outputs(grouped_outputs: Sequence[Sequence[Any]]) -> List[List[NormalizedRolloutCandidate]]:
    return [
        [normalize_output_candidate(out, prompt_index=p, candidate_index=c) for c, out in enumerate(group)]
        for p, group in enumerate(grouped_outputs)
    ]


def _as_prompt_list(prompts: Union[Prompt, Sequence[Prompt]]) -> List[Prompt]:
    if isinstance(prompts, (str, Mapping)):
        return [prompts]
    out = list(prompts)
    if not out:
        raise ValueError("at least one prompt is required")
    for p in out:
        if not isinstance(p, (str, Mapping)):
            raise TypeError(f"prompts must be strings or mappings, got {type(p)!r}")
    return out


def _regroup(outputs: Sequence[Any], num_prompts: int, generations: int) -> List[List[Any]]:
    flat = list(outputs)
    if len(flat) != num_prompts * generations:
        raise ValueError(
            f"vLLM returned {len(flat)} outputs, expected {num_prompts * generations} "
            f"({num_prompts} prompts x {generations} generations)"
        )
    return [flat[i * generations : (i + 1) * generations] for i in range(num_prompts)]


class VLLMSharedPrefixSampler:
    def __init__(self, config: VLLMSamplerConfig, *, engine: Optional[Any] = None, llm_cls: Optional[type] = None,
                 sampling_params_cls: Optional[type] = None) -> None:
        self.config = config
        self._engine = engine
        self._llm_cls = llm_cls
        self._sampling_params_cls = sampling_params_cls

    @property
    def engine(self) -> Any:
        if self._engine is None:
            self._engine = self._build_engine()
        return self._engine

    def generate(self, prompts, *, num_generations: Optional[int] = None,
                 sampling_params: Optional[Mapping[str, Any]] = None) -> Dict[str, Any]:
        plist = _as_prompt_list(prompts)
        generations = num_generations or self.config.num_generations
        if generations < 1:
            raise ValueError("num_generations must be >= 1")
        # all copies of one prompt are adjacent: the engine sees the shared prefix back to back
        expanded = [p for p in plist for _ in range(generations)]
        outputs = self.engine.generate(expanded, self._sampling_params(sampling_params))
        grouped = _regroup(outputs, len(plist), generations)
        return {
            "backend": self.config.backend,
            "prefix_cache_enabled": self.config.enable_prefix_caching,
            "num_prompts": len(plist),
            "num_generations": generations,
            "outputs": grouped,
            "normalized_outputs": normalize_grouped_outputs(grouped),
        }

    def _classes(self):
        if self._llm_cls is None or self._sampling_params_cls is None:
            vllm = importlib.import_module("vllm")
            self._llm_cls = self._llm_cls or vllm.LLM
            self._sampling_params_cls = self._sampling_params_cls or vllm.SamplingParams
        return self._llm_cls, self._sampling_params_cls

    def _build_engine(self) -> Any:
        if not self.config.model:
            raise ValueError("A model path or model name is required for vLLM rollout sampling.")
        llm_cls, _ = self._classes()
        kwargs = dict(self.config.engine_kwargs, model=self.config.model,
                      enable_prefix_caching=self.config.enable_prefix_caching)
        try:
            return llm_cls(**kwargs)
        except TypeError as exc:
            raise TypeError(
                "Failed to construct vLLM LLM with enable_prefix_caching. "
                "Verify the installed vLLM version supports this engine argument."
            ) from exc

    def _sampling_params(self, overrides: Optional[Mapping[str, Any]]) -> Any:
        _, cls = self._classes()
        return cls(**{**dict(self.config.sampling_params), **dict(overrides or {})})
