"""Data contracts between rollout, scoring and training workers, and rollout-payload decoding.

Parity: ``rl_engine/executors/training_contract.py:20-1017`` of the reference — the stage result
dataclasses, ``TrainingWorker`` protocol, ``TorchRLTrainingConfig``, ``RolloutBatchMixin`` (build a
``SyntheticRLKernelBatch`` from a vLLM-style payload: token ids ``% vocab``, payload rewards or a
token-id proxy, payload reference log-probs or a synthetic offset, else a seeded synthetic batch),
``StatelessScoringWorker``, ``build_stateless_inputs_from_rollout_payload`` and the payload
extractors, which accept dicts or objects, flat or nested under ``outputs``.

One recursive field finder replaces the reference's four near-identical candidate walkers, and
batches are assembled with padded tensor ops instead of per-candidate tensor writes.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Protocol, Sequence, Tuple

import torch

from rl_engine.executors.stateless_executor import StatelessForwardExecutor, StatelessForwardInputs, StatelessForwardResult
from rl_engine.testing import SyntheticRLKernelBatch, make_synthetic_rl_kernel_batch

_TOKEN_KEYS = ("token_ids",)
_PROMPT_KEYS = ("prompt_token_ids", "prompt_ids", "input_token_ids", "input_ids")
_REWARD_KEYS = ("reward", "score", "scalar_reward", "reward_score")
_REF_KEYS = ("reference_logps", "ref_logps", "reference_logprobs", "ref_logprobs")
_GROUP_KEYS = ("normalized_outputs", "outputs", "candidates", "groups")


@dataclass(frozen=True)
class RolloutStageResult:
    iteration: int
    weight_version: int
    payload: Any
    started_at: float
    finished_at: float
    metrics: Mapping[str, Any] = field(default_factory=dict)

    @property
    def duration_seconds(self) -> float:
        return self.finished_at - self.started_at


@dataclass(frozen=True)
class TrainingStageResult:
    iteration: int
    consumed_weight_version: int
    published_weight_version: Optional[int]
    metrics: Mapping[str, Any]
    started_at: float
    finished_at: float

    @property
    def duration_seconds(self) -> float:
        return self.finished_at - self.started_at


class TrainingWorker(Protocol):
    def train(self, rollout: RolloutStageResult) -> TrainingStageResult: ...


@dataclass(frozen=True)
class TorchRLTrainingConfig:
    num_prompts: int = 1
    samples_per_prompt: int = 2
    prompt_len: int = 4
    completion_len: int = 8
    vocab_size: int = 64
    hidden_dim: int = 32
    valid_density: float = 0.75
    lr: float = 1e-3
    device: str = "cpu"
    dtype: torch.dtype = torch.float32
    seed: int = 0
    min_completion_len: int = 1
    advantage_eps: float = 1e-8


# ------------------------------------------------------------------------------ payload walking
def _is_seq(value: Any) -> bool:
    return isinstance(value, Sequence) and not isinstance(value, (str, bytes))


def _get(node: Any, key: str) -> Any:
    return node.get(key) if isinstance(node, Mapping) else getattr(node, key, None)


def _has(node: Any, key: str) -> bool:
    return key in node if isinstance(node, Mapping) else hasattr(node, key)


def _find_field(candidate: Any, keys: Tuple[str, ...], *, nested_first: bool) -> Any:
    """Value of the first of ``keys`` on ``candidate`` or on any entry of its ``outputs`` (recursively)."""
    if candidate is None:
        return None

    def nested() -> Any:
        inner = _get(candidate, "outputs")
        if _is_seq(inner):
            for item in inner:
                found = _find_field(item, keys, nested_first=nested_first)
                if found is not None and (not _is_seq(found) or len(found)):
                    return found
        return None

    def direct() -> Any:
        for key in keys:
            if _has(candidate, key):
                value = _get(candidate, key)
                if value is not None:
                    return value
        return None

    order = (nested, direct) if nested_first else (direct, nested)
    for probe in order:
        found = probe()
        if found is not None:
            return found
    return None


def _ints(value: Any) -> List[int]:
    if value is None:
        return []
    if isinstance(value, torch.Tensor):
        return [int(v) for v in value.detach().cpu().reshape(-1).tolist()]
    return [int(v) for v in value] if _is_seq(value) else []


def _floats(value: Any) -> List[float]:
    if value is None:
        return []
    if isinstance(value, torch.Tensor):
        return [float(v) for v in value.detach().cpu().reshape(-1).tolist()]
    return [float(v) for v in value] if _is_seq(value) else []


def _scalar(value: Any) -> Optional[float]:
    if value is None:
        return None
    if isinstance(value, torch.Tensor):
        flat = value.detach().cpu().reshape(-1)
        return float(flat[0]) if flat.numel() else None
    try:
        return float(value)
    except (TypeError, ValueError):
        return None


def _grouped_outputs(payload: Any) -> List[List[Any]]:
    """``payload`` -> list of prompt groups, each a list of candidate records."""
    if payload is None:
        return []
    for key in _GROUP_KEYS:
        groups = _get(payload, key)
        if _is_seq(groups) and len(groups):
            out = []
            for group in groups:
                if _is_seq(group):
                    out.append(list(group))
                else:  # one request object holding its candidates under .outputs
                    inner = _get(group, "outputs")
                    out.append(list(inner) if _is_seq(inner) and len(inner) else [group])
            return out
    return []


def extract_rollout_candidate_groups(payload: Any) -> List[List[List[int]]]:
    direct = _get(payload, "token_groups") if payload is not None else None
    if _is_seq(direct) and len(direct):
        return [[_ints(tokens)] for tokens in direct]
    groups = []
    for group in _grouped_outputs(payload):
        tokens = [_ints(_find_field(c, _TOKEN_KEYS, nested_first=True)) for c in group]
        tokens = [t for t in tokens if t]
        if tokens:
            groups.append(tokens)
    return groups


def extract_rollout_token_groups(payload: Any) -> List[List[int]]:
    return [tokens for group in extract_rollout_candidate_groups(payload) for tokens in group]


def extract_rollout_reward_groups(payload: Any) -> List[List[float]]:
    out = []
    for group in _grouped_outputs(payload):
        rewards = [_scalar(_find_field(c, _REWARD_KEYS, nested_first=True)) for c in group]
        out.append([r for r in rewards if r is not None])
    return out


def extract_rollout_reference_logp_groups(payload: Any) -> List[List[List[float]]]:
    return [[_floats(_find_field(c, _REF_KEYS, nested_first=True)) for c in group] for group in _grouped_outputs(payload)]


def _records(payload: Any) -> List[Tuple[List[int], List[int]]]:
    """(prompt ids, completion ids) per candidate, in payload order."""
    direct = _get(payload, "token_groups") if payload is not None else None
    if _is_seq(direct) and len(direct):
        return [([], _ints(t)) for t in direct]
    out = []
    for group in _grouped_outputs(payload):
        for cand in group:
            tokens = _ints(_find_field(cand, _TOKEN_KEYS, nested_first=True))
            if tokens:
                out.append((_ints(_find_field(cand, _PROMPT_KEYS, nested_first=False)), tokens))
    return out


def _groups_match(candidates, values, *, per_token: bool = False, max_len: Optional[int] = None) -> bool:
    if len(values) != len(candidates):
        return False
    for cand_group, value_group in zip(candidates, values):
        if len(cand_group) != len(value_group):
            return False
        if per_token:
            for tokens, vals in zip(cand_group, value_group):
                need = len(tokens) if max_len is None else min(len(tokens), max_len)
                if len(vals) < need or not vals:
                    return False
    return bool(candidates)


# ------------------------------------------------------------------------------ batch building
def group_relative_advantages(rewards: torch.Tensor, group_ids: torch.Tensor, num_groups: int, eps: float) -> torch.Tensor:
    r = rewards.float()
    zeros = r.new_zeros(num_groups)
    count = zeros.index_add(0, group_ids, torch.ones_like(r)).clamp_min(1.0)
    mean = zeros.index_add(0, group_ids, r) / count
    centered = r - mean[group_ids]
    var = zeros.index_add(0, group_ids, centered * centered) / count
    return centered / torch.sqrt(var.clamp_min(0.0) + eps)[group_ids]


def objective_reference_logps(current_logps: torch.Tensor, batch: SyntheticRLKernelBatch) -> torch.Tensor:
    """Payload reference log-probs when the batch carries them, else ``current - 0.02`` (detached)."""
    if batch.metadata.get("reference_logp_source") == "payload_reference_logps":
        return batch.ref_logps.to(device=current_logps.device, dtype=current_logps.dtype)
    return current_logps.detach() - 0.02


def _pad(rows: List[List[float]], width: int, dtype, device, fill=0) -> torch.Tensor:
    out = torch.full((len(rows), width), fill, dtype=dtype)
    for i, row in enumerate(rows):
        n = min(len(row), width)
        if n:
            out[i, :n] = torch.tensor(row[:n], dtype=dtype)
    return out.to(device)


class RolloutBatchMixin:
    config: TorchRLTrainingConfig
    device: torch.device

    def _batch_from_rollout_or_synthetic(self, rollout: RolloutStageResult):
        cfg = self.config
        candidates = extract_rollout_candidate_groups(rollout.payload)
        if candidates:
            rewards = extract_rollout_reward_groups(rollout.payload)
            refs = extract_rollout_reference_logp_groups(rollout.payload)
            use_rewards = _groups_match(candidates, rewards)
            use_refs = _groups_match(candidates, refs, per_token=True, max_len=cfg.completion_len)
            batch = self._batch_from_candidate_groups(
                candidates, rollout, reward_groups=rewards if use_rewards else None,
                reference_logp_groups=refs if use_refs else None,
            )
            flat = [t for g in candidates for t in g]
            return batch, {
                "training_data_source": "rollout_payload",
                "reward_source": "payload_rewards" if use_rewards else "token_id_proxy",
                "reference_logp_source": "payload_reference_logps" if use_refs else "synthetic_current_offset",
                "rollout_prompt_groups": len(candidates),
                "rollout_sequences": len(flat),
                "rollout_tokens": sum(len(t) for t in flat),
            }
        batch = make_synthetic_rl_kernel_batch(
            num_prompts=cfg.num_prompts, samples_per_prompt=cfg.samples_per_prompt, prompt_len=cfg.prompt_len,
            completion_len=cfg.completion_len, vocab_size=cfg.vocab_size, valid_density=cfg.valid_density,
            dtype=cfg.dtype, device=self.device, seed=cfg.seed + int(rollout.iteration),
        )
        return batch, {
            "training_data_source": "synthetic_fallback", "rollout_sequences": 0, "rollout_tokens": 0,
            "reward_source": "synthetic_rewards", "reference_logp_source": "synthetic_current_offset",
        }

    def _batch_from_token_groups(self, token_groups, rollout):
        return self._batch_from_candidate_groups([[list(g)] for g in token_groups], rollout)

    def _batch_from_candidate_groups(self, candidate_groups, rollout, *, reward_groups=None, reference_logp_groups=None):
        cfg = self.config
        flat = [list(t) for g in candidate_groups for t in g]
        group_ids = [gi for gi, g in enumerate(candidate_groups) for _ in g]
        width = max(cfg.min_completion_len, min(cfg.completion_len, max(len(t) for t in flat)))
        b = len(flat)
        token_ids = _pad([[int(x) % cfg.vocab_size for x in t] for t in flat], width, torch.long, self.device)
        lengths = torch.tensor([min(len(t), width) for t in flat], device=self.device)
        completion_mask = torch.arange(width, device=self.device)[None, :] < lengths[:, None]
        if not bool(completion_mask.any()):
            completion_mask[:, :1] = True
        if reward_groups is not None:
            reward_list = [float(r) for g in reward_groups for r in g]
        else:  # deterministic proxy so that training still has a signal: mean token id scaled to [0, 1)
            reward_list = [(sum(int(x) % cfg.vocab_size for x in t) / max(len(t), 1)) / cfg.vocab_size for t in flat]
        rewards = torch.tensor(reward_list, dtype=cfg.dtype, device=self.device)
        gid = torch.tensor(group_ids, dtype=torch.long, device=self.device)
        seq_adv = group_relative_advantages(rewards, gid, len(candidate_groups), cfg.advantage_eps)
        advantages = torch.where(completion_mask, seq_adv[:, None].expand(b, width), torch.zeros(())).to(cfg.dtype)
        ref_logps = torch.zeros(b, width, dtype=cfg.dtype, device=self.device)
        if reference_logp_groups is not None:
            ref_logps = _pad([list(v) for g in reference_logp_groups for v in g], width, cfg.dtype, self.device)
        prompt = torch.zeros(b, cfg.prompt_len, dtype=torch.long, device=self.device)
        input_ids = torch.cat([prompt, token_ids], dim=1)
        prompt_mask = torch.zeros_like(input_ids, dtype=torch.bool)
        prompt_mask[:, : cfg.prompt_len] = True
        attention_mask = torch.cat([prompt_mask[:, : cfg.prompt_len], completion_mask], dim=1)
        meta: Dict[str, Any] = {
            "num_prompts": len(candidate_groups), "samples_per_prompt": max(len(g) for g in candidate_groups),
            "batch_size": b, "prompt_len": cfg.prompt_len, "completion_len": width,
            "total_seq_len": cfg.prompt_len + width, "vocab_size": cfg.vocab_size,
            "valid_density": float(completion_mask.float().mean()), "valid_tokens": int(completion_mask.sum()),
            "dtype": cfg.dtype, "device": str(self.device), "seed": cfg.seed + int(rollout.iteration),
            "source": "rollout_payload", "group_ids": group_ids,
            "reward_source": "payload_rewards" if reward_groups is not None else "token_id_proxy",
            "reference_logp_source": "payload_reference_logps" if reference_logp_groups is not None else "synthetic_current_offset",
        }
        return SyntheticRLKernelBatch(
            input_ids=input_ids, attention_mask=attention_mask, prompt_mask=prompt_mask, completion_mask=completion_mask,
            token_ids=token_ids, rewards=rewards, advantages=advantages,
            old_logps=torch.zeros(b, width, dtype=cfg.dtype, device=self.device), ref_logps=ref_logps,
            valid_indices=completion_mask.reshape(-1).nonzero().squeeze(-1), metadata=meta,
        )


# --------------------------------------------------------------------------------- stage glue
def make_rollout_result(*, iteration: int, weight_version: int, payload: Any,
                        metrics: Optional[Mapping[str, Any]] = None) -> RolloutStageResult:
    now = time.perf_counter()
    return RolloutStageResult(iteration=iteration, weight_version=weight_version, payload=payload, started_at=now,
                              finished_at=time.perf_counter(), metrics=dict(metrics or {}))


def build_stateless_inputs_from_rollout_payload(payload: Any, *, prompt_len: Optional[int] = 1, prompt_token_id: int = 0,
                                                max_completion_len: Optional[int] = None,
                                                device="cpu") -> StatelessForwardInputs:
    if prompt_len is not None and prompt_len < 0:
        raise ValueError("prompt_len must be non-negative")
    if max_completion_len is not None and max_completion_len <= 0:
        raise ValueError("max_completion_len must be greater than zero")
    records = _records(payload)
    if not records:
        raise ValueError("rollout payload does not contain candidate token ids")
    width = max(len(t) for _p, t in records)
    if max_completion_len is not None:
        width = min(width, max_completion_len)
    width = max(1, width)
    p_len = max((len(p) for p, _t in records), default=0) if prompt_len is None else prompt_len
    dev = torch.device(device)
    ids = torch.full((len(records), p_len + width), int(prompt_token_id), dtype=torch.long)
    attn = torch.zeros_like(ids, dtype=torch.bool)
    comp = torch.zeros_like(ids, dtype=torch.bool)
    if p_len and prompt_len is not None:
        attn[:, :p_len] = True
    for row, (prompt, tokens) in enumerate(records):
        if p_len and prompt:
            clipped = prompt[:p_len]
            ids[row, : len(clipped)] = torch.tensor(clipped)
            if prompt_len is None:
                attn[row, : len(clipped)] = True
        clipped = tokens[:width]
        if clipped:
            ids[row, p_len : p_len + len(clipped)] = torch.tensor(clipped)
            attn[row, p_len : p_len + len(clipped)] = True
            comp[row, p_len : p_len + len(clipped)] = True
    if not bool(comp.any()):
        raise ValueError("rollout payload does not contain active completion tokens")
    return StatelessForwardInputs(input_ids=ids.to(dev), attention_mask=attn.to(dev), completion_mask=comp.to(dev))


def _candidate_copy(candidate: Any) -> Dict[str, Any]:
    """A candidate as a fresh dict (mappings are copied, objects give their attributes), so that attaching scores never
    writes into the rollout's own records."""
    if isinstance(candidate, Mapping):
        return dict(candidate)
    try:
        return dict(vars(candidate))
    except TypeError:
        return {"candidate": candidate}


def _attach_per_candidate(scored: Dict[str, Any], values: List[Any], fields: Callable[[Any], Dict[str, Any]], what: str) -> None:
    """Gives every candidate that carries token ids, in payload order, its entry of ``values``.  The grouped outputs are
    rebuilt (``normalized_outputs`` first, else ``outputs``); a payload without such candidates is left alone; a count
    that does not match is an error rather than a partial attachment."""
    if not values:
        return
    for key in ("normalized_outputs", "outputs"):
        grouped = scored.get(key)
        if not _is_seq(grouped):
            continue
        cursor, rebuilt = 0, []
        for group in grouped:
            members = list(group) if _is_seq(group) and not isinstance(group, Mapping) else [group]
            new_group = []
            for cand in members:
                if not _ints(_find_field(cand, _TOKEN_KEYS, nested_first=True)):
                    new_group.append(cand)
                    continue
                if cursor >= len(values):
                    raise ValueError(f"stateless {what} count must match rollout candidate count, got fewer "
                                     f"{what} than candidates")
                updated = _candidate_copy(cand)
                updated.update(fields(values[cursor]))
                new_group.append(updated)
                cursor += 1
            rebuilt.append(new_group)
        if cursor == 0:
            continue
        if cursor != len(values):
            raise ValueError(f"stateless {what} count must match rollout candidate count, got {len(values)} {what} "
                             f"for {cursor} candidates")
        scored[key] = rebuilt
        return


def attach_stateless_scores_to_payload(payload: Any, result: StatelessForwardResult, *,
                                       inputs: Optional[StatelessForwardInputs] = None) -> Dict[str, Any]:
    """The rollout payload plus ``stateless_scores`` and, per candidate, ``reward`` / ``reference_logps`` with their
    ``*_source`` set to ``"stateless_executor"`` (reference: ``rl_engine/executors/training_contract.py:351-374,
    546-604``).  The input payload and its candidates are not modified."""
    scored = dict(payload) if isinstance(payload, Mapping) else {"raw_payload": payload}
    scored["stateless_scores"] = {
        "reference_logps": result.reference_logps, "rewards": result.rewards, "token_scores": result.token_scores,
        "metrics": dict(result.metrics),
    }
    if result.rewards is not None:
        rewards = [float(v) for v in result.rewards.detach().cpu().reshape(-1).tolist()]
        _attach_per_candidate(scored, rewards, lambda v: {"reward": v, "reward_source": "stateless_executor"}, "reward")
    if result.reference_logps is not None and inputs is not None:
        if result.reference_logps.shape != inputs.completion_mask.shape:
            raise ValueError("reference_logps shape must match completion_mask shape")
        ref = result.reference_logps.detach().cpu()
        mask = inputs.completion_mask.detach().cpu().to(torch.bool)
        rows = [[float(v) for v in ref[r][mask[r]].tolist()] for r in range(ref.shape[0])]
        _attach_per_candidate(scored, rows, lambda v: {"reference_logps": v, "reference_logp_source": "stateless_executor"},
                              "reference_logps row")
    return scored


class StatelessScoringWorker:
    def __init__(self, executor: StatelessForwardExecutor,
                 collate_inputs: Callable[[RolloutStageResult], StatelessForwardInputs]) -> None:
        self.executor = executor
        self.collate_inputs = collate_inputs

    def score(self, rollout: RolloutStageResult) -> RolloutStageResult:
        t0 = time.perf_counter()
        inputs = self.collate_inputs(rollout)
        result = self.executor.score(inputs)
        m = result.metrics
        return RolloutStageResult(
            iteration=rollout.iteration, weight_version=rollout.weight_version,
            payload=attach_stateless_scores_to_payload(rollout.payload, result, inputs=inputs),
            started_at=t0, finished_at=time.perf_counter(),
            metrics={
                **dict(rollout.metrics), "scoring_backend": "stateless", "scoring_mode": m["mode"],
                "scoring_elapsed_ms": m["elapsed_ms"], "scoring_active_completion_tokens": m["active_completion_tokens"],
                "scoring_zero_kv_cache": m["zero_kv_cache"], "scoring_attention_backend": m["attention_backend"],
                "scoring_kv_cache_output_mb": m["kv_cache_output_mb"],
            },
        )
