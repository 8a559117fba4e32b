"""Ray actor placement for rollout and training workers (Ray is optional, lazy and injectable).

Parity: ``rl_engine/executors/ray_actor_manager.py:13-233`` of the reference — runtime / actor-option
/ worker-spec dataclasses, a generic worker actor shim, synchronous handles
(``rollout`` / ``update_weights`` / ``release_weights`` and ``train`` / ``publish_weights`` /
``release_weights``), ``health_check`` and reverse-order ``shutdown``.  Tests pass a fake
``ray_module``; importing this file never imports Ray.
"""

from __future__ import annotations

import importlib
from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Tuple


class RayUnavailableError(RuntimeError):
    """Ray is not installed (or could not be imported) and no ``ray_module`` was injected."""


@dataclass(frozen=True)
class RayRuntimeConfig:
    """``auto_init``: call ``ray.init`` when the runtime is not up yet (off: the caller has initialised Ray);
    ``shutdown_ray_on_close``: ``ray.shutdown()`` after the actors were killed.  ``address`` / ``namespace`` are
    shorthands for the same keys of ``init_kwargs``."""

    auto_init: bool = True
    init_kwargs: Mapping[str, Any] = field(default_factory=dict)
    shutdown_ray_on_close: bool = False
    address: Optional[str] = None
    namespace: Optional[str] = None
    ignore_reinit_error: bool = True

    def resolved_init_kwargs(self) -> Dict[str, Any]:
        out = dict(self.init_kwargs)
        out.setdefault("ignore_reinit_error", self.ignore_reinit_error)
        if self.address is not None:
            out.setdefault("address", self.address)
        if self.namespace is not None:
            out.setdefault("namespace", self.namespace)
        return out


@dataclass(frozen=True)
class RayActorOptions:
    name: Optional[str] = None
    num_cpus: Optional[float] = None
    num_gpus: Optional[float] = None
    resources: Mapping[str, float] = field(default_factory=dict)
    namespace: Optional[str] = None
    max_restarts: Optional[int] = None
    max_task_retries: Optional[int] = None
    scheduling_strategy: Any = None
    lifetime: Optional[str] = None
    runtime_env: Optional[Mapping[str, Any]] = None
    extra: Mapping[str, Any] = field(default_factory=dict)

    def to_ray_options(self) -> Dict[str, Any]:
        """Only what was set: Ray's own defaults apply to everything else."""
        out: Dict[str, Any] = dict(self.extra)
        for key in ("name", "namespace", "num_cpus", "num_gpus", "max_restarts", "max_task_retries",
                    "scheduling_strategy", "lifetime"):
            value = getattr(self, key)
            if value is not None:
                out[key] = value
        if self.resources:
            out["resources"] = dict(self.resources)
        if self.runtime_env is not None:
            out["runtime_env"] = dict(self.runtime_env)
        return out


@dataclass(frozen=True)
class RayWorkerSpec:
    worker_factory: Any
    args: Tuple[Any, ...] = ()
    kwargs: Mapping[str, Any] = field(default_factory=dict)
    actor_options: RayActorOptions = field(default_factory=RayActorOptions)


class _RayWorkerActor:
    """Runs inside the actor process: builds the worker and forwards calls to it."""

    def __init__(self, worker_factory: Any, *args: Any, **kwargs: Any) -> None:
        self.worker = worker_factory(*args, **kwargs)

    def _call(self, names: Tuple[str, ...], *args: Any, **kwargs: Any) -> Any:
        for name in names:
            fn = getattr(self.worker, name, None)
            if callable(fn):
                return fn(*args, **kwargs)
        raise AttributeError(f"worker {type(self.worker).__name__} has none of {names}")

    def rollout(self, spec: Any) -> Any:
        return self._call(("rollout", "execute_rollout", "generate_candidates"), spec)

    def train(self, rollout: Any) -> Any:
        return self._call(("train",), rollout)

    def update_weights(self, manifest: Any) -> Any:
        result = self._call(("update_weights",), manifest)
        # the worker's own answer goes back to the driver, except a mapping of imported tensors (what
        # ``RolloutExecutor.update_weights`` returns): shipping the weights through the object store would defeat the
        # bridge, so that becomes a summary
        if isinstance(result, Mapping) and result and all(hasattr(v, "data_ptr") for v in result.values()):
            return {"weight_version": getattr(manifest, "weight_version", None), "tensors": len(result)}
        return result

    def publish_weights(self, weight_version: Optional[int] = None, metadata: Optional[Mapping[str, Any]] = None) -> Any:
        kwargs: Dict[str, Any] = {}
        if weight_version is not None:
            kwargs["weight_version"] = weight_version
        if metadata is not None:
            kwargs["metadata"] = metadata
        return self._call(("publish_weights",), **kwargs)

    def release_weights(self, update_id: Optional[str] = None) -> Any:
        if update_id is None:
            return self._call(("release_weights",))
        return self._call(("release_weights", "release_weight_update"), update_id)

    def health_check(self) -> Mapping[str, Any]:
        fn = getattr(self.worker, "health_check", None)
        extra = dict(fn()) if callable(fn) else {}
        return {"status": "ok", "worker_type": type(self.worker).__name__, **extra}


class _Handle:
    def __init__(self, actor: Any, ray_module: Any) -> None:
        self.actor = actor
        self._ray = ray_module

    def _sync(self, method: str, *args: Any, **kwargs: Any) -> Any:
        return self._ray.get(getattr(self.actor, method).remote(*args, **kwargs))


class RayRolloutWorkerHandle(_Handle):
    def rollout(self, spec: Any) -> Any:
        return self._sync("rollout", spec)

    def update_weights(self, manifest: Any) -> Any:
        return self._sync("update_weights", manifest)

    def release_weights(self) -> Any:
        return self._sync("release_weights")


class RayTrainingWorkerHandle(_Handle):
    def train(self, rollout: Any) -> Any:
        return self._sync("train", rollout)

    def publish_weights(self, weight_version: Optional[int] = None, metadata: Optional[Mapping[str, Any]] = None) -> Any:
        return self._sync("publish_weights", weight_version, metadata)

    def release_weights(self, update_id: str) -> Any:
        return self._sync("release_weights", update_id)


def _load_ray() -> Any:
    try:
        return importlib.import_module("ray")
    except ImportError as exc:
        raise RayUnavailableError(
            "Ray is not installed. Install ray or pass ray_module= to RayActorManager."
        ) from exc


class RayActorManager:
    def __init__(self, runtime_config: Optional[RayRuntimeConfig] = None, *, ray_module: Any = None) -> None:
        self.runtime_config = runtime_config or RayRuntimeConfig()
        self._ray = ray_module
        self._actors: List[Any] = []

    @property
    def runtime(self) -> RayRuntimeConfig:
        return self.runtime_config

    def __enter__(self) -> "RayActorManager":
        self.ensure_runtime()
        return self

    def __exit__(self, exc_type, exc, traceback) -> None:
        self.shutdown()

    def ensure_runtime(self) -> Any:
        if self._ray is None:
            self._ray = _load_ray()
        if self.runtime_config.auto_init:
            is_init = getattr(self._ray, "is_initialized", None)
            if not (callable(is_init) and is_init()):
                self._ray.init(**self.runtime_config.resolved_init_kwargs())
        return self._ray

    def create_worker_actor(self, spec: RayWorkerSpec) -> Any:
        ray = self.ensure_runtime()
        remote_cls = ray.remote(_RayWorkerActor)
        options = spec.actor_options.to_ray_options()
        if options:
            remote_cls = remote_cls.options(**options)
        actor = remote_cls.remote(spec.worker_factory, *spec.args, **dict(spec.kwargs))
        self._actors.append(actor)
        return actor

    def create_rollout_worker(self, spec: RayWorkerSpec) -> RayRolloutWorkerHandle:
        return RayRolloutWorkerHandle(self.create_worker_actor(spec), self._ray)

    def create_training_worker(self, spec: RayWorkerSpec) -> RayTrainingWorkerHandle:
        return RayTrainingWorkerHandle(self.create_worker_actor(spec), self._ray)

    def health_check(self) -> List[Mapping[str, Any]]:
        ray = self.ensure_runtime()
        return [ray.get(actor.health_check.remote()) for actor in self._actors]

    def shutdown(self) -> None:
        if self._ray is None:
            return
        for actor in reversed(self._actors):
            try:
                self._ray.kill(actor, no_restart=True)      # a worker that is shut down must not come back
            except Exception:
                pass
        self._actors.clear()
        if self.runtime_config.shutdown_ray_on_close and hasattr(self._ray, "shutdown"):
            self._ray.shutdown()
