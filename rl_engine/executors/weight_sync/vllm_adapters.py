"""Adapters that install an imported weight update into a rollout engine (vLLM-shaped, duck typed).

None of these import vLLM; they look for capabilities on the engine object they are given, and raise
``WeightBridgeUnavailableError`` with a concrete reason when a capability is missing.  Parity with
``rl_engine/executors/bridge.py:110-747``:

* ``VLLMWeightInstallAdapter``         explicit ``install_callable`` > ``engine.update_weights(request)``
  via a ``request_builder`` > a manifest-aware engine method;
* ``VLLMIPCWeightUpdateRequestBuilder`` builds ``{"update_info": {names, dtype_names, shapes,
  ipc_handles: [{gpu_uuid: handle}], is_checkpoint_format}}`` and keeps the source tensors alive;
* ``VLLMInProcessWeightReloadAdapter``  ``reload_weights(weights_iterator=..., is_checkpoint_format=...)``
  directly or through ``collective_rpc``; optional dtype/device cast;
* ``VLLMCheckpointWeightReloadAdapter`` path based reload (``weights_path`` from argument, resolver or
  ``metadata["vllm_weights_path"]``);
* ``VLLMCUDAVMMExternalStorageAdapter`` rebinds ``parameter.data`` of the worker's model to the aliasing
  tensors of a ``cuda-vmm`` update, with rollback when any parameter does not match.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

import torch

from rl_engine.executors.weight_sync.protocol import (
    BRIDGE_METADATA_KEY, CUDA_IPC_FORMAT, CUDA_VMM_FORMAT, WeightBridgeUnavailableError, WeightLayout,
    WeightManifestValidationError, WeightUpdateManifest,
)


class _ActiveVersion:
    active_weight_version: Optional[int] = None
    active_update_id: Optional[str] = None

    def _activate(self, manifest: WeightUpdateManifest) -> None:
        self.active_weight_version = manifest.weight_version
        self.active_update_id = manifest.update_id

    def _deactivate(self, update_id: str) -> None:
        if self.active_update_id == update_id:
            self.active_update_id = None


def _check_tensor_set(manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor], what: str) -> None:
    if set(tensors) != set(manifest.tensors):
        missing = sorted(set(manifest.tensors) - set(tensors))
        extra = sorted(set(tensors) - set(manifest.tensors))
        raise WeightManifestValidationError(f"{what} tensor set mismatch: missing={missing}, extra={extra}")
    for name, desc in manifest.tensors.items():
        t = tensors[name]
        if tuple(int(d) for d in t.shape) != tuple(desc.shape):
            raise WeightManifestValidationError(
                f"{what} tensor shape mismatch for {name}: expected {desc.shape}, got {tuple(t.shape)}"
            )
        if str(t.dtype) != desc.dtype:
            raise WeightManifestValidationError(
                f"{what} tensor dtype mismatch for {name}: expected {desc.dtype}, got {t.dtype}"
            )


class VLLMWeightInstallAdapter(_ActiveVersion):
    _MANIFEST_METHODS = ("install_weight_update", "update_weights_from_manifest", "load_weights_from_manifest")

    def __init__(self, engine: Any, *, install_callable=None, request_builder=None, release_callable=None) -> None:
        self.engine = engine
        self._install_callable = install_callable
        self._request_builder = request_builder
        self._release_callable = release_callable

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        tensors = dict(tensors)
        if self._install_callable is not None:
            self._install_callable(manifest, tensors)
        elif callable(getattr(self.engine, "update_weights", None)):
            if self._request_builder is None:
                raise WeightBridgeUnavailableError(
                    "vLLM weight install requires a request_builder for engines that expose "
                    "update_weights(request). vLLM does not accept a raw manifest/tensor mapping for this public API."
                )
            try:
                self.engine.update_weights(self._request_builder(manifest, tensors))
            except Exception:
                release = getattr(self._request_builder, "release", None)
                if callable(release):
                    release(manifest.update_id)
                raise
        else:
            for attr in self._MANIFEST_METHODS:
                method = getattr(self.engine, attr, None)
                if callable(method):
                    method(manifest, tensors)
                    break
            else:
                raise WeightBridgeUnavailableError(
                    "vLLM weight install is unavailable because this engine does not expose a verified "
                    "hot-weight install capability. Pass an explicit install_callable for the installed vLLM version."
                )
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        if self._release_callable is not None:
            self._release_callable(update_id)
        release = getattr(self._request_builder, "release", None)
        if callable(release):
            release(update_id)
        self._deactivate(update_id)


class VLLMIPCWeightUpdateRequestBuilder:
    def __init__(self, *, is_checkpoint_format: bool = True, reduce_tensor=None, gpu_uuid_resolver=None) -> None:
        self.is_checkpoint_format = bool(is_checkpoint_format)
        self._reduce_tensor = reduce_tensor
        self._gpu_uuid_resolver = gpu_uuid_resolver
        self._keepalive: Dict[str, List[Any]] = {}

    def __call__(self, manifest: WeightUpdateManifest, tensors: Mapping[str, Any]) -> Dict[str, Any]:
        if set(tensors) != set(manifest.tensors):
            raise WeightManifestValidationError("vLLM IPC request tensor set does not match the manifest")
        from_manifest = self._manifest_handles(manifest)
        uuid = self._manifest_uuid(manifest) if from_manifest is not None else None
        names, dtype_names, shapes, handles, alive = [], [], [], [], []
        for name, desc in manifest.tensors.items():
            t = tensors[name]
            device = getattr(t, "device", None)
            if getattr(device, "type", "cuda") != "cuda" and not getattr(t, "is_cuda", False):
                raise WeightBridgeUnavailableError(
                    f"vLLM IPC weight updates need CUDA tensors; {name} is on {device}"
                )
            if tuple(int(d) for d in t.shape) != tuple(desc.shape):
                raise WeightManifestValidationError(f"vLLM IPC tensor shape mismatch for {name}")
            if str(t.dtype) != desc.dtype:
                raise WeightManifestValidationError(f"vLLM IPC tensor dtype mismatch for {name}")
            if from_manifest is not None:
                handle = from_manifest[name]
            else:
                src = t.detach().contiguous() if hasattr(t, "detach") else t
                alive.append(src)
                handle = self._reduce()(src)
                uuid = uuid or self._uuid()
            names.append(name)
            dtype_names.append(desc.dtype.replace("torch.", ""))
            shapes.append(list(desc.shape))
            handles.append({uuid: handle})
        self._keepalive[manifest.update_id] = alive
        return {"update_info": {"names": names, "dtype_names": dtype_names, "shapes": shapes, "ipc_handles": handles,
                                "is_checkpoint_format": self.is_checkpoint_format}}

    def release(self, update_id: str) -> None:
        self._keepalive.pop(update_id, None)

    @staticmethod
    def _manifest_handles(manifest: WeightUpdateManifest) -> Optional[Dict[str, Any]]:
        block = manifest.metadata.get(BRIDGE_METADATA_KEY)
        if not isinstance(block, Mapping) or block.get("format") != CUDA_IPC_FORMAT:
            return None
        entries = block.get("tensors", {})
        if set(entries) != set(manifest.tensors):
            raise WeightManifestValidationError("vLLM IPC manifest handle mismatch")
        out = {}
        for name, entry in entries.items():
            if not isinstance(entry, Mapping) or "handle" not in entry:
                raise WeightManifestValidationError(f"vLLM IPC manifest has no handle for {name}")
            out[name] = entry["handle"]
        return out

    @staticmethod
    def _manifest_uuid(manifest: WeightUpdateManifest) -> Optional[str]:
        block = manifest.metadata.get(BRIDGE_METADATA_KEY)
        return None if not isinstance(block, Mapping) else block.get("gpu_uuid")

    def _reduce(self):
        if self._reduce_tensor is not None:
            return self._reduce_tensor
        try:
            from torch.multiprocessing.reductions import reduce_tensor
        except Exception as exc:  # pragma: no cover
            raise WeightBridgeUnavailableError(f"torch reduce_tensor is unavailable: {exc}") from exc
        return reduce_tensor

    def _uuid(self) -> str:
        if self._gpu_uuid_resolver is not None:
            return str(self._gpu_uuid_resolver())
        if not torch.cuda.is_available():
            raise WeightBridgeUnavailableError("cannot resolve a GPU UUID without CUDA")
        return str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)


def _resolve_reload(engine: Any, make_kwargs: Callable[[Any], Dict[str, Any]], what: str):
    direct = getattr(engine, "reload_weights", None)
    if callable(direct):
        return lambda payload: direct(**make_kwargs(payload))
    rpc = getattr(engine, "collective_rpc", None)
    if not callable(rpc):
        rpc = getattr(getattr(engine, "llm_engine", None), "collective_rpc", None)
    if callable(rpc):
        return lambda payload: rpc("reload_weights", kwargs=make_kwargs(payload))
    raise WeightBridgeUnavailableError(
        f"vLLM {what} weight reload is unavailable because this engine does not expose "
        "reload_weights(...) or llm_engine.collective_rpc(...)."
    )


class VLLMInProcessWeightReloadAdapter(_ActiveVersion):
    def __init__(self, engine: Any, *, target_dtype: Optional[torch.dtype] = None, target_device=None,
                 is_checkpoint_format: bool = True, synchronize_cuda: bool = True) -> None:
        self.engine = engine
        self.target_dtype, self.target_device = target_dtype, target_device
        self.is_checkpoint_format, self.synchronize_cuda = bool(is_checkpoint_format), bool(synchronize_cuda)

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        tensors = dict(tensors)
        _check_tensor_set(manifest, tensors, "vLLM reload")
        weights: List[Tuple[str, torch.Tensor]] = []
        for name in manifest.tensors:
            w = tensors[name].detach()
            if self.target_dtype is not None and w.dtype != self.target_dtype:
                w = w.to(self.target_dtype)
            if self.target_device is not None and torch.device(self.target_device) != w.device:
                w = w.to(self.target_device)
            weights.append((name, w.contiguous()))
        try:
            reload_fn = _resolve_reload(
                self.engine, lambda p: {"weights_iterator": p, "is_checkpoint_format": self.is_checkpoint_format},
                "in-process",
            )
            reload_fn(weights)
            if self.synchronize_cuda and torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            self.active_update_id = None
            raise
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        self._deactivate(update_id)


class VLLMCheckpointWeightReloadAdapter(_ActiveVersion):
    def __init__(self, engine: Any, *, weights_path: Optional[str] = None, weights_path_resolver=None,
                 is_checkpoint_format: bool = True) -> None:
        self.engine = engine
        self._weights_path, self._resolver = weights_path, weights_path_resolver
        self.is_checkpoint_format = bool(is_checkpoint_format)

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        if set(tensors) != set(manifest.tensors):
            raise WeightManifestValidationError("vLLM checkpoint reload tensor set does not match the manifest")
        path = self._path_for(manifest)
        try:
            reload_fn = _resolve_reload(
                self.engine, lambda p: {"weights_path": p, "is_checkpoint_format": self.is_checkpoint_format},
                "checkpoint",
            )
            reload_fn(path)
        except Exception:
            self.active_update_id = None
            raise
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        self._deactivate(update_id)

    def _path_for(self, manifest: WeightUpdateManifest) -> str:
        if self._weights_path:
            return str(self._weights_path)
        if self._resolver is not None:
            found = self._resolver(manifest)
            if found:
                return str(found)
        from_meta = manifest.metadata.get("vllm_weights_path")
        if from_meta:
            return str(from_meta)
        raise WeightBridgeUnavailableError(
            "vLLM checkpoint reload needs a weights_path (argument, resolver, or metadata['vllm_weights_path'])."
        )


def rebind_parameters(model: torch.nn.Module, aliases: Mapping[str, torch.Tensor]) -> Dict[str, Any]:
    """Point ``parameter.data`` at the aliasing tensors; undo everything if one entry does not fit."""
    params = dict(model.named_parameters())
    undo: List[Tuple[torch.nn.Parameter, torch.Tensor]] = []
    try:
        for name, alias in aliases.items():
            if name not in params:
                raise WeightManifestValidationError(f"model has no parameter named {name}")
            p = params[name]
            if tuple(p.shape) != tuple(alias.shape) or p.dtype != alias.dtype:
                raise WeightManifestValidationError(
                    f"parameter {name} mismatch: model {tuple(p.shape)}/{p.dtype}, update {tuple(alias.shape)}/{alias.dtype}"
                )
            undo.append((p, p.data))
            p.data = alias
    except Exception:
        for p, old in reversed(undo):
            p.data = old
        raise
    return {"rebound": len(undo), "originals": undo}


class VLLMCUDAVMMExternalStorageAdapter(_ActiveVersion):
    def __init__(self, engine: Any, *, bridge_factory=None, apply_model: Optional[Callable] = None) -> None:
        self.engine = engine
        self._bridge_factory = bridge_factory
        self._apply_model = apply_model
        self._originals: Dict[str, Any] = {}

    def _apply(self) -> Callable[[Callable], Any]:
        if self._apply_model is not None:
            return self._apply_model
        for owner in (self.engine, getattr(self.engine, "llm_engine", None)):
            fn = getattr(owner, "apply_model", None)
            if callable(fn):
                return fn
        raise WeightBridgeUnavailableError(
            "vLLM external-storage install needs engine.apply_model(fn) (or an explicit apply_model=)."
        )

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        block = manifest.metadata.get(BRIDGE_METADATA_KEY)
        if not isinstance(block, Mapping) or block.get("format") != CUDA_VMM_FORMAT:
            raise WeightBridgeUnavailableError("external-storage install needs a cuda-vmm weight update")
        if set(tensors) != set(manifest.tensors):
            raise WeightManifestValidationError("external-storage tensor set does not match the manifest")
        aliases = dict(tensors)

        def on_worker(model: torch.nn.Module) -> Dict[str, Any]:
            local = aliases
            if self._bridge_factory is not None:  # worker in another process: map the update there
                local = dict(self._bridge_factory().import_update(manifest))
            result = rebind_parameters(model, local)
            self._originals[manifest.update_id] = result.pop("originals")
            return result

        self._apply()(on_worker)
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        originals = self._originals.pop(update_id, None)
        if originals:
            def restore(_model: torch.nn.Module) -> Dict[str, Any]:
                for p, old in reversed(originals):
                    p.data = old
                return {"restored": len(originals)}

            self._apply()(restore)
        self._deactivate(update_id)
