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

import importlib

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
    def __init__(self, *, is_checkpoint_format: bool = True, reduce_tensor=None, gpu_uuid_resolver=None,
                 reduce_tensor_fn=None, gpu_uuid: Optional[str] = None) -> None:
        """``reduce_tensor`` / ``reduce_tensor_fn`` (the reference's spelling): the function that turns a CUDA tensor into
        an IPC handle (default: torch's ``reduce_tensor``).  ``gpu_uuid``: a fixed UUID for the handle table;
        ``gpu_uuid_resolver``: a callable asked when one is needed (default: the current device's)."""
        self.is_checkpoint_format = bool(is_checkpoint_format)
        self._reduce_tensor = reduce_tensor if reduce_tensor is not None else reduce_tensor_fn
        self._gpu_uuid_resolver = gpu_uuid_resolver if gpu_uuid_resolver is not None else (
            None if gpu_uuid is None else (lambda: gpu_uuid))
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
                    f"vLLM IPC weight update requires CUDA tensors; {name} is on {device}"
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
                 metadata_key: str = "vllm_weights_path", is_checkpoint_format: bool = True,
                 synchronize_cuda: bool = True) -> None:
        """The path comes from ``weights_path``, else ``weights_path_resolver(manifest)``, else
        ``manifest.metadata[metadata_key]``."""
        self.engine = engine
        self._weights_path, self._resolver = weights_path, weights_path_resolver
        self.metadata_key = metadata_key
        self.is_checkpoint_format, self.synchronize_cuda = bool(is_checkpoint_format), bool(synchronize_cuda)

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        if set(tensors) != set(manifest.tensors):
            raise WeightManifestValidationError("vLLM checkpoint reload tensor set does not match the manifest")
        path = self._path_for(manifest, tensors)
        try:
            reload_fn = _resolve_reload(
                self.engine, lambda p: {"weights_path": p, "is_checkpoint_format": self.is_checkpoint_format},
                "checkpoint",
            )
            reload_fn(path)
            if self.synchronize_cuda and torch.cuda.is_available():
                torch.cuda.synchronize()
        except Exception:
            self.active_update_id = None
            raise
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        self._deactivate(update_id)

    def _path_for(self, manifest: WeightUpdateManifest, tensors: Optional[Mapping[str, torch.Tensor]] = None) -> str:
        if self._weights_path:
            return str(self._weights_path)
        if self._resolver is not None:
            try:
                found = self._resolver(manifest, tensors)        # the reference's resolvers take (manifest, tensors)
            except TypeError:
                found = self._resolver(manifest)
            if found:
                return str(found)
        from_meta = manifest.metadata.get(self.metadata_key)
        if from_meta:
            return str(from_meta)
        raise WeightBridgeUnavailableError(
            f"vLLM checkpoint reload needs a weights_path (argument, resolver, or metadata[{self.metadata_key!r}])."
        )


def rebind_parameters(model: torch.nn.Module, aliases: Mapping[str, torch.Tensor], *, skip_unknown: bool = False,
                      originals: Optional[Dict[str, torch.Tensor]] = None) -> List[str]:
    """Point ``parameter.data`` of every parameter named in ``aliases`` at the aliasing tensor and return the names
    that were rebound; undo all of them if one entry does not fit.  ``originals`` collects the storage each parameter
    had before its FIRST rebinding.  Names the model does not have are an error unless ``skip_unknown``."""
    params = dict(model.named_parameters())
    originals = {} if originals is None else originals
    done: List[Tuple[str, torch.Tensor, bool]] = []     # (name, data before this call, first rebinding?)
    try:
        for name, alias in aliases.items():
            p = params.get(name)
            if p is None:
                if skip_unknown:
                    continue
                raise WeightManifestValidationError(f"model has no parameter named {name}")
            if tuple(p.shape) != tuple(alias.shape):
                raise WeightManifestValidationError(
                    f"parameter shape mismatch for {name}: model {tuple(p.shape)}, update {tuple(alias.shape)}")
            if p.dtype != alias.dtype:
                raise WeightManifestValidationError(
                    f"parameter dtype mismatch for {name}: model {p.dtype}, update {alias.dtype}")
            first = name not in originals
            done.append((name, p.data, first))
            originals.setdefault(name, p.data)
            p.data = alias
    except Exception:
        for name, before, first in reversed(done):
            params[name].data = before
            if first:
                originals.pop(name, None)
        raise
    return [name for name, _before, _first in done]


class _WorkerBinding:
    """What lives beside the model inside the worker process while its parameters alias an imported update: the
    consumer bridge that keeps the mapping alive, the update's tensors and the storage to go back to."""

    ATTRIBUTE = "_rl_engine_vmm_binding"

    def __init__(self) -> None:
        self.bridge: Any = None
        self.update_id: Optional[str] = None
        self.tensors: Dict[str, torch.Tensor] = {}
        self.originals: Dict[str, torch.Tensor] = {}


class VLLMCUDAVMMExternalStorageAdapter(_ActiveVersion):
    """Zero-copy install of a ``cuda-vmm`` update into vLLM workers (reference: ``rl_engine/executors/bridge.py:543-747``).

    The function handed to ``engine.apply_model`` runs INSIDE every worker: it builds a consumer
    ``CUDAVMMTensorBridge`` there, imports the manifest (mapping the publisher's allocation through the POSIX fd),
    points the ``.data`` of every parameter whose name is in the update at the imported tensor, and acknowledges.  A
    tensor that does not fit undoes the worker's rebinding and releases the import.  ``release`` goes the same way
    back.  ``require_all_parameters``: every tensor of the manifest must have been bound on some worker.

    ``bridge_factory`` (tests, other transports) replaces the construction of the consumer bridge; ``apply_model``
    replaces ``engine.apply_model`` / ``engine.llm_engine.apply_model``."""

    def __init__(self, engine: Any, *, device_index: int = 0, source_worker: str = "vllm-rollout", source_rank: int = 0,
                 require_all_parameters: bool = False, synchronize_cuda: bool = True, bridge_factory=None,
                 apply_model: Optional[Callable] = None) -> None:
        self.engine = engine
        self.device_index, self.source_worker, self.source_rank = int(device_index), source_worker, int(source_rank)
        self.require_all_parameters, self.synchronize_cuda = bool(require_all_parameters), bool(synchronize_cuda)
        self._bridge_factory = bridge_factory
        self._apply_model = apply_model
        self.last_result: List[Dict[str, Any]] = []

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

    def _consumer_bridge(self) -> Any:
        if self._bridge_factory is not None:
            return self._bridge_factory()
        # looked up through the public module at call time, inside the worker
        bridge_module = importlib.import_module("rl_engine.executors.bridge")
        return bridge_module.CUDAVMMTensorBridge(source_worker=self.source_worker, source_rank=self.source_rank,
                                                 device_index=self.device_index)

    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None:
        del tensors                       # the workers import the update themselves
        WeightLayout.from_metadata(manifest.metadata).validate_supported()
        if manifest.transport != "cuda-vmm":
            raise WeightBridgeUnavailableError(
                f"external-storage install needs a cuda-vmm weight update, got transport {manifest.transport!r}")
        apply = self._apply()
        synchronize = self.synchronize_cuda

        def bind(model: torch.nn.Module) -> Dict[str, Any]:
            binding = getattr(model, _WorkerBinding.ATTRIBUTE, None) or _WorkerBinding()
            bridge = self._consumer_bridge()
            imported = dict(bridge.import_update(manifest))
            try:
                with torch.no_grad():
                    rebound = rebind_parameters(model, imported, skip_unknown=True, originals=binding.originals)
                bridge.acknowledge(manifest.update_id)
            except Exception:
                imported.clear()
                bridge.release(manifest.update_id)
                raise
            if synchronize and torch.cuda.is_available():
                torch.cuda.synchronize()
            binding.bridge, binding.update_id, binding.tensors = bridge, manifest.update_id, imported
            setattr(model, _WorkerBinding.ATTRIBUTE, binding)
            return {"update_id": manifest.update_id, "weight_version": manifest.weight_version, "rebound": rebound,
                    "tensor_count": len(imported), "zero_copy": True}

        results = apply(bind)
        results = [dict(r or {}) for r in (results if isinstance(results, list) else [results])]
        bound = set().union(*(set(r.get("rebound", [])) for r in results)) if results else set()
        missing = sorted(set(manifest.tensors) - bound)
        if self.require_all_parameters and missing:
            self.release(manifest.update_id)
            raise WeightManifestValidationError(f"vLLM CUDA VMM install did not bind every manifest tensor: missing={missing}")
        self.last_result = results
        self._activate(manifest)

    def release(self, update_id: str) -> None:
        def unbind(model: torch.nn.Module) -> Dict[str, Any]:
            binding = getattr(model, _WorkerBinding.ATTRIBUTE, None)
            if binding is None or binding.update_id != update_id:
                return {"released": False, "update_id": update_id}
            params = dict(model.named_parameters())
            with torch.no_grad():
                for name, original in binding.originals.items():
                    if name in params:
                        params[name].data = original
            binding.tensors.clear()
            try:
                binding.bridge.release(update_id)
            finally:
                delattr(model, _WorkerBinding.ATTRIBUTE)
            return {"released": True, "update_id": update_id}

        self._apply()(unbind)
        self._deactivate(update_id)
