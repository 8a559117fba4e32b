"""Manifest schema and the update life cycle shared by every weight transport.

Parity (field names, format tags, error types and state machine) with the reference bridge:
``rl_engine/executors/bridge.py:32-107`` (``WeightLayout``), ``:1335-1441`` (errors, descriptors,
manifest, protocols) and ``:1508-1693`` (publish -> import -> acknowledge / reject / release, with
monotonic versions and "the previous version stays active until the new one is acknowledged").

Differences that matter at B200 scale:

* the integrity digest of a CUDA tensor is computed ON THE DEVICE (a 64-bit position-weighted
  checksum, stored in the same ``sha256`` field with a ``dev64:`` prefix) instead of hashing a
  device-to-host copy three times per update -- a 16 GB update would otherwise be host bound.
  ``RL_KERNEL_WEIGHT_DIGEST=sha256`` restores byte-exact SHA-256 everywhere, ``none`` disables it;
* tensor-parallel and multi-rank layouts are legal for the ``nvlink-broadcast`` transport.
"""

from __future__ import annotations

import hashlib
import os
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Protocol

import torch

from rl_engine.utils.logger import logger

BRIDGE_METADATA_KEY = "weight_bridge"
SHARED_MEMORY_FORMAT = "python-multiprocessing-shared-memory-v1"
CUDA_IPC_FORMAT = "pytorch-cuda-ipc-reduce-tensor-v1"
CUDA_VMM_FORMAT = "cuda-vmm-posix-fd-v1"
NVLINK_BROADCAST_FORMAT = "nvlink-symmetric-broadcast-v1"
FILE_BLOB_FORMAT = "packed-blob-file-v1"
TENSOR_ALIGNMENT = 256
SUPPORTED_LAYOUT_KINDS = {"full-state", "replicated"}


class WeightBridgeError(RuntimeError):
    """Base class for weight synchronisation failures."""


class WeightBridgeUnavailableError(WeightBridgeError):
    """The requested transport or layout is not supported by this runtime."""


class WeightManifestValidationError(WeightBridgeError):
    """A manifest is incomplete, inconsistent or does not match the stored update."""


class WeightUpdateRejectedError(WeightBridgeError):
    """An update cannot be imported or acknowledged (unknown, rejected or released)."""


@dataclass(frozen=True)
class WeightLayout:
    kind: str = "full-state"
    world_size: int = 1
    rank: int = 0
    tensor_parallel_size: int = 1
    data_parallel_size: int = 1
    zero_stage: int = 0
    node_count: int = 1
    rdma_enabled: bool = False

    _FIELDS = ("kind", "world_size", "rank", "tensor_parallel_size", "data_parallel_size", "zero_stage", "node_count",
               "rdma_enabled")

    @classmethod
    def from_metadata(cls, metadata: Optional[Mapping[str, Any]]) -> "WeightLayout":
        raw = None if metadata is None else metadata.get("layout", {})
        if raw is None or raw == {}:
            return cls()
        if not isinstance(raw, Mapping):
            raise WeightManifestValidationError("weight layout metadata must be a mapping")
        default = cls()
        values = {}
        for name in cls._FIELDS:
            caster = type(getattr(default, name))
            values[name] = caster(raw.get(name, getattr(default, name)))
        return cls(**values)

    def to_metadata(self) -> Dict[str, Any]:
        return {name: getattr(self, name) for name in self._FIELDS}

    def validate_supported(self, *, allow_multi_rank: bool = False) -> None:
        if self.kind not in SUPPORTED_LAYOUT_KINDS:
            raise WeightBridgeUnavailableError(
                f"weight layout {self.kind!r} is not supported by this bridge. Publish a gathered "
                "full-state update or implement a layout-aware transport before exposing it to rollout workers."
            )
        if self.tensor_parallel_size != 1 and not allow_multi_rank:
            raise WeightBridgeUnavailableError(
                "tensor-parallel weight layouts are not supported by this bridge. Publish a complete "
                "per-consumer layout or use the nvlink-broadcast transport."
            )
        if self.node_count != 1 or self.rdma_enabled:
            raise WeightBridgeUnavailableError(
                "multi-node/RDMA weight transport is not implemented. Use a same-node transport."
            )
        if self.world_size < 1 or not 0 <= self.rank < self.world_size:
            raise WeightManifestValidationError(
                f"invalid weight layout rank/world_size: rank={self.rank}, world_size={self.world_size}"
            )
        if self.data_parallel_size < 1:
            raise WeightManifestValidationError("data_parallel_size must be >= 1")


def digest_policy() -> str:
    return os.environ.get("RL_KERNEL_WEIGHT_DIGEST", "auto").strip().lower()


_DIGEST_MUL = -7046029254386353131  # 0x9E3779B97F4A7C15 as a signed 64-bit value


def _dev64_reference(t: torch.Tensor) -> int:
    """The ``dev64`` digest with plain tensor ops (any device): sum over the tensor's 64-bit words ``w_i`` (tail
    zero-padded) of ``(w_i ^ (w_i >> 29)) * ((i + 1) * C)`` modulo 2^64.  The fused kernel computes the same bits in
    one pass; this form is the fallback for unaligned views and the oracle of the kernel's test."""
    flat = t.contiguous().view(-1).view(torch.uint8)
    pad = (-flat.numel()) % 8
    if pad:
        flat = torch.cat([flat, flat.new_zeros(pad)])
    words = flat.view(torch.int64)
    total = 0
    step = 1 << 24  # bounded temporaries: the weights of 16 M words at a time
    for i0 in range(0, words.numel(), step):
        w = words[i0 : i0 + step]
        weights = torch.arange(i0 + 1, i0 + w.numel() + 1, device=w.device, dtype=torch.int64) * _DIGEST_MUL
        total += int(((w ^ (w >> 29)) * weights).sum().item())
    return total & 0xFFFFFFFFFFFFFFFF


_DIGEST_UNIT_WORDS = 1 << 15  # 64-bit words per work unit of the table-driven digest kernel


_DIGEST_KERNEL: Optional[bool] = None  # whether the extension with the digest kernel is loaded (looked up once)


def _kernel_digest_ok(t: torch.Tensor) -> bool:
    global _DIGEST_KERNEL
    if not t.is_cuda or t.numel() == 0 or not t.is_contiguous() or t.data_ptr() % 16:
        return False
    if _DIGEST_KERNEL is None:
        from rl_engine.kernels.ops.base import _C, _EXT_AVAILABLE

        _DIGEST_KERNEL = bool(_EXT_AVAILABLE and hasattr(_C, "weight_digest"))
    return _DIGEST_KERNEL


def tensor_digests(tensors: Mapping[str, torch.Tensor]) -> Dict[str, str]:
    """Integrity digests of many tensors (the ``TensorDescriptor.sha256`` field; see the module docstring).  The CUDA
    tensors of a device are digested by ONE kernel launch over a table of (address, size) rows into a shared result
    buffer that is read back once, so a model state of hundreds of tensors costs one launch and one host
    synchronisation, not one of each per tensor (291 tensors, 16 GB: 17 ms with a launch per tensor)."""
    policy = digest_policy()
    out: Dict[str, str] = {}
    if policy == "none":
        return {name: "none" for name in tensors}
    batched: Dict[torch.device, list] = {}
    for name, tensor in tensors.items():
        t = tensor.detach()
        if t.is_cuda and policy != "sha256":
            nbytes = t.numel() * t.element_size()
            if _kernel_digest_ok(t):
                batched.setdefault(t.device, []).append((name, t, nbytes))
            else:
                c = t.contiguous()
                if c.numel() and _kernel_digest_ok(c):
                    batched.setdefault(c.device, []).append((name, c, nbytes))
                else:
                    out[name] = f"dev64:{_dev64_reference(t):016x}:{(nbytes + 7) // 8 * 8}"
            continue
        data = t.contiguous().cpu()
        raw = data.view(torch.uint8).numpy().tobytes() if data.numel() else b""
        out[name] = hashlib.sha256(raw).hexdigest()
    for device, items in batched.items():
        from rl_engine.kernels.ops.base import require_ext

        ext = require_ext()
        results = torch.zeros(len(items), dtype=torch.int64, device=device)
        if hasattr(ext, "digest_segments"):
            rows, units = [], 0
            for slot, (_name, t, nbytes) in enumerate(items):
                rows.append((t.data_ptr(), slot, nbytes, units))
                units += max(1, (nbytes // 8 + _DIGEST_UNIT_WORDS - 1) // _DIGEST_UNIT_WORDS)
            ext.digest_segments(torch.tensor(rows, dtype=torch.int64).to(device), units, results)
        else:
            for slot, (_name, t, _n) in enumerate(items):
                ext.weight_digest(t, results, slot)
        for (name, _t, nbytes), value in zip(items, results.cpu().tolist()):
            out[name] = f"dev64:{value & 0xFFFFFFFFFFFFFFFF:016x}:{(nbytes + 7) // 8 * 8}"
    return out


def tensor_digest(tensor: torch.Tensor) -> str:
    """Integrity digest stored in ``TensorDescriptor.sha256`` (see the module docstring)."""
    return tensor_digests({"t": tensor})["t"]


@dataclass(frozen=True)
class TensorDescriptor:
    name: str
    shape: tuple
    dtype: str
    stride: tuple
    device: str
    numel: int
    nbytes: int
    sha256: str

    @classmethod
    def from_tensors(cls, tensors: Mapping[str, torch.Tensor]) -> Dict[str, "TensorDescriptor"]:
        """Descriptors of a whole state; the digests are computed in one batch (see ``tensor_digests``)."""
        digests = tensor_digests(tensors)
        return {name: cls.from_tensor(name, t, digest=digests[name]) for name, t in tensors.items()}

    @classmethod
    def from_tensor(cls, name: str, tensor: torch.Tensor, digest: Optional[str] = None) -> "TensorDescriptor":
        return cls(
            name=name,
            shape=tuple(int(d) for d in tensor.shape),
            dtype=str(tensor.dtype),
            stride=tuple(int(s) for s in tensor.stride()),
            device=str(tensor.device),
            numel=int(tensor.numel()),
            nbytes=int(tensor.numel() * tensor.element_size()),
            sha256=tensor_digest(tensor) if digest is None else digest,
        )

    def to_json(self) -> Dict[str, Any]:
        return {"name": self.name, "shape": list(self.shape), "dtype": self.dtype, "stride": list(self.stride),
                "device": self.device, "numel": self.numel, "nbytes": self.nbytes, "sha256": self.sha256}

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "TensorDescriptor":
        return cls(str(raw["name"]), tuple(raw["shape"]), str(raw["dtype"]), tuple(raw["stride"]), str(raw["device"]),
                   int(raw["numel"]), int(raw["nbytes"]), str(raw["sha256"]))


@dataclass(frozen=True)
class WeightUpdateManifest:
    update_id: str
    source_worker: str
    source_rank: int
    weight_version: int
    transport: str
    tensors: Mapping[str, TensorDescriptor]
    created_at: float
    metadata: Mapping[str, Any] = field(default_factory=dict)

    @property
    def tensor_count(self) -> int:
        return len(self.tensors)

    @property
    def total_nbytes(self) -> int:
        return sum(d.nbytes for d in self.tensors.values())


class WeightPublisher(Protocol):
    def publish(self, model: torch.nn.Module, *, weight_version: int,
                metadata: Optional[Mapping[str, Any]] = None) -> WeightUpdateManifest: ...

    def release(self, update_id: str) -> None: ...


class WeightConsumer(Protocol):
    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]: ...

    def acknowledge(self, update_id: str) -> None: ...

    def reject(self, update_id: str, reason: str) -> None: ...

    def release(self, update_id: str) -> None: ...


class WeightBridge(WeightPublisher, WeightConsumer, Protocol):
    pass


class WeightInstallAdapter(Protocol):
    def install(self, manifest: WeightUpdateManifest, tensors: Mapping[str, torch.Tensor]) -> None: ...

    def release(self, update_id: str) -> None: ...


def validated_metadata(metadata: Optional[Mapping[str, Any]], *, allow_multi_rank: bool = False) -> Dict[str, Any]:
    out = dict(metadata or {})
    layout = WeightLayout.from_metadata(out)
    layout.validate_supported(allow_multi_rank=allow_multi_rank)
    out["layout"] = layout.to_metadata()
    return out


def state_dict_tensors(model: Any) -> Dict[str, torch.Tensor]:
    """Checkpoint-format names -> tensors from a module, a mapping, or anything with ``state_dict()``."""
    source = model.state_dict() if hasattr(model, "state_dict") else model
    if not isinstance(source, Mapping):
        raise WeightManifestValidationError("publish() needs a module or a mapping of tensors")
    return {str(k): v for k, v in source.items() if isinstance(v, torch.Tensor)}


@dataclass
class UpdateRecord:
    manifest: WeightUpdateManifest
    tensors: Dict[str, torch.Tensor]
    state: str = "published"  # published -> imported -> acknowledged | rejected | released
    import_count: int = 0
    rejection_reason: Optional[str] = None
    resources: Dict[str, Any] = field(default_factory=dict)


class BridgeStateMachine:
    """Life cycle common to all transports; subclasses provide capture / hand-out / dispose."""

    transport = "abstract"
    allow_multi_rank = False
    writes_transport_block = True       # transports that put their own block under ``metadata["weight_bridge"]``

    def __init__(self, *, source_worker: str = "local-training", source_rank: int = 0) -> None:
        self.source_worker = source_worker
        self.source_rank = int(source_rank)
        self._updates: Dict[str, UpdateRecord] = {}
        self._latest_published_weight_version = -1
        self.active_weight_version: Optional[int] = None
        self.active_update_id: Optional[str] = None

    # -- transport hooks ---------------------------------------------------------------------
    def _capture(self, tensors: Dict[str, torch.Tensor], update_id: str):
        """-> (stored tensors, transport metadata block or None, resources)."""
        raise NotImplementedError

    def _hand_out(self, record: UpdateRecord) -> Dict[str, torch.Tensor]:
        raise NotImplementedError

    def _attach(self, manifest: WeightUpdateManifest) -> UpdateRecord:
        """Consumer side in another process: build a record from the manifest alone."""
        raise WeightUpdateRejectedError(f"unknown weight update {manifest.update_id}")

    def _dispose(self, record: UpdateRecord) -> None:
        record.tensors.clear()

    # -- publisher -----------------------------------------------------------------------------
    def publish(self, model: Any, *, weight_version: int, metadata: Optional[Mapping[str, Any]] = None):
        if metadata is not None and BRIDGE_METADATA_KEY in metadata and self.writes_transport_block:
            raise WeightManifestValidationError(
                f"metadata key {BRIDGE_METADATA_KEY!r} is reserved for the transport's own description of the update")
        meta = validated_metadata(metadata, allow_multi_rank=self.allow_multi_rank)
        version = int(weight_version)
        if version <= self._latest_published_weight_version:
            raise WeightManifestValidationError(
                "weight_version must increase monotonically "
                f"(got {version}, latest {self._latest_published_weight_version})"
            )
        source = state_dict_tensors(model)
        if not source:
            raise WeightManifestValidationError("model state_dict produced no tensors")
        update_id = str(uuid.uuid4())
        stored, block, resources = self._capture(source, update_id)
        if block is not None:
            meta[BRIDGE_METADATA_KEY] = block
        manifest = WeightUpdateManifest(
            update_id=update_id, source_worker=self.source_worker, source_rank=self.source_rank, weight_version=version,
            transport=self.transport, tensors=TensorDescriptor.from_tensors(stored),
            created_at=time.perf_counter(), metadata=meta,
        )
        self._updates[update_id] = UpdateRecord(manifest=manifest, tensors=stored, resources=resources)
        self._latest_published_weight_version = version
        logger.info("Published weight update %s version=%s tensors=%s bytes=%s", update_id, version,
                    manifest.tensor_count, manifest.total_nbytes)
        return manifest

    # -- consumer ------------------------------------------------------------------------------
    def import_update(self, manifest: WeightUpdateManifest) -> Mapping[str, torch.Tensor]:
        record = self._updates.get(manifest.update_id)
        if record is None:
            record = self._attach(manifest)
            self._updates[manifest.update_id] = record
        if record.state == "rejected":
            raise WeightUpdateRejectedError(
                f"weight update {manifest.update_id} was rejected: {record.rejection_reason}"
            )
        if record.state == "released":
            raise WeightUpdateRejectedError(f"weight update {manifest.update_id} was released")
        self._validate(record, manifest)
        record.import_count += 1
        if record.state == "published":
            record.state = "imported"
        return self._hand_out(record)

    def acknowledge(self, update_id: str) -> None:
        record = self._require(update_id)
        if record.state == "rejected":
            raise WeightUpdateRejectedError(
                f"cannot acknowledge rejected update {update_id}: {record.rejection_reason}"
            )
        if record.state == "released":
            raise WeightUpdateRejectedError(f"cannot acknowledge released update {update_id}")
        if record.import_count == 0:
            raise WeightUpdateRejectedError(f"cannot acknowledge update {update_id} before import_update succeeds")
        self._validate(record, record.manifest)
        record.state = "acknowledged"
        self.active_weight_version = record.manifest.weight_version
        self.active_update_id = update_id

    def reject(self, update_id: str, reason: str) -> None:
        record = self._require(update_id)
        if record.state == "acknowledged":
            raise WeightUpdateRejectedError(f"cannot reject acknowledged update {update_id}")
        record.state = "rejected"
        record.rejection_reason = reason

    def release(self, update_id: str) -> None:
        record = self._updates.pop(update_id, None)
        if record is None:
            return
        self._dispose(record)
        record.state = "released"
        if self.active_update_id == update_id:
            self.active_update_id = None

    # -- introspection ---------------------------------------------------------------------------
    def update_status(self, update_id: str) -> str:
        record = self._updates.get(update_id)
        return "released" if record is None else record.state

    def get_manifest(self, update_id: str) -> WeightUpdateManifest:
        return self._require(update_id).manifest

    def debug_tensor_data_ptrs(self, update_id: str) -> Mapping[str, int]:
        return {n: int(t.data_ptr()) for n, t in self._require(update_id).tensors.items()}

    # -- helpers -----------------------------------------------------------------------------------
    def _require(self, update_id: str) -> UpdateRecord:
        try:
            return self._updates[update_id]
        except KeyError as exc:
            raise WeightUpdateRejectedError(f"unknown weight update {update_id}") from exc

    def _validate(self, record: UpdateRecord, manifest: WeightUpdateManifest) -> None:
        expected = record.manifest
        WeightLayout.from_metadata(manifest.metadata).validate_supported(allow_multi_rank=self.allow_multi_rank)
        if manifest.transport != expected.transport:
            raise WeightManifestValidationError(
                f"transport mismatch: expected {expected.transport}, got {manifest.transport}"
            )
        if manifest.weight_version != expected.weight_version:
            raise WeightManifestValidationError(
                f"weight_version mismatch: expected {expected.weight_version}, got {manifest.weight_version}"
            )
        if set(manifest.tensors) != set(expected.tensors):
            missing = sorted(set(expected.tensors) - set(manifest.tensors))
            extra = sorted(set(manifest.tensors) - set(expected.tensors))
            raise WeightManifestValidationError(f"tensor manifest mismatch: missing={missing}, extra={extra}")
        for name, want in expected.tensors.items():
            got = manifest.tensors[name]
            if got != want:
                raise WeightManifestValidationError(
                    f"tensor descriptor mismatch for {name}: expected {want}, got {got}"
                )
        current = TensorDescriptor.from_tensors({name: record.tensors[name] for name in expected.tensors})
        for name, want in expected.tensors.items():
            now = current[name]
            if now.sha256 != want.sha256:
                raise WeightManifestValidationError(
                    f"tensor checksum mismatch for {name}: expected {want.sha256}, got {now.sha256}"
                )
            if (now.shape, now.dtype, now.numel) != (want.shape, want.dtype, want.numel):
                raise WeightManifestValidationError(
                    f"stored tensor descriptor mismatch for {name}: expected {want}, got {now}"
                )
