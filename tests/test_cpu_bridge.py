"""CPU tests: weight-sync life cycle, transports (incl. cross-process shared memory), install adapters."""

import multiprocessing as mp
import os
import sys

import pytest
import torch

from rl_engine.executors.bridge import (
    CUDAVMMTensorBridge, FileBlobBridge, IPCWeightBridge, LocalTensorCopyBridge, SharedMemoryTensorBridge,
    TensorDescriptor, VLLMCheckpointWeightReloadAdapter, VLLMCUDAVMMExternalStorageAdapter,
    VLLMInProcessWeightReloadAdapter, VLLMIPCWeightUpdateRequestBuilder, VLLMWeightInstallAdapter,
    WeightBridgeUnavailableError, WeightLayout, WeightManifestValidationError, WeightUpdateRejectedError,
    make_weight_bridge, manifest_from_json, manifest_to_json,
)
from rl_engine.executors.rollout import RolloutExecutor


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(4, 3), torch.nn.Linear(3, 2, bias=False))


# ----------------------------------------------------------------------------------- life cycle
@pytest.mark.parametrize("transport", ["local-clone", "shared-memory"])
def test_publish_import_ack_release_state_machine(transport):
    bridge = make_weight_bridge(transport)
    model = _model()
    manifest = bridge.publish(model, weight_version=1, metadata={"note": "x"})
    assert manifest.transport == bridge.transport and manifest.tensor_count == 3
    assert manifest.total_nbytes == sum(p.numel() * 4 for p in model.parameters())
    assert manifest.metadata["layout"]["kind"] == "full-state" and bridge.update_status(manifest.update_id) == "published"
    with pytest.raises(WeightUpdateRejectedError):
        bridge.acknowledge(manifest.update_id)  # ack before import
    tensors = bridge.import_update(manifest)
    assert bridge.update_status(manifest.update_id) == "imported"
    for name, p in model.state_dict().items():
        assert torch.equal(tensors[name], p)
    bridge.acknowledge(manifest.update_id)
    assert bridge.active_weight_version == 1 and bridge.active_update_id == manifest.update_id
    with pytest.raises(WeightUpdateRejectedError):
        bridge.reject(manifest.update_id, "too late")
    with pytest.raises(WeightManifestValidationError):
        bridge.publish(model, weight_version=1)  # versions are monotonic
    bridge.release(manifest.update_id)
    assert bridge.update_status(manifest.update_id) == "released" and bridge.active_update_id is None
    bridge.release(manifest.update_id)  # idempotent
    with pytest.raises(WeightUpdateRejectedError):
        bridge.acknowledge(manifest.update_id)


def test_local_clone_isolates_and_detects_tampering():
    bridge = LocalTensorCopyBridge()
    model = _model()
    manifest = bridge.publish(model, weight_version=0)
    with torch.no_grad():
        model[0].weight.add_(1.0)  # later training must not leak into the published snapshot
    imported = bridge.import_update(manifest)
    assert not torch.equal(imported["0.weight"], model[0].weight)
    imported["0.weight"].zero_()  # nor may a consumer's edits
    assert bridge.import_update(manifest)["0.weight"].abs().sum() > 0
    ptrs = bridge.debug_tensor_data_ptrs(manifest.update_id)
    assert ptrs["0.weight"] != model[0].weight.data_ptr()
    bridge._updates[manifest.update_id].tensors["1.weight"].add_(1.0)  # corrupt the stored copy
    with pytest.raises(WeightManifestValidationError, match="checksum"):
        bridge.import_update(manifest)


def test_rejected_update_cannot_be_imported_and_unknown_ids():
    bridge = LocalTensorCopyBridge()
    manifest = bridge.publish(_model(), weight_version=3)
    bridge.reject(manifest.update_id, "bad eval")
    with pytest.raises(WeightUpdateRejectedError, match="bad eval"):
        bridge.import_update(manifest)
    other = LocalTensorCopyBridge()
    with pytest.raises(WeightUpdateRejectedError, match="unknown"):
        other.import_update(manifest)
    with pytest.raises(WeightManifestValidationError):
        bridge.publish(torch.nn.Module(), weight_version=9)  # no tensors


def test_manifest_mismatch_is_rejected():
    import dataclasses

    bridge = LocalTensorCopyBridge()
    manifest = bridge.publish(_model(), weight_version=1)
    with pytest.raises(WeightManifestValidationError, match="weight_version"):
        bridge.import_update(dataclasses.replace(manifest, weight_version=2))
    fewer = {k: v for k, v in manifest.tensors.items() if k != "1.weight"}
    with pytest.raises(WeightManifestValidationError, match="missing"):
        bridge.import_update(dataclasses.replace(manifest, tensors=fewer))
    wrong = dict(manifest.tensors)
    wrong["1.weight"] = dataclasses.replace(wrong["1.weight"], sha256="0" * 64)
    with pytest.raises(WeightManifestValidationError, match="descriptor"):
        bridge.import_update(dataclasses.replace(manifest, tensors=wrong))


def test_layout_rules_and_factory_names():
    assert WeightLayout.from_metadata(None) == WeightLayout()
    assert WeightLayout.from_metadata({"layout": {"zero_stage": "3"}}).zero_stage == 3
    with pytest.raises(WeightManifestValidationError):
        WeightLayout.from_metadata({"layout": 5})
    bridge = LocalTensorCopyBridge()
    for layout, err in (({"kind": "tp-shard"}, WeightBridgeUnavailableError),
                        ({"tensor_parallel_size": 2}, WeightBridgeUnavailableError),
                        ({"node_count": 2}, WeightBridgeUnavailableError), ({"rdma_enabled": True}, WeightBridgeUnavailableError),
                        ({"rank": 2, "world_size": 2}, WeightManifestValidationError),
                        ({"data_parallel_size": 0}, WeightManifestValidationError)):
        with pytest.raises(err):
            bridge.publish(_model(), weight_version=10, metadata={"layout": layout})
    assert isinstance(make_weight_bridge("local"), LocalTensorCopyBridge)
    assert isinstance(make_weight_bridge("shm"), SharedMemoryTensorBridge)
    assert isinstance(make_weight_bridge("cuda-vmm-fd"), CUDAVMMTensorBridge)
    assert isinstance(make_weight_bridge("ipc"), IPCWeightBridge)
    for name in ("rdma", "multi-node", "nccl-rdma", "carrier-pigeon"):
        with pytest.raises(WeightBridgeUnavailableError):
            make_weight_bridge(name)
    with pytest.raises(WeightBridgeUnavailableError):
        make_weight_bridge("nvlink-broadcast")  # needs a SymmetricMemory


def test_descriptor_and_manifest_json_roundtrip(tmp_path):
    t = torch.arange(12, dtype=torch.float32).view(3, 4).t()
    d = TensorDescriptor.from_tensor("w", t)
    assert d.shape == (4, 3) and d.stride == (1, 4) and d.nbytes == 48 and len(d.sha256) == 64
    assert d.sha256 == TensorDescriptor.from_tensor("w", t.contiguous()).sha256  # digest is over logical values
    bridge = FileBlobBridge(str(tmp_path))
    model = _model()
    manifest = bridge.publish(model, weight_version=4)
    again = manifest_from_json(manifest_to_json(manifest))
    assert again.tensors == manifest.tensors and again.weight_version == 4
    block = manifest.metadata["weight_bridge"]
    assert block["format"] == "packed-blob-file-v1" and all(e["offset"] % 256 == 0 for e in block["tensors"].values())
    fresh = FileBlobBridge(str(tmp_path))  # e.g. another process, later: manifest + blob on disk are enough
    tensors = fresh.import_update(fresh.load_manifest(manifest.update_id))
    for name, p in model.state_dict().items():
        assert torch.equal(tensors[name], p)


# ----------------------------------------------------------------------- shared memory transport
def _child_import(manifest, queue):
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from rl_engine.executors.bridge import SharedMemoryTensorBridge as Bridge

    try:
        bridge = Bridge()
        tensors = bridge.import_update(manifest)
        before = float(tensors["0.weight"].sum())
        bridge.acknowledge(manifest.update_id)
        tensors["0.bias"].fill_(7.0)  # zero copy: the publisher must see this write
        queue.put(("ok", before))
        bridge.release(manifest.update_id)
    except Exception as exc:  # pragma: no cover
        queue.put(("error", f"{type(exc).__name__}: {exc}"))


def test_shared_memory_is_zero_copy_across_processes_and_released_segments_vanish():
    bridge = SharedMemoryTensorBridge()
    model = _model()
    manifest = bridge.publish(model, weight_version=1)
    assert manifest.metadata["weight_bridge"]["format"] == "python-multiprocessing-shared-memory-v1"
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    child = ctx.Process(target=_child_import, args=(manifest, queue))
    child.start()
    status, value = queue.get(timeout=120)
    child.join(timeout=30)
    assert status == "ok", value
    assert abs(value - float(model[0].weight.sum())) < 1e-6
    assert (bridge._updates[manifest.update_id].tensors["0.bias"] == 7.0).all()  # the child's write is visible here
    with pytest.raises(WeightManifestValidationError, match="checksum"):
        bridge.import_update(manifest)  # ... and counts as tampering for any later import
    bridge.release(manifest.update_id)
    with pytest.raises((FileNotFoundError, WeightUpdateRejectedError)):
        SharedMemoryTensorBridge().import_update(manifest)
    with pytest.raises(WeightBridgeUnavailableError):
        bridge.publish({"w": torch.zeros(2, device="meta")}, weight_version=2)


# ---------------------------------------------------------------------------------- CUDA VMM
class _FakeSegment:
    """Stands in for _C.VmmSegment on machines without a GPU: a host buffer keyed by a fake descriptor."""

    store = {}

    def __init__(self, device, nbytes, fd=-1):
        if fd >= 0:
            self.buf = _FakeSegment.store["shared"]
        else:
            self.buf = torch.zeros(max(nbytes, 1) + 256, dtype=torch.uint8)
            _FakeSegment.store["shared"] = self.buf
        self.closed = False

    def export_fd(self):
        r, w = os.pipe()
        os.close(w)
        return r

    def size(self):
        return self.buf.numel()

    def tensor(self, offset, shape, strides, dtype):
        n = int(torch.tensor(shape).prod()) if len(shape) else 1
        item = torch.empty((), dtype=dtype).element_size()
        return self.buf[offset : offset + n * item].view(dtype).view(shape)

    def close(self):
        self.closed = True


def test_cuda_vmm_bridge_protocol_with_injected_backend():
    publisher = CUDAVMMTensorBridge(segment_factory=_FakeSegment, device_index=0)
    model = _model()
    manifest = publisher.publish(model, weight_version=1)
    block = manifest.metadata["weight_bridge"]
    assert block["format"] == "cuda-vmm-posix-fd-v1" and os.path.exists(block["socket_path"])
    assert all(e["offset"] % 256 == 0 for e in block["tensors"].values())
    consumer = CUDAVMMTensorBridge(segment_factory=_FakeSegment)
    tensors = consumer.import_update(manifest)  # fd arrives over the unix socket
    for name, p in model.state_dict().items():
        assert torch.equal(tensors[name], p)
    consumer.acknowledge(manifest.update_id)
    assert tensors["0.weight"].data_ptr() == publisher._updates[manifest.update_id].tensors["0.weight"].data_ptr()
    consumer.release(manifest.update_id)
    publisher.release(manifest.update_id)
    assert not os.path.exists(block["socket_path"])
    with pytest.raises(WeightUpdateRejectedError):
        CUDAVMMTensorBridge(segment_factory=_FakeSegment).import_update(manifest)  # publisher is gone


# ------------------------------------------------------------------------- rollout executor
class _FailingAdapter:
    def __init__(self):
        self.released = []

    def install(self, manifest, tensors):
        raise RuntimeError("engine refused the weights")

    def release(self, update_id):
        self.released.append(update_id)


def test_rollout_executor_switches_versions_and_keeps_previous_on_failure():
    bridge = LocalTensorCopyBridge()
    installs = []
    adapter = VLLMWeightInstallAdapter(object(), install_callable=lambda m, t: installs.append(m.weight_version))
    executor = RolloutExecutor(weight_bridge=bridge, weight_install_adapter=adapter)
    m1 = bridge.publish(_model(1), weight_version=1)
    executor.update_weights(m1)
    m2 = bridge.publish(_model(2), weight_version=2)
    executor.update_weights(m2)
    assert installs == [1, 2] and executor.active_weight_version == 2
    assert bridge.update_status(m1.update_id) == "released"  # superseded update is released
    executor.weight_install_adapter = _FailingAdapter()
    m3 = bridge.publish(_model(3), weight_version=3)
    with pytest.raises(RuntimeError, match="refused"):
        executor.update_weights(m3)
    assert bridge.update_status(m3.update_id) == "rejected"
    assert executor.active_weight_version == 2 and executor.active_weight_update_id == m2.update_id
    with pytest.raises(WeightBridgeUnavailableError):
        executor.update_weights_via_ipc({})
    executor.weight_install_adapter = None
    executor.release_weights()
    assert executor.shared_weights == {} and executor.active_weight_update_id is None


# ------------------------------------------------------------------------------ vLLM adapters
def test_vllm_install_adapter_capability_resolution():
    manifest = LocalTensorCopyBridge().publish(_model(), weight_version=1)
    tensors = {n: torch.zeros(d.shape) for n, d in manifest.tensors.items()}
    with pytest.raises(WeightBridgeUnavailableError, match="install capability"):
        VLLMWeightInstallAdapter(object()).install(manifest, tensors)

    class WithUpdate:
        def __init__(self):
            self.requests = []

        def update_weights(self, request):
            self.requests.append(request)

    with pytest.raises(WeightBridgeUnavailableError, match="request_builder"):
        VLLMWeightInstallAdapter(WithUpdate()).install(manifest, tensors)
    engine = WithUpdate()
    adapter = VLLMWeightInstallAdapter(engine, request_builder=lambda m, t: {"names": sorted(t)})
    adapter.install(manifest, tensors)
    assert engine.requests == [{"names": sorted(tensors)}] and adapter.active_weight_version == 1

    class ManifestAware:
        def load_weights_from_manifest(self, m, t):
            self.seen = (m.weight_version, len(t))

    aware = ManifestAware()
    VLLMWeightInstallAdapter(aware).install(manifest, tensors)
    assert aware.seen == (1, 3)
    adapter.release(manifest.update_id)
    assert adapter.active_update_id is None


class _FakeCudaTensor:
    """Duck-typed CUDA tensor so the IPC request builder can be exercised on a CPU box."""

    is_cuda = True

    def __init__(self, t):
        self._t = t
        self.shape, self.dtype, self.device = t.shape, t.dtype, type("D", (), {"type": "cuda"})()

    def detach(self):
        return self

    def contiguous(self):
        return self


def test_ipc_request_builder_shape_and_keepalive():
    manifest = LocalTensorCopyBridge().publish(_model(), weight_version=5)
    tensors = {n: _FakeCudaTensor(torch.zeros(d.shape)) for n, d in manifest.tensors.items()}
    builder = VLLMIPCWeightUpdateRequestBuilder(reduce_tensor=lambda t: ("handle", id(t)), gpu_uuid_resolver=lambda: "GPU-abc")
    info = builder(manifest, tensors)["update_info"]
    assert info["names"] == list(manifest.tensors) and info["dtype_names"] == ["float32"] * 3
    assert info["shapes"][0] == [3, 4] and list(info["ipc_handles"][0]) == ["GPU-abc"] and info["is_checkpoint_format"] is True
    assert len(builder._keepalive[manifest.update_id]) == 3
    builder.release(manifest.update_id)
    assert manifest.update_id not in builder._keepalive
    cpu = {n: torch.zeros(d.shape) for n, d in manifest.tensors.items()}
    with pytest.raises(WeightBridgeUnavailableError):
        builder(manifest, cpu)
    with pytest.raises(WeightManifestValidationError):
        builder(manifest, {})


def test_reload_adapters_in_process_and_checkpoint():
    manifest = LocalTensorCopyBridge().publish(_model(), weight_version=2)
    tensors = {n: torch.randn(d.shape) for n, d in manifest.tensors.items()}

    class Direct:
        def reload_weights(self, weights_iterator=None, is_checkpoint_format=None, weights_path=None):
            self.got = (weights_iterator, is_checkpoint_format, weights_path)

    eng = Direct()
    VLLMInProcessWeightReloadAdapter(eng, target_dtype=torch.bfloat16, synchronize_cuda=False).install(manifest, tensors)
    weights, fmt, _ = eng.got
    assert [n for n, _ in weights] == list(manifest.tensors) and weights[0][1].dtype == torch.bfloat16 and fmt is True

    class Rpc:
        class llm_engine:
            calls = []

            @classmethod
            def collective_rpc(cls, method, kwargs=None):
                cls.calls.append((method, kwargs))

    VLLMInProcessWeightReloadAdapter(Rpc(), synchronize_cuda=False).install(manifest, tensors)
    assert Rpc.llm_engine.calls[0][0] == "reload_weights"
    with pytest.raises(WeightBridgeUnavailableError):
        VLLMInProcessWeightReloadAdapter(object(), synchronize_cuda=False).install(manifest, tensors)
    bad = dict(tensors)
    bad["0.bias"] = torch.zeros(5)
    with pytest.raises(WeightManifestValidationError, match="shape"):
        VLLMInProcessWeightReloadAdapter(eng, synchronize_cuda=False).install(manifest, bad)

    eng2 = Direct()
    with pytest.raises(WeightBridgeUnavailableError, match="weights_path"):
        VLLMCheckpointWeightReloadAdapter(eng2).install(manifest, tensors)
    VLLMCheckpointWeightReloadAdapter(eng2, weights_path_resolver=lambda m: f"/ckpt/v{m.weight_version}").install(manifest, tensors)
    assert eng2.got[2] == "/ckpt/v2"


def test_external_storage_adapter_rebinds_and_rolls_back():
    """The function run on the worker imports the update through its own consumer bridge, rebinds the parameters it
    knows, acknowledges; release restores the original storage; a tensor that does not fit undoes the rebinding and
    releases the import; ``require_all_parameters`` insists on every tensor."""
    model = _model(3)
    publisher = CUDAVMMTensorBridge(segment_factory=_FakeSegment, device_index=0)
    manifest = publisher.publish(_model(4), weight_version=1)
    aliases = dict(publisher.import_update(manifest))
    originals = {n: p.data_ptr() for n, p in model.named_parameters()}
    calls = []

    class Consumer:
        def __init__(self, tensors):
            self.tensors = tensors

        def import_update(self, m):
            calls.append(("import", m.update_id))
            return self.tensors

        def acknowledge(self, update_id):
            calls.append(("ack", update_id))

        def release(self, update_id):
            calls.append(("release", update_id))

    adapter = VLLMCUDAVMMExternalStorageAdapter(object(), apply_model=lambda fn: fn(model), synchronize_cuda=False,
                                                bridge_factory=lambda: Consumer(aliases))
    adapter.install(manifest, {})
    assert adapter.active_weight_version == 1 and adapter.last_result[0]["zero_copy"] is True
    assert sorted(adapter.last_result[0]["rebound"]) == sorted(aliases)
    for name, p in model.named_parameters():
        assert p.data_ptr() == aliases[name].data_ptr()  # parameters now alias the published memory
    adapter.release(manifest.update_id)
    assert {n: p.data_ptr() for n, p in model.named_parameters()} == originals
    assert calls == [("import", manifest.update_id), ("ack", manifest.update_id), ("release", manifest.update_id)]
    assert adapter.active_update_id is None
    # not a cuda-vmm update
    local = LocalTensorCopyBridge().publish(_model(), weight_version=1)
    with pytest.raises(WeightBridgeUnavailableError, match="cuda-vmm"):
        adapter.install(local, {})
    # a tensor that does not fit: nothing stays rebound, the import is released, nothing is acknowledged
    calls.clear()
    broken = dict(aliases)
    broken["1.weight"] = torch.zeros(7, 7)
    bad = VLLMCUDAVMMExternalStorageAdapter(object(), apply_model=lambda fn: fn(model), synchronize_cuda=False,
                                            bridge_factory=lambda: Consumer(broken))
    with pytest.raises(WeightManifestValidationError, match="shape mismatch"):
        bad.install(manifest, {})
    assert {n: p.data_ptr() for n, p in model.named_parameters()} == originals
    assert ("release", manifest.update_id) in calls and ("ack", manifest.update_id) not in calls
    # a worker whose model lacks a parameter: fine by default, an error when every tensor is required
    partial = dict(aliases)
    partial["extra.weight"] = torch.zeros(2)
    import dataclasses

    wider = dataclasses.replace(manifest, tensors={**manifest.tensors, "extra.weight": manifest.tensors["1.weight"]})
    lenient = VLLMCUDAVMMExternalStorageAdapter(object(), apply_model=lambda fn: [fn(model)], synchronize_cuda=False,
                                                bridge_factory=lambda: Consumer(partial))
    lenient.install(wider, {})
    assert "extra.weight" not in lenient.last_result[0]["rebound"]
    lenient.release(wider.update_id)
    strict = VLLMCUDAVMMExternalStorageAdapter(object(), apply_model=lambda fn: [fn(model)], synchronize_cuda=False,
                                               bridge_factory=lambda: Consumer(partial), require_all_parameters=True)
    with pytest.raises(WeightManifestValidationError, match="extra.weight"):
        strict.install(wider, {})
    assert {n: p.data_ptr() for n, p in model.named_parameters()} == originals
    publisher.release(manifest.update_id)
    with pytest.raises(WeightBridgeUnavailableError):
        VLLMCUDAVMMExternalStorageAdapter(object()).install(manifest, aliases)
