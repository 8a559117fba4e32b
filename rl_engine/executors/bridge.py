"""Weight-sync bridge: public import path (same names as the reference's ``executors/bridge.py:2662-2684``).

The implementation lives in ``rl_engine.executors.weight_sync`` (protocol / transports / adapters).
"""

from rl_engine.executors.weight_sync.protocol import (
    BRIDGE_METADATA_KEY, TensorDescriptor, WeightBridge, WeightBridgeError, WeightBridgeUnavailableError, WeightConsumer,
    WeightInstallAdapter, WeightLayout, WeightManifestValidationError, WeightPublisher, WeightUpdateManifest,
    WeightUpdateRejectedError,
)
from rl_engine.executors.weight_sync.transports import (
    CUDAVMMTensorBridge, FileBlobBridge, IPCWeightBridge, LocalTensorCopyBridge, NVLinkBroadcastBridge,
    SharedMemoryTensorBridge, make_weight_bridge, manifest_from_json, manifest_to_json,
)
from rl_engine.executors.weight_sync.vllm_adapters import (
    VLLMCheckpointWeightReloadAdapter, VLLMCUDAVMMExternalStorageAdapter, VLLMInProcessWeightReloadAdapter,
    VLLMIPCWeightUpdateRequestBuilder, VLLMWeightInstallAdapter,
)

__all__ = [
    "BRIDGE_METADATA_KEY", "CUDAVMMTensorBridge", "FileBlobBridge", "IPCWeightBridge", "LocalTensorCopyBridge",
    "NVLinkBroadcastBridge", "SharedMemoryTensorBridge", "TensorDescriptor", "VLLMCUDAVMMExternalStorageAdapter",
    "VLLMCheckpointWeightReloadAdapter", "VLLMInProcessWeightReloadAdapter", "VLLMIPCWeightUpdateRequestBuilder",
    "VLLMWeightInstallAdapter", "WeightBridge", "WeightBridgeError", "WeightBridgeUnavailableError", "WeightConsumer",
    "WeightInstallAdapter", "WeightLayout", "WeightManifestValidationError", "WeightPublisher", "WeightUpdateManifest",
    "WeightUpdateRejectedError", "make_weight_bridge", "manifest_from_json", "manifest_to_json",
]
