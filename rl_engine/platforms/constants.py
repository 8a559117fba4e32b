"""Enumerations shared across the engine.

Parity: reference ``rl_engine/platforms/constants.py:4-112`` exposes the same enum names and
string values through a ``constants`` bag object.  This build targets NVIDIA B200 only, so the
non-CUDA members exist purely so that user code comparing against them keeps working.
"""

from __future__ import annotations

from enum import Enum
from types import SimpleNamespace


def _enum(name: str, **members: str) -> type:
    return Enum(name, {k: v for k, v in members.items()}, module=__name__)


DeviceType = _enum("DeviceType", CUDA="cuda", ROCM="rocm", NPU="npu", TPU="tpu", XPU="xpu", CPU="cpu")
BackendLib = _enum(
    "BackendLib",
    SM100="sm100",  # this build's hand-written Blackwell kernels
    FLASHINFER="flashinfer",
    AITER="aiter",
    TRITON="triton",
    CANN="cann",
    NATIVE="native",
)
PrecisionType = _enum(
    "PrecisionType", FP32="float32", FP16="float16", BF16="bfloat16", FP8="float8_e4m3", INT8="int8", INT4="int4"
)
SamplingMethod = _enum(
    "SamplingMethod",
    TOP_K="top_k",
    TOP_P="top_p",
    TOP_K_TOP_P="top_k_top_p",
    GREEDY="greedy",
    TEMPERATURE="temperature",
    NUCLEUS="nucleus",
)
MemoryFormat = _enum("MemoryFormat", CONTIGUOUS="contiguous", CHANNELS_LAST="channels_last", PRESERVE="preserve")
OperatorFusionLevel = _enum("OperatorFusionLevel", NONE="none", PARTIAL="partial", FULL="full")
KernelOptimizationLevel = _enum("KernelOptimizationLevel", DEFAULT="default", AGGRESSIVE="aggressive", CUSTOM="custom")
LoggingLevel = _enum(
    "LoggingLevel", DEBUG="debug", INFO="info", WARNING="warning", ERROR="error", CRITICAL="critical"
)
ProfilingMode = _enum("ProfilingMode", OFF="off", BASIC="basic", DETAILED="detailed", CUSTOM="custom")
DistributedStrategy = _enum(
    "DistributedStrategy",
    DATA_PARALLEL="data_parallel",
    MODEL_PARALLEL="model_parallel",
    PIPELINE_PARALLEL="pipeline_parallel",
    TENSOR_PARALLEL="tensor_parallel",
    CONTEXT_PARALLEL="context_parallel",
    EXPERT_PARALLEL="expert_parallel",
    HYBRID="hybrid",
)
CheckpointFormat = _enum(
    "CheckpointFormat", PT="pt", ONNX="onnx", TORCHSCRIPT="torchscript", MANIFEST_BLOB="manifest_blob", CUSTOM="custom"
)
ActivationFunction = _enum(
    "ActivationFunction", RELU="relu", GELU="gelu", SILU="silu", TANH="tanh", SIGMOID="sigmoid"
)

_GROUPS = dict(
    DeviceType=DeviceType, BackendLib=BackendLib, PrecisionType=PrecisionType, SamplingMethod=SamplingMethod,
    MemoryFormat=MemoryFormat, OperatorFusionLevel=OperatorFusionLevel, KernelOptimizationLevel=KernelOptimizationLevel,
    LoggingLevel=LoggingLevel, ProfilingMode=ProfilingMode, DistributedStrategy=DistributedStrategy,
    CheckpointFormat=CheckpointFormat, ActivationFunction=ActivationFunction,
)


class Constants(SimpleNamespace):
    """All enum groups as attributes of one object (``constants.DeviceType.CUDA``); the reference exposes the class as
    well as the instance (``rl_engine/platforms/constants.py:96-112``)."""

    def __init__(self) -> None:
        super().__init__(**_GROUPS)


constants = Constants()
