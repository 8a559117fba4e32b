"""Device context: which accelerator this process drives.

Parity: reference ``rl_engine/platforms/device.py:10-55`` (``device_ctx`` singleton with
``device``, ``device_type``, ``is_rocm``, ``backend_version``, ``get_preferred_dtype``).
This build is B200-only: ``device_type`` is ``"cuda"`` or ``"cpu"``, ``is_rocm`` is always
False, and the preferred dtype on GPU is bfloat16 (the tcgen05 kernels are bf16-in/fp32-acc).
The context also records the process rank/local rank/world size from the launcher environment.
"""

from __future__ import annotations

import os

import torch

from rl_engine.platforms.constants import DeviceType
from rl_engine.utils.logger import logger


class DeviceContext:
    def __init__(self) -> None:
        self.rank = int(os.environ.get("RANK", "0") or 0)
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0") or 0)
        self.world_size = int(os.environ.get("WORLD_SIZE", "1") or 1)
        self.is_rocm = False
        self.backend_version = "N/A"
        self.capability = (0, 0)
        self.sm_count = 0
        if torch.cuda.is_available():
            index = self.local_rank % max(torch.cuda.device_count(), 1)
            self.device = torch.device("cuda", index)
            self.device_type = DeviceType.CUDA.value
            self.backend_version = str(torch.version.cuda)
            try:
                self.capability = tuple(torch.cuda.get_device_capability(index))
                self.sm_count = torch.cuda.get_device_properties(index).multi_processor_count
            except Exception as exc:  # pragma: no cover - driver hiccup
                logger.warning("could not query device properties: %s", exc)
            logger.info_once(
                "RL-Engine initialized with NVIDIA CUDA backend (Version: %s, sm_%d%d, %d SMs)",
                self.backend_version,
                self.capability[0],
                self.capability[1],
                self.sm_count,
            )
        else:
            self.device = torch.device("cpu")
            self.device_type = DeviceType.CPU.value
            logger.info_once("No GPU detected. RL-Engine runs its CPU reference operators.")

    @property
    def is_blackwell(self) -> bool:
        """True when the visible GPU can run the sm_100a kernels of this build."""
        return self.device_type == DeviceType.CUDA.value and self.capability[0] == 10

    def get_preferred_dtype(self) -> torch.dtype:
        return torch.bfloat16 if self.device_type == DeviceType.CUDA.value else torch.float32


device_ctx = DeviceContext()
