from rl_engine.platforms.constants import constants
from rl_engine.platforms.device import DeviceContext, device_ctx

__all__ = ["constants", "DeviceContext", "device_ctx"]
