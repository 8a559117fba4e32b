"""``rl_kernel_b200``: the same library under a layout-by-concern name space.

The implementation lives in ``rl_engine`` (the import paths users of the reference already have:
``rl_engine.kernels.registry.kernel_registry`` and friends).  This package only re-exports it grouped as

    rl_kernel_b200.ops       kernels and operators   (``rl_engine.kernels``)
    rl_kernel_b200.models    model definitions, GRPO trainer   (``rl_engine.models``)
    rl_kernel_b200.parallel  symmetric memory, data / tensor / context / expert parallelism   (``rl_engine.parallel``)
    rl_kernel_b200.utils     logger, tracing   (``rl_engine.utils``)
    rl_kernel_b200.executors rollout / training / scoring executors and the weight-sync bridge
"""

import importlib
import sys

_ALIASES = {
    "ops": "rl_engine.kernels",
    "models": "rl_engine.models",
    "parallel": "rl_engine.parallel",
    "utils": "rl_engine.utils",
    "executors": "rl_engine.executors",
    "testing": "rl_engine.testing",
    "platforms": "rl_engine.platforms",
    "alignment": "rl_engine.alignment",
    "integrations": "rl_engine.integrations",
}


def __getattr__(name: str):
    target = _ALIASES.get(name)
    if target is None:
        raise AttributeError(f"module 'rl_kernel_b200' has no attribute {name!r}")
    module = importlib.import_module(target)
    if name == "ops":  # make ops.registry / ops.sampling reachable without a second import
        importlib.import_module("rl_engine.kernels.registry")
        importlib.import_module("rl_engine.kernels.sampling")
    sys.modules[f"{__name__}.{name}"] = module
    return module


def __dir__():
    return sorted(_ALIASES)
