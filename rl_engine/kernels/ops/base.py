"""Import guard for the native extension.

Parity: reference ``rl_engine/kernels/ops/base.py:8-17`` exposes ``_C`` and ``_EXT_AVAILABLE``.
Added here: ``require_ext()`` raises instead of silently falling back when a GPU is present but
the extension is missing, so a GPU run can never pass on a PyTorch fallback by accident.
"""

from __future__ import annotations

from typing import Any

import torch  # noqa: F401  (must be loaded first: the extension links against libc10 / libtorch)

from rl_engine.utils.logger import logger

_C: Any = None
_EXT_ERROR: str = ""

import os

try:
    if os.environ.get("RLK_DEBUG_BOUNDS") == "1":
        # the debug-bounds build: every index that comes from the caller (token ids, gathered rows, positions, group
        # bounds, expert slots) is range-checked on the device and a bad one is reported in the error word
        from rl_engine import _C_dbg as _C  # type: ignore[no-redef]
    else:
        from rl_engine import _C  # type: ignore[no-redef]

    _EXT_AVAILABLE = True
except ImportError as exc:  # not built, or built for another torch
    _EXT_AVAILABLE = False
    _EXT_ERROR = str(exc)
    logger.warn_once("Native extension rl_engine._C unavailable (%s); only CPU reference ops can run.", _EXT_ERROR)


def require_ext() -> Any:
    if not _EXT_AVAILABLE:
        raise RuntimeError(
            "rl_engine._C is not built; run `python setup.py build_ext --inplace` "
            f"(import error: {_EXT_ERROR})"
        )
    return _C


def check_device_errors(device: int = 0) -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait timeout or a bad argument."""
    code, kernel_id, block, site = require_ext().error_state(device)
    if code:
        require_ext().reset_error(device)
        names = {1: "mbarrier wait timed out", 2: "peer wait timed out", 3: "bad argument", 4: "index out of range"}
        raise RuntimeError(
            f"rl_engine kernel error: {names.get(code, code)} (kernel {kernel_id}, block {block}, site {site})"
        )
