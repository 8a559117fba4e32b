"""Process-wide logger with once-only and rank-filtered helpers.

Parity: reference ``rl_engine/utils/logger.py:10-75`` (format string, ``info_once`` /
``warn_once`` / ``info_on_rank`` helpers, stdout handler, logger name ``RL-Kernel``).
Unlike the reference, ``info_on_rank`` reads the real rank from ``RANK`` when the device
context does not carry one, so multi-process runs do not print once per rank.
"""

from __future__ import annotations

import logging
import os
import sys
from typing import Any, Set, Tuple

_FMT = "%(levelname)s %(asctime)s [%(name)s]: %(message)s"
_DATEFMT = "%m-%d %H:%M:%S"


class RLEngineLogger(logging.Logger):
    """``logging.Logger`` with the three helpers the engine uses everywhere."""

    def __init__(self, name: str, level: int = logging.NOTSET) -> None:
        super().__init__(name, level)
        self._seen: Set[Tuple[int, str, Tuple[Any, ...]]] = set()

    def _once(self, level: int, msg: str, args: Tuple[Any, ...]) -> None:
        key = (level, msg, args)
        if key in self._seen:
            return
        self._seen.add(key)
        self.log(level, msg, *args, stacklevel=3)

    def info_once(self, msg: str, *args: Any) -> None:
        self._once(logging.INFO, msg, args)

    def warn_once(self, msg: str, *args: Any) -> None:
        self._once(logging.WARNING, msg, args)

    def info_on_rank(self, msg: str, rank: int = 0, *args: Any) -> None:
        if _current_rank() == rank:
            self.info(msg, *args)


def _current_rank() -> int:
    try:
        from rl_engine.platforms.device import device_ctx

        ctx_rank = getattr(device_ctx, "rank", None)
        if ctx_rank is not None:
            return int(ctx_rank)
    except Exception:  # device module may still be importing
        pass
    return int(os.environ.get("RANK", "0") or 0)


def init_logger(name: str) -> RLEngineLogger:
    """Return the named engine logger, creating and configuring it on first use."""
    previous = logging.getLoggerClass()
    logging.setLoggerClass(RLEngineLogger)
    try:
        log = logging.getLogger(name)
    finally:
        logging.setLoggerClass(previous)
    if not isinstance(log, RLEngineLogger):  # created earlier by someone else
        log.__class__ = RLEngineLogger
        log._seen = set()  # type: ignore[attr-defined]
    if not log.handlers:
        handler = logging.StreamHandler(sys.stdout)
        handler.setFormatter(logging.Formatter(_FMT, datefmt=_DATEFMT))
        log.addHandler(handler)
        log.setLevel(os.environ.get("RL_KERNEL_LOG_LEVEL", "INFO").upper())
        log.propagate = False
    return log  # type: ignore[return-value]


logger = init_logger("RL-Kernel")
