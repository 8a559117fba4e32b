"""Tracing and on-device timing helpers.

* ``trace_range(name)``: NVTX range (``torch.cuda.nvtx``) as a context manager / decorator; a no-op without CUDA.
  The native launchers open their own ranges when the process was started with ``RLK_NVTX=1``.
* ``PhaseTimer``: CUDA-event pairs per named phase on the launching stream, read once at the end, so the
  timed region contains no host synchronisation; ``summary()`` gives per-phase totals and
  ``max_over_ranks()`` reduces them with ``torch.distributed`` (a multi-GPU number is the slowest rank's).
* ``DeviceStamps``: ``%globaltimer`` stamps written by a one-thread kernel in stream order (same clock
  domain across the GPUs of a node), for intervals that start on one stream and end on another.

The reference has no tracing layer; its profiler brackets every repetition with host-synchronised CUDA
events (``benchmarks/profiler.py:187-214``).
"""

from __future__ import annotations

import contextlib
import functools
import time
from collections import OrderedDict
from typing import Dict, Iterator, List, Optional, Tuple

import torch


@contextlib.contextmanager
def trace_range(name: str) -> Iterator[None]:
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


def traced(name: Optional[str] = None):
    """Decorator form of ``trace_range``."""

    def deco(fn):
        label = name or fn.__qualname__

        @functools.wraps(fn)
        def wrapper(*args, **kwargs):
            with trace_range(label):
                return fn(*args, **kwargs)

        return wrapper

    return deco


class PhaseTimer:
    """Accumulates device time per named phase; host wall-clock on CPU."""

    def __init__(self, device: Optional[torch.device] = None) -> None:
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self._cuda = self.device.type == "cuda"
        self._pending: List[Tuple[str, object, object]] = []
        self._totals: "OrderedDict[str, float]" = OrderedDict()
        self._counts: Dict[str, int] = {}

    @contextlib.contextmanager
    def phase(self, name: str) -> Iterator[None]:
        if self._cuda:
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            with trace_range(name):
                yield
            stop.record()
            self._pending.append((name, start, stop))
        else:
            t0 = time.perf_counter()
            yield
            self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name: str, ms: float) -> None:
        self._totals[name] = self._totals.get(name, 0.0) + ms
        self._counts[name] = self._counts.get(name, 0) + 1

    def flush(self) -> None:
        """Read the recorded events (synchronises the device once)."""
        if self._pending:
            torch.cuda.synchronize(self.device)
            for name, start, stop in self._pending:
                self._add(name, start.elapsed_time(stop))
            self._pending.clear()

    def summary(self) -> "OrderedDict[str, Dict[str, float]]":
        self.flush()
        return OrderedDict((k, {"total_ms": v, "calls": self._counts[k], "mean_ms": v / self._counts[k]})
                           for k, v in self._totals.items())

    def max_over_ranks(self, group=None) -> "OrderedDict[str, float]":
        """Per-phase total time of the slowest rank (all ranks must have recorded the same phases)."""
        import torch.distributed as dist

        self.flush()
        names = list(self._totals)
        values = torch.tensor([self._totals[n] for n in names], dtype=torch.float64,
                              device=self.device if self._cuda else "cpu")
        if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
            dist.all_reduce(values, op=dist.ReduceOp.MAX, group=group)
        return OrderedDict(zip(names, values.tolist()))

    def reset(self) -> None:
        self._pending.clear()
        self._totals.clear()
        self._counts.clear()


class DeviceStamps:
    """``stamp(i)`` writes the device's global nanosecond timer into slot ``i`` in stream order."""

    def __init__(self, slots: int = 64, device: Optional[torch.device] = None) -> None:
        from rl_engine.kernels.ops.base import require_ext

        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._ext = require_ext()
        self.values = torch.zeros(slots, dtype=torch.int64, device=self.device)

    def stamp(self, slot: int) -> None:
        self._ext.device_stamp(self.values, int(slot))

    def read(self) -> List[int]:
        return self.values.cpu().tolist()

    def elapsed_ms(self, first: int, second: int) -> float:
        v = self.read()
        return (v[second] - v[first]) / 1e6
