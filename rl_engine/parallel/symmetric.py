"""Symmetric memory for the ranks of one node.

Every rank allocates one CUDA virtual-memory segment of the same size (``_C.SymmetricHeap``),
exports it as a POSIX file descriptor and maps every peer's segment, so a kernel can address any
rank's copy of a buffer as ``peer_base[r] + offset``.  File descriptors are exchanged once over
unix sockets (``SCM_RIGHTS``); socket paths are agreed on through the ``torch.distributed`` group
that is passed in (NCCL or Gloo -- only ``all_gather_object`` / ``barrier`` are used, and only at
set-up time).  Allocation is a bump pointer kept in lock-step on all ranks, so equal call sequences
give equal offsets.

``barrier()`` is a device-side barrier (one tiny kernel): each rank raises a flag in every peer's
signal pad and waits, with a time limit, for all peers' flags.  When the limit expires the kernel
records the event, returns normally, and the next ``check()`` raises ``PeerTimeoutError``; the CUDA
context stays usable.

The reference has no symmetric memory; its closest relative is the single-writer CUDA-VMM weight
bridge (``rl_engine/executors/bridge.py:1993-2368``).
"""

from __future__ import annotations

import os
import socket
import tempfile
import threading
import uuid
from typing import List, Optional, Sequence

import torch

from rl_engine.kernels.ops.base import require_ext

_ALIGN = 256
_PAD_BYTES = 4096  # signal pad at the start of every segment
_BARRIER_CHANNELS = 8  # independent barrier sequences, 64 bytes of the pad each (one per stream that synchronises)


class PeerTimeoutError(RuntimeError):
    """A bounded device-side wait on a peer expired."""


def _serve_fd(server: socket.socket, fd: int, connections: int) -> None:
    for _ in range(connections):
        conn, _ = server.accept()
        with conn:
            socket.send_fds(conn, [b"fd"], [fd])


class SymmetricMemory:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None,
                 wait_limit_ms: float = 20000.0) -> None:
        import torch.distributed as dist

        self.group = group
        if dist.is_available() and dist.is_initialized():
            self.rank = dist.get_rank(group)
            self.world = dist.get_world_size(group)
        else:
            self.rank, self.world = 0, 1
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.wait_limit_ms = float(wait_limit_ms)
        ext = require_ext()
        self.heap = ext.SymmetricHeap(self.device.index or 0, int(nbytes) + _PAD_BYTES, self.rank, self.world)
        self._cursor = _PAD_BYTES
        self._epochs = [0] * _BARRIER_CHANNELS
        self._err = torch.zeros(4, dtype=torch.int32, device=self.device)
        if self.world > 1:
            self._exchange(dist)
        self.ptrs: List[int] = list(self.heap.ptrs())

    # -- set-up -------------------------------------------------------------------------------
    def _exchange(self, dist) -> None:
        fd = self.heap.export_fd()
        path = os.path.join(tempfile.gettempdir(), f"rlk-symm-{os.getpid()}-{uuid.uuid4().hex}.sock")
        server = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        server.bind(path)
        server.listen(self.world)
        thread = threading.Thread(target=_serve_fd, args=(server, fd, self.world - 1), daemon=True)
        thread.start()
        paths: List[Optional[str]] = [None] * self.world
        dist.all_gather_object(paths, path, group=self.group)
        try:
            for peer in range(self.world):
                if peer == self.rank:
                    continue
                with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as client:
                    client.settimeout(60.0)
                    client.connect(paths[peer])
                    _msg, fds, _flags, _addr = socket.recv_fds(client, 16, 1)
                if not fds:
                    raise RuntimeError(f"rank {peer} sent no file descriptor")
                self.heap.import_peer(peer, fds[0])
                os.close(fds[0])
            thread.join(timeout=60.0)
        finally:
            server.close()
            os.close(fd)
            try:
                os.unlink(path)
            except OSError:
                pass
        dist.barrier(group=self.group)

    # -- allocation ---------------------------------------------------------------------------
    def alloc(self, shape: Sequence[int], dtype: torch.dtype) -> "SymmetricTensor":
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        offset = (self._cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if offset + nbytes > self.heap.size():
            raise MemoryError(
                f"symmetric heap exhausted: need {offset + nbytes} bytes, segment has {self.heap.size()}"
            )
        self._cursor = offset + nbytes
        return SymmetricTensor(self, offset, tuple(int(s) for s in shape), dtype)

    # -- synchronisation ------------------------------------------------------------------------
    def barrier(self, channel: int = 0) -> None:
        """Device-side barrier on the current stream (bounded).

        Barriers of one ``channel`` must be issued by all ranks in the same order and on one stream per rank: the
        flags of a channel are epoch counters, so two barriers of a channel that ran concurrently on different
        streams could overtake each other.  Work on a second stream uses its own channel (0..7)."""
        if not 0 <= channel < _BARRIER_CHANNELS:
            raise ValueError(f"barrier channel must be in [0, {_BARRIER_CHANNELS})")
        self._epochs[channel] += 1
        pads = self.ptrs if channel == 0 else [p + 64 * channel for p in self.ptrs]
        require_ext().peer_barrier(pads, self.rank, self._epochs[channel], self.wait_limit_ms, self._err)

    @property
    def error_word(self) -> torch.Tensor:
        """int32[4] on the device: non-zero first element once a bounded wait of ``barrier`` has expired."""
        return self._err

    def check(self) -> None:
        """Synchronise and raise ``PeerTimeoutError`` if a bounded wait expired since the last check."""
        code, kernel, block, site = (int(x) for x in self._err.cpu())
        if code:
            self._err.zero_()
            raise PeerTimeoutError(
                f"peer wait timed out on rank {self.rank} (kernel {kernel}, waiting for rank {site}, "
                f"limit {self.wait_limit_ms} ms)"
            )

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self.heap.close()


class SymmetricTensor:
    """The same ``(offset, shape, dtype)`` window in every rank's segment."""

    def __init__(self, mem: SymmetricMemory, offset: int, shape, dtype) -> None:
        self.mem, self.offset, self.shape, self.dtype = mem, offset, shape, dtype
        self.local = mem.heap.tensor(mem.rank, offset, list(shape), dtype)

    def peer(self, rank: int) -> torch.Tensor:
        """A local COPY of rank ``rank``'s window (for tests and debugging; kernels use ``ptrs``)."""
        if rank == self.mem.rank:
            return self.local.clone()
        return self.mem.heap.read_peer(rank, self.offset, list(self.shape), self.dtype)

    @property
    def ptrs(self) -> List[int]:
        return [p + self.offset for p in self.mem.ptrs]
