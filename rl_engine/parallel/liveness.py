"""Host-side liveness of the ranks of a multi-GPU job.

The device-side waits of this library are bounded: a peer that never arrives turns into ``PeerTimeoutError`` after the
wait limit instead of a hang.  That is the last line of defence; the first one is not to launch a step whose peers are
gone.  ``RankLiveness`` gives the ranks a place to say "I reached step n" and "I am leaving" through any
``torch.distributed`` key-value store (``TCPStore``, ``FileStore``, ``HashStore``), and a check that every rank calls on
the host between steps, with none of its kernels or collectives in flight:

    live = RankLiveness(store, rank, world, timeout_s=5.0)
    for step in range(...):
        live.check(step)          # raises RankLeftError if a peer left or stopped reporting
        trainer.step(...)
    live.leave("done")

A rank that stops on purpose (an exception between steps, a preemption notice) calls ``leave(reason)``; the others
learn of it at their next ``check`` without waiting (a check of a step that the leaver had still reported passes).
A rank that dies without a word is found by its missing report after ``timeout_s``.  Nothing here touches a GPU, so
failures are tested with CPU ranks.  The reference has no counterpart (no elasticity, heartbeats or retries).
"""

from __future__ import annotations

import time
from typing import Dict, Optional


class RankLeftError(RuntimeError):
    """One or more ranks announced that they leave, or stopped reporting.  ``ranks``: rank -> what is known."""

    def __init__(self, ranks: Dict[int, str], step: int) -> None:
        self.ranks, self.step = dict(ranks), int(step)
        detail = ", ".join(f"rank {r}: {why}" for r, why in sorted(ranks.items()))
        super().__init__(f"step {step} cannot start: {detail}")


class RankLiveness:
    def __init__(self, store, rank: int, world: int, *, timeout_s: float = 5.0, poll_s: float = 0.01,
                 prefix: str = "rl_engine/liveness") -> None:
        if not 0 <= rank < world:
            raise ValueError(f"rank {rank} is not in a world of {world}")
        self.store, self.rank, self.world = store, int(rank), int(world)
        self.timeout_s, self.poll_s, self.prefix = float(timeout_s), float(poll_s), prefix
        self._left = False

    # -- what this rank says ---------------------------------------------------------------------------------
    def beat(self, step: int) -> None:
        """This rank is alive and about to run ``step``."""
        self.store.set(f"{self.prefix}/step/{self.rank}", str(int(step)))

    def leave(self, reason: str = "left") -> None:
        """This rank takes no part in later steps.  Call it between steps, with nothing of this rank in flight."""
        if not self._left:
            self.store.set(f"{self.prefix}/left/{self.rank}", reason or "left")
            self._left = True

    # -- what this rank learns -------------------------------------------------------------------------------
    def _get(self, key: str) -> Optional[str]:
        if not self.store.check([key]):
            return None
        value = self.store.get(key)
        return value.decode() if isinstance(value, (bytes, bytearray)) else str(value)

    def departed(self) -> Dict[int, str]:
        """Ranks that have announced their departure, with their reasons."""
        out = {}
        for r in range(self.world):
            why = self._get(f"{self.prefix}/left/{r}")
            if why is not None:
                out[r] = f"left ({why})"
        return out

    def reached(self, rank: int) -> int:
        """The last step ``rank`` reported, or -1."""
        value = self._get(f"{self.prefix}/step/{rank}")
        return -1 if value is None else int(value)

    def check(self, step: int) -> None:
        """Reports ``step`` and returns once every rank has reported it (or a later one).  Raises ``RankLeftError``
        at once if a rank announced its departure, and after ``timeout_s`` if a rank stays silent."""
        if self._left:
            raise RuntimeError("this rank has left the job")
        self.beat(step)
        deadline = time.monotonic() + self.timeout_s
        while True:
            behind = {r: self.reached(r) for r in range(self.world) if r != self.rank}
            behind = {r: s for r, s in behind.items() if s < step}
            if not behind:
                return
            # a rank that left AFTER reporting this step took part in it; one that left before will never report it
            gone = {r: why for r, why in self.departed().items() if r in behind}
            if gone:
                raise RankLeftError(gone, step)
            if time.monotonic() > deadline:
                raise RankLeftError({r: (f"silent for {self.timeout_s:g} s (last reported step {s})" if s >= 0
                                         else f"never reported within {self.timeout_s:g} s") for r, s in behind.items()}, step)
            time.sleep(self.poll_s)
