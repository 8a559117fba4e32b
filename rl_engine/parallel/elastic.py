"""Elastic training loop: keep stepping while every rank is alive, and leave a checkpoint to restart from when one is not.

Pieces it joins: ``RankLiveness`` (who is still here, decided on the host between steps), the per-rank checkpoint
files of ``rl_engine.executors.checkpoint`` and their world-size-agnostic loading (``OptimizerShardReader``).  With a
sharded optimiser the state of a rank that dies is gone with it, so two cases differ:

* a rank that leaves ON PURPOSE (preemption notice, an exception it caught between steps) first writes its own files
  for the step it stops at, then announces ``saved:<step>``; the survivors see the announcement at their next check,
  write their files for the same step, and the checkpoint of that very step is complete;
* a rank that dies WITHOUT a word is noticed by its missing report; the survivors fall back to the last periodic
  checkpoint (``save_every``), which all ranks wrote together.

Either way ``run`` returns an ``ElasticOutcome`` naming the checkpoint directory, the step it holds and the ranks that
are left; a supervisor restarts the job on that many ranks and ``load_checkpoint(..., world=len(survivors))`` re-cuts the
optimiser state.  Nothing here touches a device; the loop calls back into the trainer only between steps.  The
reference has no elasticity, heartbeats or retries.
"""

from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from rl_engine.parallel.liveness import RankLeftError, RankLiveness

_SAVED = "saved:"


@dataclass
class ElasticOutcome:
    status: str                       # "finished" | "left" (this rank left on purpose) | "rank_lost"
    next_step: int                    # the first step that has not run on this rank
    survivors: List[int] = field(default_factory=list)
    lost: Dict[int, str] = field(default_factory=dict)
    checkpoint: Optional[str] = None  # directory of the newest complete checkpoint, if any
    checkpoint_step: Optional[int] = None


class ElasticLoop:
    """``step_fn(step)`` runs one training step; ``save_fn(directory)`` writes THIS rank's checkpoint files into
    ``directory`` (e.g. ``lambda d: worker.save_checkpoint(d)``); both are called between steps only."""

    def __init__(self, liveness: RankLiveness, step_fn: Callable[[int], None], save_fn: Callable[[str], None],
                 checkpoint_root: str, *, save_every: int = 0, step_errors: Tuple[type, ...] = ()) -> None:
        """``step_errors``: exception types with which a step reports that a peer did not arrive (``PeerTimeoutError``
        of the bounded device waits, a process-group timeout).  After one of them the loop asks the liveness record who
        is gone; if nobody is, the exception is re-raised."""
        self.live, self.step_fn, self.save_fn = liveness, step_fn, save_fn
        self.step_errors = tuple(step_errors)
        self.root, self.save_every = checkpoint_root, int(save_every)
        self._leave_reason: Optional[str] = None
        self._periodic: List[int] = []

    def request_leave(self, reason: str = "preempted") -> None:
        """Ask this rank to stop at the next step boundary (callable from a signal handler or another thread)."""
        self._leave_reason = reason or "left"

    def directory(self, step: int) -> str:
        return os.path.join(self.root, f"step_{int(step):08d}")

    def _save(self, step: int) -> str:
        path = self.directory(step)
        os.makedirs(path, exist_ok=True)
        self.save_fn(path)
        self.live.store.set(f"{self.live.prefix}/saved/{int(step)}/{self.live.rank}", "1")   # my files are on disk
        return path

    def _complete(self, step: int) -> bool:
        """Whether every rank of the job has finished writing its files for ``step``."""
        return bool(self.live.store.check([f"{self.live.prefix}/saved/{int(step)}/{r}" for r in range(self.live.world)]))

    def _survivors(self, lost: Dict[int, str]) -> List[int]:
        return [r for r in range(self.live.world) if r not in lost]

    def run(self, first_step: int, last_step: int) -> ElasticOutcome:
        """Runs steps ``first_step .. last_step - 1``."""
        step = int(first_step)
        while step < last_step:
            if self._leave_reason is not None:
                # leave on purpose: my files first, then the announcement that tells the others which step to save
                path = self._save(step)
                self.live.leave(f"{_SAVED}{step}:{self._leave_reason}")
                return ElasticOutcome("left", step, checkpoint=path, checkpoint_step=step)
            try:
                self.live.check(step)
            except RankLeftError as err:
                return self._rank_lost(step, err)
            if self.save_every and step > first_step and step % self.save_every == 0:
                self._save(step)                    # every rank reaches this point for the same steps
                self._periodic.append(step)
            try:
                self.step_fn(step)
            except self.step_errors:
                # the step gave up on a peer: its result is void.  Everybody still alive arrives here (or at the next
                # check) and reports; whoever stays silent is the one that is gone.
                try:
                    self.live.check(step + 1)
                except RankLeftError as err:
                    return self._rank_lost(step, err, void_step=True)
                raise
            step += 1
        self.live.leave("done")
        return ElasticOutcome("finished", step, survivors=list(range(self.live.world)))

    def _rank_lost(self, step: int, err: RankLeftError, void_step: bool = False) -> ElasticOutcome:
        lost = dict(err.ranks)
        survivors = self._survivors(lost)
        saved_at = {None} if void_step else set()   # after a void step the state in memory is not a step boundary
        for why in lost.values():                   # "left (saved:<step>:<reason>)"
            marker = why.find(_SAVED)
            saved_at.add(int(why[marker + len(_SAVED):].split(":")[0].rstrip(")")) if marker >= 0 else None)
        if saved_at == {step}:
            # everybody who left wrote its files for this step: add mine; complete once all survivors have done so
            return ElasticOutcome("rank_lost", step, survivors, lost, self._save(step), step)
        for done in reversed(self._periodic):       # the newest periodic checkpoint that every rank finished writing
            if self._complete(done):
                return ElasticOutcome("rank_lost", step, survivors, lost, self.directory(done), done)
        return ElasticOutcome("rank_lost", step, survivors, lost)
