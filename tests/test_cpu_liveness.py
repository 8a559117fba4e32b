"""Host-side failure detection with CPU ranks: a rank that announces its departure between steps, a rank that dies
without a word, and the healthy case.  No GPU is involved; the failing rank simply stops (or raises) on the host."""

import os
import tempfile
import threading
import time

import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from rl_engine.parallel.liveness import RankLeftError, RankLiveness


def test_healthy_ranks_pass_every_step_together():
    store = dist.HashStore()
    world, steps, seen = 3, 5, []

    def run(rank):
        live = RankLiveness(store, rank, world, timeout_s=5.0)
        for step in range(steps):
            live.check(step)
            seen.append((rank, step))
        live.leave("done")

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=30)
    assert len(seen) == world * steps
    assert RankLiveness(store, 0, world).departed() == {r: "left (done)" for r in range(world)}


def test_announced_departure_is_seen_at_once_and_names_the_rank():
    store = dist.HashStore()
    a, b = RankLiveness(store, 0, 2, timeout_s=30.0), RankLiveness(store, 1, 2, timeout_s=30.0)
    t = threading.Thread(target=lambda: b.check(0))
    t.start()
    a.check(0)
    t.join(timeout=10)
    b.leave("out of memory in the data loader")
    t0 = time.monotonic()
    with pytest.raises(RankLeftError) as info:
        a.check(1)
    assert time.monotonic() - t0 < 5.0                      # no waiting for the 30 s limit
    assert info.value.ranks == {1: "left (out of memory in the data loader)"} and info.value.step == 1
    with pytest.raises(RuntimeError):
        b.check(1)                                          # a rank that left does not come back


def test_silent_rank_is_found_by_its_missing_report():
    store = dist.HashStore()
    a = RankLiveness(store, 0, 3, timeout_s=0.3)
    c = RankLiveness(store, 2, 3, timeout_s=0.3)
    c.beat(0)                                               # rank 2 reported step 0 once, rank 1 never did
    with pytest.raises(RankLeftError) as info:
        a.check(1)
    assert set(info.value.ranks) == {1, 2}
    assert "never reported" in info.value.ranks[1] and "last reported step 0" in info.value.ranks[2]


def _process_rank(rank, world, path, leave_after, queue):
    try:
        store = dist.FileStore(path, world)
        live = RankLiveness(store, rank, world, timeout_s=20.0)
        done = 0
        try:
            for step in range(6):
                live.check(step)
                done += 1
                if rank == 1 and step == leave_after:
                    live.leave("stopping after step %d" % step)     # between steps: nothing in flight
                    break
            queue.put((rank, done, None))
        except RankLeftError as exc:
            queue.put((rank, done, dict(exc.ranks)))
    except Exception as exc:  # pragma: no cover - reported to the parent
        queue.put((rank, -1, f"{type(exc).__name__}: {exc}"))


def test_departure_between_steps_across_processes():
    """Three processes share a file store; rank 1 leaves after step 2; the others stop at step 3 with its name instead
    of entering a collective that could never complete."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "store")
        procs = [ctx.Process(target=_process_rank, args=(r, 3, path, 2, queue)) for r in range(3)]
        for p in procs:
            p.start()
        results = {}
        try:
            for _ in procs:
                rank, done, info = queue.get(timeout=120)
                results[rank] = (done, info)
        finally:
            for p in procs:
                p.join(timeout=10)
                if p.is_alive():
                    p.terminate()
    assert results[1] == (3, None)
    for rank in (0, 2):
        done, info = results[rank]
        assert done == 3 and isinstance(info, dict) and set(info) == {1} and "stopping after step 2" in info[1], results


def test_trainer_checks_its_peers_before_launching_a_step():
    """A trainer with a liveness object raises before any work of the step when a peer has left, and steps normally
    while everybody reports."""
    import torch

    from rl_engine.models.config import tiny_llama
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel

    store = dist.HashStore()
    cfg = tiny_llama(head_dim=32)
    model = LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=1, activation_checkpointing=False)
    trainer = GRPOTrainer(model, lr=1e-3, micro_group=None)
    trainer.liveness = RankLiveness(store, 0, 2, timeout_s=5.0)
    peer = RankLiveness(store, 1, 2, timeout_s=5.0)
    batch = synthetic_batch(cfg.vocab_size, prompt_len=4, group=2, completion_len=3, seed=2)
    before = model.flat.clone()
    peer.beat(0)
    trainer.step_device(batch)                       # the peer reported step 0: the step runs
    assert not torch.equal(model.flat, before)
    after_first = model.flat.clone()
    peer.leave("preempted")
    with pytest.raises(RankLeftError):
        trainer.step_device(batch)                   # step 1 never starts
    assert torch.equal(model.flat, after_first)
