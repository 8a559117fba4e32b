"""Elastic loop on CPU ranks (threads sharing a store): a rank that leaves on purpose, a rank that dies silently, and
the resume of the survivors on a smaller world from the checkpoint the loop names.  Optimiser shards are the real
``ShardedFusedAdamW`` state (host tensors, stand-in symmetric memory), checkpoints are the real files."""

import threading
import types

import torch
import torch.distributed as dist

from rl_engine.executors.checkpoint import load_checkpoint, save_checkpoint
from rl_engine.models.config import ModelConfig
from rl_engine.models.llama import LlamaModel
from rl_engine.parallel.elastic import ElasticLoop
from rl_engine.parallel.liveness import RankLiveness


def tiny():
    cfg = ModelConfig("tiny", 64, 32, 2, 2, 1, 16, 48)
    return LlamaModel(cfg, dtype=torch.float32, device="cpu", seed=3, max_positions=32)


def sharded(model, rank, world):
    from rl_engine.parallel.data_parallel import ShardedFusedAdamW

    n = model.flat.numel()
    padded = (n + 7) // 8 * 8
    flat = torch.zeros(padded, dtype=model.flat.dtype)
    flat[:n].copy_(model.flat)
    holder = types.SimpleNamespace(local=flat, ptrs=[0] * world)
    mem = types.SimpleNamespace(rank=rank, world=world)
    return ShardedFusedAdamW(model, mem, holder, types.SimpleNamespace(local=torch.zeros_like(flat), ptrs=[0] * world),
                             lr=1e-3, overlap=False, layers_per_bucket=1)


def launch(world, body):
    results, errors = {}, []

    def run(rank):
        try:
            results[rank] = body(rank)
        except Exception as exc:  # noqa: BLE001
            errors.append((rank, exc))

    threads = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=60)
    assert not errors, errors
    return results


def make_rank(store, root, rank, world, *, timeout_s=5.0, save_every=0, die_at=None, leave_at=None):
    """One rank's loop over a fake step that moves the optimiser state in a rank- and step-dependent way."""
    model = tiny()
    opt = sharded(model, rank, world)
    holder = {}

    def step_fn(step):
        if die_at is not None and step == die_at:
            raise SystemExit                                      # gone without a word (caught by the thread body below)
        opt.m.add_(0.01 * (step + 1))
        opt.v.add_(0.001 * (rank + 1))
        opt.steps = step + 1
        if leave_at is not None and step + 1 == leave_at:
            holder["loop"].request_leave("preemption notice")

    def save_fn(directory):
        save_checkpoint(directory, model, opt, weight_version=opt.steps, rank=rank, world=world)

    live = RankLiveness(store, rank, world, timeout_s=timeout_s)
    holder["loop"] = ElasticLoop(live, step_fn, save_fn, root, save_every=save_every)
    return holder["loop"], opt, model


def test_announced_departure_leaves_a_complete_checkpoint_of_that_step_and_the_survivors_resume(tmp_path):
    store, world, root = dist.HashStore(), 3, str(tmp_path)
    states = {}

    def body(rank):
        loop, opt, _ = make_rank(store, root, rank, world, leave_at=4 if rank == 1 else None)
        states[rank] = opt
        return loop.run(0, 10)

    out = launch(world, body)
    assert out[1].status == "left" and out[1].next_step == 4 and out[1].checkpoint_step == 4
    for r in (0, 2):
        assert out[r].status == "rank_lost" and out[r].survivors == [0, 2] and out[r].checkpoint_step == 4
        assert "saved:4:preemption notice" in out[r].lost[1] and out[r].checkpoint == out[1].checkpoint
    # the survivors restart as a world of two from that directory; every element lands at its flat index
    truth = {}
    for opt in states.values():
        for lo, hi, off in opt.slices:
            for i in range(lo, hi):
                truth[i] = (float(opt.m[off + i - lo]), float(opt.v[off + i - lo]))
    for new_rank in range(2):
        model = tiny()
        fresh = sharded(model, new_rank, 2)
        state = load_checkpoint(out[0].checkpoint, model, fresh, rank=new_rank, world=2)
        assert state["world"] == 3 and fresh.steps == 4
        for lo, hi, off in fresh.slices:
            for i in range(lo, hi, 97):
                assert (float(fresh.m[off + i - lo]), float(fresh.v[off + i - lo])) == truth[i]


def test_silent_death_falls_back_to_the_last_periodic_checkpoint_that_every_rank_finished(tmp_path):
    store, world, root = dist.HashStore(), 3, str(tmp_path)

    def body(rank):
        loop, _, _ = make_rank(store, root, rank, world, timeout_s=0.5, save_every=2, die_at=5 if rank == 2 else None)
        try:
            return loop.run(0, 10)
        except SystemExit:
            return None

    out = launch(world, body)
    assert out[2] is None
    for r in (0, 1):
        assert out[r].status == "rank_lost" and out[r].next_step == 6 and out[r].survivors == [0, 1]
        assert "silent" in out[r].lost[2] and out[r].checkpoint_step == 4
    model = tiny()
    fresh = sharded(model, 1, 2)
    assert load_checkpoint(out[0].checkpoint, model, fresh, rank=1, world=2)["weight_version"] == 4 and fresh.steps == 4


def test_without_any_checkpoint_the_outcome_says_so_and_a_healthy_job_finishes(tmp_path):
    store = dist.HashStore()

    def body(rank):
        loop, _, _ = make_rank(store, str(tmp_path), rank, 2, timeout_s=0.3, die_at=1 if rank == 0 else None)
        try:
            return loop.run(0, 4)
        except SystemExit:
            return None

    out = launch(2, body)
    assert out[1].status == "rank_lost" and out[1].checkpoint is None and out[1].survivors == [1]
    store2 = dist.HashStore()
    done = launch(2, lambda rank: make_rank(store2, str(tmp_path / "ok"), rank, 2, save_every=2)[0].run(0, 5))
    assert all(o.status == "finished" and o.next_step == 5 for o in done.values())


def test_a_step_that_gives_up_on_a_peer_is_void_and_the_silent_rank_is_named(tmp_path):
    """The device-side form of a lost rank: the survivors' step raises (a bounded wait ran out).  The loop then asks
    who is gone, discards the step and points at the periodic checkpoint; with everybody alive the error propagates."""
    class PeerGone(RuntimeError):
        pass

    store, world, root = dist.HashStore(), 3, str(tmp_path)

    def body(rank):
        loop, opt, _ = make_rank(store, root, rank, world, timeout_s=0.5, save_every=2)
        inner = loop.step_fn

        def step_fn(step):
            if step == 3 and rank == 1:
                raise SystemExit                     # rank 1 dies inside step 3 ...
            if step == 3:
                raise PeerGone("peer 1 did not arrive within 20 ms")   # ... and the others' waits run out
            inner(step)

        loop.step_fn, loop.step_errors = step_fn, (PeerGone,)
        try:
            return loop.run(0, 8)
        except SystemExit:
            return None

    out = launch(world, body)
    for r in (0, 2):
        assert out[r].status == "rank_lost" and out[r].next_step == 3 and out[r].survivors == [0, 2]
        assert out[r].checkpoint_step == 2 and list(out[r].lost) == [1]
    # nobody is gone: the step's error is the caller's to see
    store2 = dist.HashStore()

    def healthy(rank):
        loop, _, _ = make_rank(store2, str(tmp_path / "h"), rank, 2, timeout_s=2.0)
        loop.step_errors = (PeerGone,)
        loop.step_fn = lambda step: (_ for _ in ()).throw(PeerGone("spurious"))
        try:
            loop.run(0, 2)
        except PeerGone:
            return "raised"

    assert launch(2, healthy) == {0: "raised", 1: "raised"}
