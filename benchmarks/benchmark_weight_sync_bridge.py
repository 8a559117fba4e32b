"""Weight-sync bridge round trips: publish -> import -> acknowledge -> release, per transport.

Counterpart of the reference's ``benchmarks/benchmark_weight_sync_bridge.py`` (one JSON row on stdout,
optional CSV).  Modes:

    local            clone into the consumer
    shared-memory    POSIX shared memory (CPU tensors)
    file             blob + manifest on disk (checkpoint transport)
    cuda-vmm         one VMM allocation per update, exported as a POSIX fd          (GPU)
    nvlink-broadcast cast + broadcast kernel into the symmetric-memory window; on a single rank this
                     measures the kernel's copy bandwidth                           (GPU)
    rollout-update   RolloutExecutor.update_weights end to end over the local transport
    runtime-blockers which transports this machine cannot run, and why

``--cross-process`` (shared-memory, file, cuda-vmm): the consumer is a SEPARATE process, as in deployment: the parent
publishes and ships the pickled manifest, the child attaches to the update through the transport (segment names, the
blob path, or the file descriptor received over the unix socket), validates every tensor against the manifest,
acknowledges and reports its timings; the parent then releases the update and the child checks that a released update
can no longer be imported.  The row doubles as an integration test of the transport (reference: the consumer-process
modes of its ``benchmark_weight_sync_bridge.py:164-259,432-508``).
"""

import argparse
import csv
import json
import multiprocessing as mp
import tempfile
import time
from pathlib import Path

import torch

import common  # noqa: F401  (puts the repository root on sys.path)


def make_model(hidden: int, layers: int, device, dtype) -> torch.nn.Module:
    torch.manual_seed(0)
    return torch.nn.Sequential(*[torch.nn.Linear(hidden, hidden) for _ in range(layers)]).to(device=device, dtype=dtype)


def model_bytes(model) -> int:
    return sum(p.numel() * p.element_size() for p in model.state_dict().values())


def round_trip(bridge, model, version: int, sync) -> dict:
    sync()
    t0 = time.perf_counter()
    manifest = bridge.publish(model, weight_version=version)
    sync()
    t1 = time.perf_counter()
    tensors = bridge.import_update(manifest)
    sync()
    t2 = time.perf_counter()
    bridge.acknowledge(manifest.update_id)
    bridge.release(manifest.update_id)
    sync()
    t3 = time.perf_counter()
    names = list(tensors)
    state = model.state_dict()
    ok = all(torch.equal(tensors[n].to(state[n].device, state[n].dtype), state[n]) for n in names[:4])
    return {"publish_ms": (t1 - t0) * 1e3, "import_ms": (t2 - t1) * 1e3, "ack_release_ms": (t3 - t2) * 1e3,
            "total_ms": (t3 - t0) * 1e3, "tensors": len(names), "verified": bool(ok), "manifest_bytes": manifest.total_nbytes}


def run_transport(args, transport: str, device: str, **kwargs) -> dict:
    from rl_engine.executors.weight_sync.transports import make_weight_bridge

    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    model = make_model(args.hidden_dim, args.layers, device, dtype)
    sync = (lambda: torch.cuda.synchronize()) if device == "cuda" else (lambda: None)
    bridge = make_weight_bridge(transport, **kwargs)
    round_trip(bridge, model, args.weight_version, sync)  # warm-up
    row = round_trip(bridge, model, args.weight_version + 1, sync)
    nbytes = model_bytes(model)
    row.update({"mode": args.mode, "transport": transport, "device": device, "weight_bytes": nbytes,
                "publish_gbs": nbytes / row["publish_ms"] / 1e6, "status": "pass"})
    return row


def _consumer_process(transport: str, kwargs: dict, conn) -> None:
    """Child side of ``--cross-process``: import, validate, acknowledge; after the parent's release, import must fail."""
    import common  # noqa: F401
    from rl_engine.executors.weight_sync.transports import make_weight_bridge

    try:
        manifest = conn.recv()
        bridge = make_weight_bridge(transport, **kwargs)
        t0 = time.perf_counter()
        tensors = bridge.import_update(manifest)
        if transport == "cuda-vmm":
            torch.cuda.synchronize()
        t1 = time.perf_counter()
        checksum = float(sum(t.double().sum() for t in tensors.values() if t.is_floating_point()))
        bridge.acknowledge(manifest.update_id)
        t2 = time.perf_counter()
        conn.send({"status": "imported", "import_ms": (t1 - t0) * 1e3, "ack_ms": (t2 - t1) * 1e3, "tensors": len(tensors),
                   "checksum": checksum, "active_version": bridge.active_weight_version})
        assert conn.recv() == "released"
        del tensors
        bridge.release(manifest.update_id)
        try:
            make_weight_bridge(transport, **kwargs).import_update(manifest)
            conn.send({"status": "stale import succeeded"})
        except Exception as exc:  # noqa: BLE001 - any refusal is the expected outcome
            conn.send({"status": "stale import refused", "error": type(exc).__name__})
    except Exception as exc:  # noqa: BLE001
        conn.send({"status": "failed", "error": f"{type(exc).__name__}: {exc}"[:300]})


def run_cross_process(args, transport: str, device: str, **kwargs) -> dict:
    from rl_engine.executors.weight_sync.transports import make_weight_bridge

    dtype = torch.bfloat16 if device == "cuda" else torch.float32
    model = make_model(args.hidden_dim, args.layers, device, dtype)
    sync = (lambda: torch.cuda.synchronize()) if device == "cuda" else (lambda: None)
    bridge = make_weight_bridge(transport, **kwargs)
    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_consumer_process, args=(transport, kwargs, child), daemon=True)
    proc.start()
    try:
        sync()
        t0 = time.perf_counter()
        manifest = bridge.publish(model, weight_version=args.weight_version)
        sync()
        publish_ms = (time.perf_counter() - t0) * 1e3
        parent.send(manifest)
        if not parent.poll(args.child_timeout):
            raise TimeoutError(f"the consumer process did not answer within {args.child_timeout} s")
        seen = parent.recv()
        if seen.get("status") != "imported":
            raise RuntimeError(f"consumer process: {seen}")
        want = float(sum(t.double().sum() for t in model.state_dict().values() if t.is_floating_point()))
        bridge.release(manifest.update_id)
        parent.send("released")
        after = parent.recv() if parent.poll(args.child_timeout) else {"status": "no answer"}
    finally:
        proc.join(timeout=30)
        if proc.is_alive():
            proc.terminate()
    nbytes = model_bytes(model)
    return {"mode": args.mode, "transport": transport, "device": device, "cross_process": True, "weight_bytes": nbytes,
            "publish_ms": publish_ms, "import_ms": seen["import_ms"], "ack_ms": seen["ack_ms"], "tensors": seen["tensors"],
            "verified": abs(seen["checksum"] - want) <= 1e-6 * max(1.0, abs(want)), "consumer_version": seen["active_version"],
            "after_release": after.get("status"), "status": "pass" if after.get("status") == "stale import refused" else "fail"}


def run_nvlink(args) -> dict:
    from rl_engine.parallel.symmetric import SymmetricMemory

    model = make_model(args.hidden_dim, args.layers, "cuda", torch.float32)
    cap = model_bytes(model) + (1 << 20)
    mem = SymmetricMemory(cap + (1 << 20))
    return run_transport_with(args, "nvlink-broadcast", model, memory=mem, capacity_bytes=cap, target_dtype=torch.bfloat16)


def run_transport_with(args, transport, model, **kwargs) -> dict:
    from rl_engine.executors.weight_sync.transports import make_weight_bridge

    bridge = make_weight_bridge(transport, **kwargs)
    sync = lambda: torch.cuda.synchronize()
    sync()
    rows = []
    for i in range(3):
        t0 = time.perf_counter()
        manifest = bridge.publish(model, weight_version=args.weight_version + i)
        sync()
        t1 = time.perf_counter()
        tensors = bridge.import_update(manifest)
        bridge.acknowledge(manifest.update_id)
        bridge.release(manifest.update_id)
        rows.append((t1 - t0) * 1e3)
    nbytes = model_bytes(model)
    name = next(iter(tensors))
    return {"mode": args.mode, "transport": transport, "device": "cuda", "weight_bytes": nbytes, "publish_ms": min(rows),
            "publish_gbs": nbytes / min(rows) / 1e6, "tensors": len(tensors), "target_dtype": str(tensors[name].dtype),
            "note": "fp32 -> bf16 cast fused into the broadcast kernel; checksum computed on the device", "status": "pass"}


def run_rollout_update(args) -> dict:
    from rl_engine.executors.rollout import RolloutExecutor
    from rl_engine.executors.weight_sync.transports import make_weight_bridge

    model = make_model(args.hidden_dim, args.layers, "cpu", torch.float32)
    bridge = make_weight_bridge("local-clone")
    rollout = RolloutExecutor({"name": "benchmark"}, weight_bridge=bridge)
    t0 = time.perf_counter()
    manifest = bridge.publish(model, weight_version=args.weight_version)
    tensors = rollout.update_weights(manifest)
    dt = (time.perf_counter() - t0) * 1e3
    return {"mode": args.mode, "transport": "local-clone", "total_ms": dt, "tensors": len(tensors),
            "weight_version": rollout.active_weight_version, "status": "pass"}


def run_blockers() -> dict:
    row = {"mode": "runtime-blockers", "cuda_available": torch.cuda.is_available(), "status": "pass"}
    try:
        from rl_engine.kernels.ops.base import require_ext

        require_ext()
        row["native_extension"] = "loaded"
    except Exception as exc:
        row["native_extension"] = f"blocked: {str(exc).splitlines()[0]}"
    if not torch.cuda.is_available():
        row["cuda-vmm"] = row["cuda-ipc"] = row["nvlink-broadcast"] = "blocked: no CUDA device"
    row["multi-node"] = "blocked: multi-node/RDMA weight transport is not implemented"
    return row


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--smoke", action="store_true")
    ap.add_argument("--mode", default="local", choices=["local", "shared-memory", "file", "cuda-vmm", "nvlink-broadcast",
                                                          "rollout-update", "runtime-blockers"])
    ap.add_argument("--hidden-dim", type=int, default=64)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--weight-version", type=int, default=1)
    ap.add_argument("--cross-process", action="store_true", help="run the consumer in a separate process")
    ap.add_argument("--child-timeout", type=float, default=120.0)
    ap.add_argument("--output", type=Path, default=None, help="optional CSV output; JSON always goes to stdout")
    args = ap.parse_args()
    if args.smoke:
        args.hidden_dim, args.layers = min(args.hidden_dim, 64), min(args.layers, 4)
    try:
        if args.cross_process:
            if args.mode == "shared-memory":
                row = run_cross_process(args, "shared-memory", "cpu")
            elif args.mode == "file":
                with tempfile.TemporaryDirectory() as d:
                    row = run_cross_process(args, "file", "cpu", directory=d)
            elif args.mode == "cuda-vmm":
                row = run_cross_process(args, "cuda-vmm", "cuda")
            else:
                raise ValueError("--cross-process supports the shared-memory, file and cuda-vmm transports")
        elif args.mode == "local":
            row = run_transport(args, "local-clone", "cuda" if torch.cuda.is_available() else "cpu")
        elif args.mode == "shared-memory":
            row = run_transport(args, "shared-memory", "cpu")
        elif args.mode == "file":
            with tempfile.TemporaryDirectory() as d:
                row = run_transport(args, "file", "cpu", directory=d)
        elif args.mode == "cuda-vmm":
            row = run_transport(args, "cuda-vmm", "cuda")
        elif args.mode == "nvlink-broadcast":
            row = run_nvlink(args)
        elif args.mode == "rollout-update":
            row = run_rollout_update(args)
        else:
            row = run_blockers()
    except Exception as exc:
        row = {"mode": args.mode, "status": "blocked", "notes": (str(exc).splitlines() or [type(exc).__name__])[0]}
    if args.output is not None:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        new = not args.output.exists()
        with args.output.open("a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=sorted(row))
            if new:
                w.writeheader()
            w.writerow(row)
    print(json.dumps(row, sort_keys=True))


if __name__ == "__main__":
    main()
