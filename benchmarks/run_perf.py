"""One-panel serving/training summary at RL shapes: fused log-prob speed-up and memory saving,
sampling speed-up, weight-sync latency.  Counterpart of the reference's ``scripts/run_perf.py``.

    python benchmarks/run_perf.py --vocab-size 128256 --seq-len 512 --g-sizes 8,16
"""

import argparse
import time

import torch

from common import peak_gb, time_ms


def main() -> None:
    ap = argparse.ArgumentParser(description="rl_engine summary benchmark")
    ap.add_argument("--vocab-size", type=int, default=128256)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--g-sizes", default="8,16", help="batch sizes (completions per step) to test")
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--repeat", type=int, default=5)
    args = ap.parse_args()
    from rl_engine.executors.weight_sync.transports import make_weight_bridge
    from rl_engine.kernels.registry import kernel_registry
    from rl_engine.kernels.sampling import SamplerBackend
    from rl_engine.testing import selected_logprobs_reference

    dev = "cuda" if torch.cuda.is_available() else "cpu"
    dtype = torch.bfloat16 if dev == "cuda" else torch.float32
    logp = kernel_registry.get_op("logp")
    rows = []
    for g in [int(x) for x in args.g_sizes.split(",") if x]:
        logits = torch.randn(g, args.seq_len, args.vocab_size, device=dev).to(dtype)
        ids = torch.randint(0, args.vocab_size, (g, args.seq_len), device=dev)
        fused, native = (lambda: logp.apply_fp32(logits, ids)), (lambda: selected_logprobs_reference(logits, ids))
        tf, tn = time_ms(fused, 2, args.repeat), time_ms(native, 2, args.repeat)
        saved = peak_gb(native) - peak_gb(fused)
        flat = logits.reshape(-1, args.vocab_size).float()[: min(g * args.seq_len, 512)]
        fs, ns = SamplerBackend(seed=0), SamplerBackend(seed=0)
        ns.backend = "torch"
        ts_f = time_ms(lambda: fs.sample(flat, top_k=args.top_k, top_p=args.top_p), 2, args.repeat)
        ts_n = time_ms(lambda: ns.sample(flat, top_k=args.top_k, top_p=args.top_p), 2, args.repeat)
        rows.append({"g": g, "logp_ms": tf["ms"], "logp_speedup": tn["ms"] / tf["ms"], "vram_saved": saved,
                     "sample_ms": ts_f["ms"], "sample_speedup": ts_n["ms"] / ts_f["ms"]})
        del logits
    bridge = make_weight_bridge("local-clone")
    model = torch.nn.Linear(1024, 1024).to(dev)
    t0 = time.perf_counter()
    manifest = bridge.publish(model, weight_version=1)
    bridge.import_update(manifest)
    bridge.acknowledge(manifest.update_id)
    sync_ms = (time.perf_counter() - t0) * 1e3

    def row(k, v):
        print(f"{k:<36}{str(v):>26}")

    print("=" * 62)
    print(f"{'rl_engine summary benchmark':^62}")
    row("device", torch.cuda.get_device_name(0) if dev == "cuda" else "cpu")
    row("shape", f"vocab={args.vocab_size} seq={args.seq_len} dtype={dtype}")
    print("-" * 62)
    for r in rows:
        row(f"G={r['g']}: logp ms / speed-up", f"{r['logp_ms']:.3f} / {r['logp_speedup']:.2f}x")
        row(f"G={r['g']}: logp memory saved (GB)", f"{r['vram_saved']:.2f}")
        row(f"G={r['g']}: sampling ms / speed-up", f"{r['sample_ms']:.3f} / {r['sample_speedup']:.2f}x")
    row("weight sync round trip (ms)", f"{sync_ms:.3f}")
    print("=" * 62)


if __name__ == "__main__":
    main()
