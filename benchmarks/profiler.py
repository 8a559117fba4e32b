"""Automated performance profiler: workloads x shapes -> metrics -> JSON / CSV reports.

Report contract (kept from the reference profiler, ``benchmarks/profiler.py:29-79,391-437``): a JSON report
is ``{"report_version": "1.0", "generated_at", "gpu_target": {...}, "metrics": [...]}``; a CSV report
appends one row per metric with the nested GPU description flattened to ``gpu_*`` columns and the
free-form ``extra`` dict to ``extra_*`` columns.  A workload that cannot run on the present machine is
recorded with ``status="blocked"``, infinite latency and the first line of the exception in ``notes``
instead of aborting the suite (reference ``benchmarks/profiler.py:578-603``).

Timing: CUDA events on the launching stream around each repetition, a synchronize on both sides, and a
write larger than L2 between repetitions so that no repetition starts with its inputs cached.

    python benchmarks/profiler.py --workloads logp_fused,linear_logp_fused --batch-sizes 8 --seq-lens 512 \
        --vocab-sizes 128256 --output report.json --format json
    python benchmarks/profiler.py --smoke --device cpu
"""

from __future__ import annotations

import argparse
import csv
import json
import statistics
import sys
import time
from dataclasses import asdict, dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Any, Callable, Dict, List, Optional, Tuple

import torch

REPO_ROOT = Path(__file__).resolve().parents[1]
if str(REPO_ROOT) not in sys.path:
    sys.path.insert(0, str(REPO_ROOT))


@dataclass(frozen=True)
class GPUTargetInfo:
    name: str
    architecture: str
    total_memory_gb: float
    driver_version: str
    backend: str
    compute_capability: Optional[str] = None
    device_index: int = 0


@dataclass
class BenchmarkMetrics:
    timestamp: str
    benchmark_name: str
    gpu_target: GPUTargetInfo
    batch_size: int
    seq_len: int
    vocab_size: int
    total_tokens: int
    latency_ms: float
    latency_std_ms: Optional[float] = None
    warmup_iterations: int = 0
    repeat_iterations: int = 1
    tokens_per_sec: float = 0.0
    tflops: float = 0.0
    peak_vram_gb: float = 0.0
    peak_vram_reduction_gb: Optional[float] = None
    status: str = "pass"
    notes: str = ""
    extra: Dict[str, Any] = field(default_factory=dict)

    def to_dict(self) -> Dict[str, Any]:
        out = asdict(self)
        out["gpu_target"] = asdict(self.gpu_target)
        return out


class GPUProfiler:
    @staticmethod
    def get_target_info(device_index: int = 0) -> GPUTargetInfo:
        if not torch.cuda.is_available():
            return GPUTargetInfo("CPU", "unknown", 0.0, "N/A", "cpu", None, -1)
        props = torch.cuda.get_device_properties(device_index)
        major, minor = props.major, props.minor
        arch = {10: "blackwell", 9: "hopper", 8: "ampere"}.get(major, f"sm_{major}{minor}")
        driver = "unknown"
        try:
            import pynvml

            pynvml.nvmlInit()
            driver = pynvml.nvmlSystemGetDriverVersion()
            driver = driver.decode() if isinstance(driver, bytes) else str(driver)
        except Exception:
            pass
        return GPUTargetInfo(props.name, arch, round(props.total_memory / 2**30, 2), driver, "cuda", f"{major}.{minor}",
                             device_index)


class PerformanceProfiler:
    def __init__(self, device: Optional[torch.device] = None, warmup: int = 3, repeat: int = 10) -> None:
        self.device = torch.device(device) if device is not None else torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.warmup, self.repeat = int(warmup), int(repeat)
        self.gpu_info = GPUProfiler.get_target_info(self.device.index or 0)
        self._metrics: List[BenchmarkMetrics] = []
        self._flush = None

    # -- FLOP models of the report (the reference's: ``benchmarks/profiler.py:226-245``) -------------------
    @staticmethod
    def estimate_logp_tflops(batch_size: int, seq_len: int, vocab_size: int) -> float:
        """TFLOP of one selected-token log-prob pass over ``[B, S, V]`` logits: about five operations per element
        (subtract the maximum, exponentiate, sum, divide, take the logarithm)."""
        return 5.0 * batch_size * seq_len * vocab_size / 1e12

    @staticmethod
    def estimate_sampling_tflops(batch_size: int, vocab_size: int) -> float:
        """TFLOP of one sampling step over ``[B, V]`` logits (the softmax dominates)."""
        return 5.0 * batch_size * vocab_size / 1e12

    # -- timing -------------------------------------------------------------------------------------
    def _flush_l2(self) -> None:
        if self.device.type != "cuda":
            return
        if self._flush is None:
            self._flush = torch.empty(256 << 20, dtype=torch.uint8, device=self.device)
        self._flush.zero_()

    def time_fn(self, fn: Callable[[], Any]) -> Tuple[Any, float, Optional[float]]:
        """(last result, median latency ms, stdev ms or None)."""
        result = None
        for _ in range(self.warmup):
            result = fn()
        samples: List[float] = []
        for _ in range(max(self.repeat, 1)):
            if self.device.type == "cuda":
                self._flush_l2()
                start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize(self.device)
                start.record()
                result = fn()
                stop.record()
                torch.cuda.synchronize(self.device)
                samples.append(start.elapsed_time(stop))
            else:
                t0 = time.perf_counter()
                result = fn()
                samples.append((time.perf_counter() - t0) * 1e3)
        return result, statistics.median(samples), (statistics.stdev(samples) if len(samples) > 1 else None)

    def peak_memory_gb(self, fn: Callable[[], Any]) -> float:
        if self.device.type != "cuda":
            return 0.0
        torch.cuda.synchronize(self.device)
        torch.cuda.reset_peak_memory_stats(self.device)
        base = torch.cuda.memory_allocated(self.device)
        fn()
        torch.cuda.synchronize(self.device)
        return (torch.cuda.max_memory_allocated(self.device) - base) / 2**30

    # -- records ------------------------------------------------------------------------------------
    def record(self, name: str, batch: int, seq: int, vocab: int, latency_ms: float, std_ms: Optional[float],
               flops: float = 0.0, peak_gb: float = 0.0, status: str = "pass", notes: str = "",
               extra: Optional[Dict[str, Any]] = None, reduction_gb: Optional[float] = None) -> BenchmarkMetrics:
        tokens = batch * seq
        finite = latency_ms > 0 and latency_ms != float("inf")
        m = BenchmarkMetrics(
            timestamp=datetime.now(timezone.utc).isoformat(), benchmark_name=name, gpu_target=self.gpu_info,
            batch_size=batch, seq_len=seq, vocab_size=vocab, total_tokens=tokens, latency_ms=latency_ms,
            latency_std_ms=std_ms, warmup_iterations=self.warmup, repeat_iterations=self.repeat,
            tokens_per_sec=(tokens / latency_ms * 1e3) if finite else 0.0,
            tflops=(flops / latency_ms / 1e9) if finite else 0.0, peak_vram_gb=peak_gb,
            peak_vram_reduction_gb=reduction_gb, status=status, notes=notes, extra=dict(extra or {}),
        )
        self._metrics.append(m)
        return m

    # -- one-call profiling of a user's callable (the reference's ``profile_logp`` / ``profile_sampling``) ------
    def profile_logp(self, candidate_fn: Callable[[], Any], batch_size: int, seq_len: int, vocab_size: int,
                     benchmark_name: str = "logp_forward", native_fn: Optional[Callable[[], Any]] = None) -> BenchmarkMetrics:
        """Times ``candidate_fn`` (a selected-token log-prob over ``[B, S, V]`` logits), measures its peak memory and,
        when ``native_fn`` is given, how much less memory it needs than that baseline."""
        _, ms, std = self.time_fn(candidate_fn)
        peak = self.peak_memory_gb(candidate_fn)
        saved = None if native_fn is None else self.peak_memory_gb(native_fn) - peak
        return self.record(benchmark_name, batch_size, seq_len, vocab_size, ms, std,
                           self.estimate_logp_tflops(batch_size, seq_len, vocab_size) * 1e12, peak, reduction_gb=saved)

    def profile_sampling(self, candidate_fn: Callable[[], Any], batch_size: int, vocab_size: int, seq_len: int = 1,
                         benchmark_name: str = "sampling_step") -> BenchmarkMetrics:
        """Times one sampling step over ``[B, V]`` logits and records it."""
        _, ms, std = self.time_fn(candidate_fn)
        return self.record(benchmark_name, batch_size, seq_len, vocab_size, ms, std,
                           self.estimate_sampling_tflops(batch_size, vocab_size) * 1e12, self.peak_memory_gb(candidate_fn))

    def blocked(self, name: str, batch: int, seq: int, vocab: int, exc: Exception) -> BenchmarkMetrics:
        first = (str(exc).splitlines() or [type(exc).__name__])[0]
        return self.record(name, batch, seq, vocab, float("inf"), None, status="blocked", notes=first)

    def get_metrics(self) -> List[BenchmarkMetrics]:
        return list(self._metrics)

    def clear_metrics(self) -> None:
        self._metrics.clear()

    # -- reports ------------------------------------------------------------------------------------
    def save_json(self, path) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        payload = {
            "report_version": "1.0",
            "generated_at": datetime.now(timezone.utc).isoformat(),
            "gpu_target": asdict(self.gpu_info),
            "metrics": [m.to_dict() for m in self._metrics],
        }
        path.write_text(json.dumps(payload, indent=2))

    def save_csv(self, path) -> None:
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        if not self._metrics:
            return
        rows = []
        for m in self._metrics:
            row = m.to_dict()
            for k, v in row.pop("gpu_target").items():
                row[f"gpu_{k}"] = v
            for k, v in row.pop("extra", {}).items():
                row[f"extra_{k}"] = v
            rows.append(row)
        fields = sorted({k for r in rows for k in r})
        new = not (path.exists() and path.stat().st_size > 0)
        with path.open("a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=fields)
            if new:
                w.writeheader()
            w.writerows(rows)

    def print_summary(self) -> None:
        from tabulate import tabulate

        table = [[m.benchmark_name, m.batch_size, m.seq_len, m.vocab_size, f"{m.latency_ms:.3f}",
                  f"{m.tokens_per_sec:,.0f}", f"{m.tflops:.1f}", f"{m.peak_vram_gb:.3f}", m.status, m.notes[:60]]
                 for m in self._metrics]
        print(tabulate(table, headers=["workload", "batch", "seq", "vocab", "ms", "tokens/s", "TFLOP/s", "peak GB",
                                       "status", "notes"]))


# ---------------------------------------------------------------------------------------------------
# Workloads.  Each runner takes (profiler, args, device, dtype, batch, seq, vocab) and records one metric.
# "native" = the PyTorch oracle path; "fused" = the registry's sm_100a kernels.
# ---------------------------------------------------------------------------------------------------
def _rand_logits(device, dtype, batch, seq, vocab, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(batch, seq, vocab, device=device, generator=g, dtype=torch.float32).to(dtype)


def _ids(device, batch, seq, vocab, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randint(0, vocab, (batch, seq), device=device, generator=g)


def _logp_flops(batch, seq, vocab):
    return 5.0 * batch * seq * vocab  # max, subtract, exp, sum, gather-subtract per element (rough)


def _fused(op):
    """A ``*_fused`` workload measures the sm_100a kernels.  If the registry handed out a PyTorch fallback (no GPU, no
    extension) the workload is reported as ``blocked`` instead of timing the wrong thing under the fused name."""
    if type(op).__name__.startswith("Native"):
        raise RuntimeError(f"fused backend unavailable: the registry dispatched {type(op).__name__}")
    return op


def _guard(name):
    def deco(fn):
        def run(profiler, args, device, dtype, batch, seq, vocab):
            try:
                return fn(profiler, args, device, dtype, batch, seq, vocab)
            except Exception as exc:  # recorded, never fatal
                if device.type == "cuda":
                    torch.cuda.empty_cache()
                return profiler.blocked(name, batch, seq, vocab, exc)
        run.__name__ = fn.__name__
        return run
    return deco


@_guard("logp_native")
def _run_logp_native(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.testing import selected_logprobs_reference

    logits, ids = _rand_logits(device, dtype, batch, seq, vocab, args.seed), _ids(device, batch, seq, vocab, args.seed + 1)
    fn = lambda: selected_logprobs_reference(logits, ids)
    _, ms, std = profiler.time_fn(fn)
    return profiler.record("logp_native", batch, seq, vocab, ms, std, _logp_flops(batch, seq, vocab), profiler.peak_memory_gb(fn))


@_guard("logp_fused")
def _run_logp_fused(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.registry import kernel_registry
    from rl_engine.testing import selected_logprobs_reference

    op = _fused(kernel_registry.get_op("logp"))
    logits, ids = _rand_logits(device, dtype, batch, seq, vocab, args.seed), _ids(device, batch, seq, vocab, args.seed + 1)
    fn = lambda: op.apply_fp32(logits, ids)
    out, ms, std = profiler.time_fn(fn)
    ref_fn = lambda: selected_logprobs_reference(logits, ids)
    err = float((out.float().reshape(-1) - ref_fn().float().reshape(-1)).abs().max())
    peak, ref_peak = profiler.peak_memory_gb(fn), profiler.peak_memory_gb(ref_fn)
    return profiler.record("logp_fused", batch, seq, vocab, ms, std, _logp_flops(batch, seq, vocab), peak,
                           extra={"max_abs_err": err, "backend": type(op).__name__, "bytes": logits.numel() * logits.element_size()},
                           reduction_gb=ref_peak - peak)


@_guard("linear_logp_fused")
def _run_linear_logp_fused(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.registry import kernel_registry

    op = _fused(kernel_registry.get_op("linear_logp"))
    hidden = args.hidden
    g = torch.Generator(device=device).manual_seed(args.seed)
    h = torch.randn(batch * seq, hidden, device=device, generator=g).to(dtype)
    w = (torch.randn(vocab, hidden, device=device, generator=g) * 0.02).to(dtype)
    t = _ids(device, batch, seq, vocab, args.seed + 1).reshape(-1)
    fn = lambda: op(h, w, t)
    _, ms, std = profiler.time_fn(fn)
    logits_gb = batch * seq * vocab * 4 / 2**30
    peak = profiler.peak_memory_gb(fn)
    return profiler.record("linear_logp_fused", batch, seq, vocab, ms, std, 2.0 * batch * seq * hidden * vocab, peak,
                           extra={"hidden": hidden, "backend": type(op).__name__}, reduction_gb=logits_gb - peak)


@_guard("linear_logp_native")
def _run_linear_logp_native(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.ops.pytorch.loss.linear_logp import NativeLinearLogpOp

    op = NativeLinearLogpOp()
    hidden = args.hidden
    g = torch.Generator(device=device).manual_seed(args.seed)
    h = torch.randn(batch * seq, hidden, device=device, generator=g).to(dtype)
    w = (torch.randn(vocab, hidden, device=device, generator=g) * 0.02).to(dtype)
    t = _ids(device, batch, seq, vocab, args.seed + 1).reshape(-1)
    fn = lambda: op(h, w, t)
    _, ms, std = profiler.time_fn(fn)
    return profiler.record("linear_logp_native", batch, seq, vocab, ms, std, 2.0 * batch * seq * hidden * vocab,
                           profiler.peak_memory_gb(fn), extra={"hidden": hidden})


def _sampling(profiler, args, device, dtype, batch, seq, vocab, name, fused):
    from rl_engine.kernels.sampling import SamplerBackend

    sampler = SamplerBackend(seed=args.seed)
    if fused and sampler.backend != "sm100":
        raise RuntimeError(f"fused sampler unavailable: backend is {sampler.backend}")
    if not fused:
        sampler.backend = "torch"
    rows = batch * seq
    logits = _rand_logits(device, torch.float32, 1, rows, vocab, args.seed)[0]
    fn = lambda: sampler.sample(logits, top_k=args.top_k, top_p=args.top_p, temperature=1.0)
    out, ms, std = profiler.time_fn(fn)
    assert out.shape[0] == rows
    return profiler.record(name, batch, seq, vocab, ms, std, 4.0 * rows * vocab, profiler.peak_memory_gb(fn),
                           extra={"top_k": args.top_k, "top_p": args.top_p, "backend": sampler.backend})


@_guard("sampling_native")
def _run_sampling_native(profiler, args, device, dtype, batch, seq, vocab):
    return _sampling(profiler, args, device, dtype, batch, seq, vocab, "sampling_native", False)


@_guard("sampling_fused")
def _run_sampling_fused(profiler, args, device, dtype, batch, seq, vocab):
    return _sampling(profiler, args, device, dtype, batch, seq, vocab, "sampling_fused", True)


@_guard("ratio_kl_fused")
def _run_ratio_kl(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.registry import kernel_registry

    op = _fused(kernel_registry.get_op("ratio_kl"))
    pol, ref = _rand_logits(device, dtype, batch, seq, vocab, args.seed), _rand_logits(device, dtype, batch, seq, vocab, args.seed + 2)
    ids = _ids(device, batch, seq, vocab, args.seed + 1)
    mask = torch.ones(batch, seq, device=device, dtype=torch.bool)
    old = torch.full((batch, seq), -5.0, device=device)
    fn = lambda: op(pol, ref, ids, mask, old)
    _, ms, std = profiler.time_fn(fn)
    return profiler.record("ratio_kl_fused", batch, seq, vocab, ms, std, 10.0 * batch * seq * vocab, profiler.peak_memory_gb(fn),
                           extra={"backend": type(op).__name__, "bytes": 2 * pol.numel() * pol.element_size()})


@_guard("grpo_loss_fused")
def _run_grpo_loss(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.registry import kernel_registry

    op = _fused(kernel_registry.get_op("grpo_loss"))
    pol = _rand_logits(device, dtype, batch, seq, vocab, args.seed).requires_grad_(True)
    ref = _rand_logits(device, dtype, batch, seq, vocab, args.seed + 2)
    ids = _ids(device, batch, seq, vocab, args.seed + 1)
    mask = torch.ones(batch, seq, device=device, dtype=torch.bool)
    old = torch.full((batch, seq), -5.0, device=device)
    rewards = torch.randn(batch, device=device)

    def fn():
        pol.grad = None
        loss, _, _ = op(pol, ref, ids, old, rewards, mask, samples_per_prompt=batch, beta=0.04)
        loss.backward()
        return loss

    _, ms, std = profiler.time_fn(fn)
    return profiler.record("grpo_loss_fused", batch, seq, vocab, ms, std, 20.0 * batch * seq * vocab, profiler.peak_memory_gb(fn),
                           extra={"backend": type(op).__name__, "includes": "forward + backward"})


@_guard("attention_fused")
def _run_attention(profiler, args, device, dtype, batch, seq, vocab):
    from rl_engine.kernels.registry import kernel_registry

    op = _fused(kernel_registry.get_op("attn"))
    g = torch.Generator(device=device).manual_seed(args.seed)
    q = torch.randn(batch, seq, 32, 128, device=device, generator=g).to(dtype)
    k = torch.randn(batch, seq, 8, 128, device=device, generator=g).to(dtype)
    v = torch.randn(batch, seq, 8, 128, device=device, generator=g).to(dtype)
    fn = lambda: op(q, k, v, causal=True)
    _, ms, std = profiler.time_fn(fn)
    return profiler.record("attention_fused", batch, seq, vocab, ms, std, 2.0 * batch * 32 * 128 * seq * seq,
                           profiler.peak_memory_gb(fn), extra={"heads": "32q/8kv", "head_dim": 128, "causal": True})


WORKLOAD_REGISTRY: Dict[str, Callable] = {
    "logp_native": _run_logp_native,
    "logp_fused": _run_logp_fused,
    "linear_logp_native": _run_linear_logp_native,
    "linear_logp_fused": _run_linear_logp_fused,
    "sampling_native": _run_sampling_native,
    "sampling_fused": _run_sampling_fused,
    "ratio_kl_fused": _run_ratio_kl,
    "grpo_loss_fused": _run_grpo_loss,
    "attention_fused": _run_attention,
}


def available_workloads() -> Tuple[str, ...]:
    return tuple(WORKLOAD_REGISTRY)


def _parse_int_list(value: str) -> List[int]:
    return [int(x) for x in value.split(",") if x.strip()]


def _parse_dtype(value: str) -> torch.dtype:
    table = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
             "float32": torch.float32, "fp32": torch.float32}
    if value not in table:
        raise ValueError(f"unsupported dtype {value!r}; choose from {sorted(table)}")
    return table[value]


def _parse_workloads(value: str) -> List[str]:
    raw = [x.strip() for x in value.split(",") if x.strip()]
    # the reference's CLI spells workloads with hyphens (``logp-native``); both spellings name the same workload
    unknown = sorted(x for x in set(raw) if x.replace("-", "_") not in WORKLOAD_REGISTRY)
    if unknown:
        raise ValueError(f"unsupported workloads: {', '.join(unknown)}; supported: {', '.join(available_workloads())}")
    return [x.replace("-", "_") for x in raw]


def run_automated_suite(args: argparse.Namespace) -> PerformanceProfiler:
    device = torch.device(args.device)
    dtype = _parse_dtype(args.dtype)
    profiler = PerformanceProfiler(device=device, warmup=args.warmup, repeat=args.repeat)
    if args.smoke:
        batches, seqs, vocabs = [2], [4], [32]
    else:
        batches, seqs, vocabs = _parse_int_list(args.batch_sizes), _parse_int_list(args.seq_lens), _parse_int_list(args.vocab_sizes)
    for b in batches:
        for s in seqs:
            for v in vocabs:
                for name in _parse_workloads(args.workloads):
                    WORKLOAD_REGISTRY[name](profiler, args, device, dtype, b, s, v)
    return profiler


def build_arg_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="rl_engine automated performance profiler")
    p.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--batch-sizes", default="8,16,32")
    p.add_argument("--seq-lens", default="128,512")
    p.add_argument("--vocab-sizes", default="4096,128256")
    p.add_argument("--workloads", default=",".join(available_workloads()),
                   help=f"comma-separated subset of: {', '.join(available_workloads())}")
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--top-k", type=int, default=50)
    p.add_argument("--top-p", type=float, default=0.9)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--repeat", type=int, default=10)
    p.add_argument("--output", type=Path, default=None)
    p.add_argument("--format", choices=["csv", "json"], default="csv")
    p.add_argument("--no-summary", action="store_true")
    p.add_argument("--smoke", action="store_true", help="tiny shapes, fp32, one repetition (runs on CPU too)")
    return p


def main() -> None:
    args = build_arg_parser().parse_args()
    if args.smoke:
        args.dtype, args.warmup, args.repeat, args.hidden = "float32", 0, 1, 16
    profiler = run_automated_suite(args)
    if args.output is not None:
        (profiler.save_json if args.format == "json" else profiler.save_csv)(args.output)
    if not args.no_summary:
        profiler.print_summary()


if __name__ == "__main__":
    main()
