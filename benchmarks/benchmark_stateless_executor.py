"""Stateless reference / reward scoring (no KV cache is ever allocated) vs a generation-style paged-KV
reservation.  Counterpart of the reference's ``benchmarks/benchmark_stateless_executor.py``: one CSV row
per run (appended) and the same row as JSON on stdout.

    python benchmarks/benchmark_stateless_executor.py --mode both --compare-paged-kv --device cuda
    python benchmarks/benchmark_stateless_executor.py --smoke
"""

import argparse
import csv
import json
from pathlib import Path

import torch

import common  # noqa: F401  (puts the repository root on sys.path)

DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


class ToyCausalLM(torch.nn.Module):
    """Embedding -> two-layer MLP -> vocabulary head + scalar reward head; accepts and honours ``use_cache``."""

    def __init__(self, vocab: int, hidden: int) -> None:
        super().__init__()
        self.embed = torch.nn.Embedding(vocab, hidden)
        self.mlp = torch.nn.Sequential(torch.nn.Linear(hidden, 2 * hidden), torch.nn.SiLU(), torch.nn.Linear(2 * hidden, hidden))
        self.head = torch.nn.Linear(hidden, vocab, bias=False)
        self.value = torch.nn.Linear(hidden, 1)

    def forward(self, input_ids, attention_mask=None, use_cache=False, **_):
        h = self.embed(input_ids)
        h = h + self.mlp(h)
        out = {"logits": self.head(h), "rewards": self.value(h[:, -1]).squeeze(-1)}
        if use_cache:
            out["past_key_values"] = ((h.detach(), h.detach()),)
        return out


def build_inputs(args, device):
    from rl_engine.executors.stateless_executor import StatelessForwardInputs

    g = torch.Generator().manual_seed(args.seed)
    ids = torch.randint(0, args.vocab_size, (args.batch_size, args.seq_len), generator=g).to(device)
    attn = torch.ones_like(ids, dtype=torch.bool)
    comp = torch.zeros_like(attn)
    comp[:, -args.completion_len:] = torch.rand(args.batch_size, args.completion_len, generator=g).to(device) < args.valid_density
    comp[:, -1] = True
    return StatelessForwardInputs(input_ids=ids, attention_mask=attn, completion_mask=comp)


def run(args) -> dict:
    from rl_engine.executors.paged_kv_baseline import PagedKVScoringBaseline, PagedKVScoringConfig
    from rl_engine.executors.stateless_executor import StatelessForwardConfig, StatelessForwardExecutor

    device = torch.device(args.device)
    torch.manual_seed(args.seed)
    model = ToyCausalLM(args.vocab_size, args.hidden_dim).to(device).eval()
    inputs = build_inputs(args, device)
    mode = "reference" if args.mode == "paged-kv-compare" else args.mode
    executor = StatelessForwardExecutor(model, StatelessForwardConfig(mode=mode, attention_backend="model_default"))
    executor.score(inputs)  # warm-up
    result = executor.score(inputs)
    row = {"benchmark": "stateless_executor", "mode": args.mode, "device": str(device), "batch_size": args.batch_size,
           "seq_len": args.seq_len, "completion_len": args.completion_len, "vocab_size": args.vocab_size,
           "hidden_dim": args.hidden_dim}
    row.update({f"stateless_{k}": v for k, v in result.metrics.items() if isinstance(v, (int, float, str, bool))})
    if args.compare_paged_kv or args.mode == "paged-kv-compare":
        cfg = PagedKVScoringConfig(mode=mode, num_layers=args.paged_kv_layers, num_kv_heads=args.paged_kv_heads,
                                   head_dim=args.paged_kv_head_dim, block_size=args.paged_kv_block_size,
                                   kv_cache_dtype=DTYPES[args.paged_kv_dtype], kv_cache_blocks=args.paged_kv_blocks)
        baseline = PagedKVScoringBaseline(model, cfg)
        baseline.score(inputs)
        paged = baseline.score(inputs)
        row.update({f"paged_{k}": v for k, v in paged.metrics.items() if isinstance(v, (int, float, str, bool))})
        if result.reference_logps is not None and paged.reference_logps is not None:
            row["max_abs_logp_diff"] = float((result.reference_logps - paged.reference_logps).abs().max())
    return row


def main() -> None:
    ap = argparse.ArgumentParser(description="stateless reference / reward executor benchmark")
    ap.add_argument("--mode", choices=["reference", "reward", "both", "paged-kv-compare"], default="reference")
    ap.add_argument("--smoke", action="store_true")
    ap.add_argument("--compare-paged-kv", action="store_true")
    ap.add_argument("--batch-size", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--completion-len", type=int, default=256)
    ap.add_argument("--vocab-size", type=int, default=4096)
    ap.add_argument("--hidden-dim", type=int, default=256)
    ap.add_argument("--paged-kv-layers", type=int, default=4)
    ap.add_argument("--paged-kv-heads", type=int, default=8)
    ap.add_argument("--paged-kv-head-dim", type=int, default=32)
    ap.add_argument("--paged-kv-block-size", type=int, default=16)
    ap.add_argument("--paged-kv-blocks", type=int, default=None)
    ap.add_argument("--paged-kv-dtype", choices=sorted(DTYPES), default="float16")
    ap.add_argument("--valid-density", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=47)
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--output", type=Path, default=None, help="CSV file to append the row to")
    ap.add_argument("--json-output", type=Path, default=None)
    args = ap.parse_args()
    if args.smoke:
        args.batch_size, args.seq_len, args.completion_len = min(args.batch_size, 2), min(args.seq_len, 16), min(args.completion_len, 8)
        args.vocab_size, args.hidden_dim = min(args.vocab_size, 128), min(args.hidden_dim, 32)
        args.paged_kv_layers, args.paged_kv_heads, args.paged_kv_head_dim = 2, 2, 8
    if not 0 < args.completion_len < args.seq_len:
        raise ValueError("completion-len must be greater than zero and less than seq-len")
    if not 0.0 < args.valid_density <= 1.0:
        raise ValueError("valid-density must be in (0, 1]")
    row = run(args)
    if args.output is not None:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        new = not args.output.exists()
        with args.output.open("a", newline="") as f:
            w = csv.DictWriter(f, fieldnames=sorted(row))
            if new:
                w.writeheader()
            w.writerow(row)
    if args.json_output is not None:
        args.json_output.parent.mkdir(parents=True, exist_ok=True)
        args.json_output.write_text(json.dumps(row, indent=2, sort_keys=True))
    print(json.dumps(row, indent=2, sort_keys=True))


if __name__ == "__main__":
    main()
