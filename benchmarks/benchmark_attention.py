"""Attention kernels: causal self-attention (the registry's ``attn`` op) and the GRPO shared-prefix
layout, forward and backward, vs PyTorch SDPA.  Counterpart of the reference's ``benchmarks/benchmark_attention.py``.

    python benchmarks/benchmark_attention.py --prompt 1024 --group 16 --completion 512
"""

import argparse

import torch

from common import randn, report, time_ms


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--group", type=int, default=16)
    ap.add_argument("--completion", type=int, default=512)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--repeat", type=int, default=10)
    args = ap.parse_args()
    from rl_engine.kernels.ops.sm100.attention import grouped_prefix_attention
    from rl_engine.kernels.registry import kernel_registry

    p, g, l, hq, hkv = args.prompt, args.group, args.completion, args.heads, args.kv_heads
    t = p + g * l
    q = randn((t, hq, 128)).requires_grad_(True)
    k = randn((t, hkv, 128), seed=1).requires_grad_(True)
    v = randn((t, hkv, 128), seed=2).requires_grad_(True)
    do = randn((t, hq, 128), seed=3)
    visible = g * l * p + g * l * (l + 1) / 2 + p * (p + 1) / 2
    fwd_flops = 4.0 * hq * 128 * visible

    def fwd():
        with torch.no_grad():
            grouped_prefix_attention(q, k, v, p, g, l)

    def fwd_bwd():
        q.grad = k.grad = v.grad = None
        grouped_prefix_attention(q, k, v, p, g, l).backward(do)

    shape = {"prompt": p, "group": g, "completion": l, "heads": f"{hq}q/{hkv}kv"}
    report("prefix_group_attention_fwd", shape, time_ms(fwd, args.warmup, args.repeat), flops=fwd_flops)
    report("prefix_group_attention_fwd_bwd", shape, time_ms(fwd_bwd, args.warmup, args.repeat), flops=3.5 * fwd_flops)

    # the same tokens as G independent causal sequences of length prompt + completion (what a framework
    # without prefix sharing computes), through the registry's attn op and through SDPA
    s = p + l
    qb, kb, vb = randn((g, s, hq, 128)), randn((g, s, hkv, 128), seed=1), randn((g, s, hkv, 128), seed=2)
    op = kernel_registry.get_op("attn")
    dense_flops = 4.0 * hq * 128 * g * s * (s + 1) / 2
    report("causal_attention_unshared_fwd", {"batch": g, "seq": s}, time_ms(lambda: op(qb, kb, vb, causal=True), args.warmup, args.repeat),
           flops=dense_flops, backend=type(op).__name__)
    qs, ks, vs = (x.transpose(1, 2) for x in (qb, kb, vb))
    sdpa = lambda: torch.nn.functional.scaled_dot_product_attention(qs, ks, vs, is_causal=True, enable_gqa=True)
    try:
        report("causal_attention_sdpa_fwd", {"batch": g, "seq": s}, time_ms(sdpa, args.warmup, args.repeat), flops=dense_flops)
    except Exception as exc:
        print({"benchmark": "causal_attention_sdpa_fwd", "status": "blocked", "notes": str(exc).splitlines()[0]})


if __name__ == "__main__":
    main()
