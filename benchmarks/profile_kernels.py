"""Small, self-terminating workloads for per-kernel profiling and CUDA-event timing.

    python benchmarks/profile_kernels.py --kernel gemm            # one of the names below
    ncu --set full --clock-control none -k regex:gemm_sm100 -s 2 -c 1 -o out python benchmarks/profile_kernels.py --kernel gemm

Each case touches more than the 126 MB L2 but at most a few GB, launches the kernel under test a
handful of times, prints one JSON line with the CUDA-event time of the last launch (L2 flushed before
it) and the achieved fraction of the measured peaks in ``MEASURED_PEAKS.json`` when that file exists.
"""

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def timed(fn, launches=3):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ms = 0.0
    for _ in range(launches):
        flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop)
    return ms


def rand(shape, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * scale).to(torch.bfloat16)


def case_gemm():
    from rl_engine.kernels.ops.sm100.gemm import gemm

    m, n, k = 8192, 14336, 4096  # 67 + 117 + 235 MB
    a, b = rand((m, k)), rand((n, k), 0.02, 1)
    ms = timed(lambda: gemm(a, b))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms, "shape": [m, n, k]}


def case_gemm_fp8():
    from rl_engine.kernels.ops.sm100.gemm_fp8 import gemm_fp8, quantize_rows

    m, n, k = 8192, 14336, 4096
    (aq, sa), (bq, sb) = quantize_rows(rand((m, k))), quantize_rows(rand((n, k), 0.02, 1))
    pair = os.environ.get("PROFILE_FP8_PAIR", "1") != "0"
    ms = timed(lambda: gemm_fp8(aq, sa, bq, sb, pair=pair))
    return {"flops": 2.0 * m * n * k, "bytes": 1.0 * (m * k + n * k) + 2.0 * m * n, "ms": ms, "shape": [m, n, k],
            "note": f"e4m3 x e4m3 with row-wise scales, bf16 out, pair={pair}; the fraction is against the bf16 cuBLAS peak"}


def case_quantize_fp8():
    from rl_engine.kernels.ops.sm100.gemm_fp8 import quantize_rows

    m, k = 65536, 4096  # 537 MB in, 268 MB out
    x = rand((m, k))
    ms = timed(lambda: quantize_rows(x))
    return {"flops": 0.0, "bytes": 3.0 * m * k, "ms": ms, "shape": [m, k], "note": "bf16 read twice (amax, convert) is counted once"}


def _decode_case(fp8: bool):
    """One key / value cached decoding step of 4 Llama-3-8B layers: 32 completions at token 256 after a 1024-token
    prompt.  Bytes = the layers' projection weights, which every step streams once."""
    from rl_engine.models.config import llama3_8b
    from rl_engine.models.llama import LlamaModel

    cfg = llama3_8b().with_layers(4)
    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=0, max_positions=2048)
    if fp8:
        model.enable_fp8_inference()
    p, g, lmax, t = 1024, 32, 512, 256
    cache = model.new_kv_cache(p + g * lmax)
    for ck, cv in cache:
        ck.normal_()
        cv.normal_()
    tokens = torch.randint(0, cfg.vocab_size, (g,), device="cuda")
    pos = torch.full((g,), p + t, dtype=torch.long, device="cuda")
    slots = p + torch.arange(g, device="cuda") * lmax + t
    prefix_layout, own_layout = model.decode_layouts(g, p, lmax, t + 1)
    ms = timed(lambda: model.decode_step(tokens, pos, cache, slots, prefix_layout, own_layout))
    per_layer = cfg.hidden_size * (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim * cfg.hidden_size + 3 * cfg.hidden_size * cfg.ffn_size
    return {"flops": 0.0, "bytes": (1.0 if fp8 else 2.0) * per_layer * cfg.num_layers, "ms": ms, "shape": [g, p, t, cfg.num_layers],
            "note": ("fp8" if fp8 else "bf16") + " projections; 4 layers, embedding and final norm included, LM head not"}


def case_decode_step():
    return _decode_case(False)


def case_decode_step_fp8():
    return _decode_case(True)


def case_gemm_wgrad():
    from rl_engine.kernels.ops.sm100.gemm import gemm

    m, n, k = 8192, 14336, 4096
    dy, x = rand((m, n)), rand((m, k), 1.0, 1)
    ms = timed(lambda: gemm(dy, x, a_mn=True, b_mn=True))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms, "shape": [n, k, m]}


def case_gemm_pair():
    from rl_engine.kernels.ops.sm100.gemm import gemm

    m, n, k = 8192, 14336, 4096
    a, b = rand((m, k)), rand((n, k), 0.02, 1)
    ms = timed(lambda: gemm(a, b, pair=True))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms, "shape": [m, n, k],
            "note": "256 x 256 tiles on SM pairs (cta_group::2)"}


def case_gemm_wgrad_pair():
    from rl_engine.kernels.ops.sm100.gemm import gemm

    m, n, k = 8192, 14336, 4096
    dy, x = rand((m, n)), rand((m, k), 1.0, 1)
    ms = timed(lambda: gemm(dy, x, a_mn=True, b_mn=True, pair=True))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms, "shape": [n, k, m],
            "note": "256 x 256 tiles on SM pairs (cta_group::2)"}


def case_gemm_dgrad_pair():
    from rl_engine.kernels.ops.sm100.gemm import gemm

    m, n, k = 8192, 4096, 14336
    dy, w = rand((m, k)), rand((k, n), 0.02, 1)
    ms_pair = timed(lambda: gemm(dy, w, b_mn=True, pair=True))
    ms_single = timed(lambda: gemm(dy, w, b_mn=True, pair=False))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms_pair, "shape": [m, n, k],
            "note": f"B as [K, N]; single-CTA kernel on the same problem: {ms_single:.4f} ms"}


def case_gemm_shape():
    """Any GEMM: PROFILE_GEMM="M,N,K,layout,pair" with layout in nt|nn|tn|tt (A then B; t = MN-major) and pair 0|1."""
    from rl_engine.kernels.ops.sm100.gemm import gemm

    spec = os.environ.get("PROFILE_GEMM", "8192,4096,28672,nn,1").split(",")
    m, n, k = int(spec[0]), int(spec[1]), int(spec[2])
    a_mn, b_mn, pair = spec[3][0] == "t", spec[3][1] == "n", spec[4] == "1"
    a = rand((k, m) if a_mn else (m, k))
    b = rand((k, n) if b_mn else (n, k), 0.02, 1)
    ms = timed(lambda: gemm(a, b, a_mn=a_mn, b_mn=b_mn, pair=pair))
    return {"flops": 2.0 * m * n * k, "bytes": 2.0 * (m * k + n * k + m * n), "ms": ms, "shape": [m, n, k],
            "note": f"layout {spec[3]} (A {'MN' if a_mn else 'K'}-major, B {'MN' if b_mn else 'K'}-major), pair={int(pair)}"}


def case_tp_ag_gemm():
    """The fused all-gather -> GEMM kernel on ONE rank: the copy warps feed this GPU's own gathered buffer, so the
    kernel (copy warps + arrival counters + waiting TMA producer) can be captured without a multi-rank launch."""
    from rl_engine.parallel.tp_linear import TensorParallelLinears

    tp = TensorParallelLinears()
    t, h, n = 16384, 4096, 7168
    x, w = rand((t, h)), rand((n, h), 0.02, 1)
    ms = timed(lambda: tp.ag_gemm(x, w))
    return {"flops": 2.0 * t * h * n, "bytes": 2.0 * (2 * t * h + n * h + t * n), "ms": ms, "shape": [t, n, h],
            "note": "world = 1: gathered rows are written and read locally"}


def case_tp_gemm_rs():
    from rl_engine.parallel.tp_linear import TensorParallelLinears

    tp = TensorParallelLinears()
    t, h, k = 16384, 4096, 7168
    a, w = rand((t, k)), rand((h, k), 0.02, 1)
    ms = timed(lambda: tp.gemm_rs(a, w))
    return {"flops": 2.0 * t * h * k, "bytes": 2.0 * (t * k + h * k + 3 * t * h), "ms": ms, "shape": [t, h, k],
            "note": "world = 1: one partial slab, written by the epilogue and summed by the in-kernel reduce phase"}


def case_zero1_step():
    """Fused reduce-scatter + AdamW + all-gather kernel on ONE rank (the peer lists hold this GPU's own buffers)."""
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.parallel.symmetric import SymmetricMemory

    ext = require_ext()
    n = 1 << 28  # 268 M parameters: 0.5 GB of bf16 params + grads, 3 GB of fp32 state
    mem = SymmetricMemory(4 * n + (1 << 20))
    params, grads = mem.alloc((n,), torch.bfloat16), mem.alloc((n,), torch.bfloat16)
    params.local.normal_()
    grads.local.normal_()
    m, v, master = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda"), params.local.float()
    step = [0]

    def run():
        step[0] += 1
        ext.zero1_fused_step(grads.ptrs, params.ptrs, 0, n, m, v, master, 1e-6, 0.9, 0.95, 1e-8, 0.0, step[0], 1.0, 0, None, 0)

    ms = timed(run)
    return {"flops": 0.0, "bytes": n * (2.0 + 2.0 + 3 * 4 * 2), "ms": ms, "shape": [n],
            "note": "world = 1; bytes = grad read + param write + fp32 master/m/v read and write"}


def case_cast_broadcast():
    from rl_engine.kernels.ops.base import require_ext
    from rl_engine.parallel.symmetric import SymmetricMemory

    ext = require_ext()
    n = 1 << 28
    mem = SymmetricMemory(2 * n + (1 << 20))
    window = mem.alloc((n,), torch.bfloat16)
    src = torch.randn(n, device="cuda")
    ms = timed(lambda: ext.cast_broadcast(src, window.ptrs, 1))
    return {"flops": 0.0, "bytes": n * 6.0, "ms": ms, "shape": [n], "note": "world = 1: fp32 read, bf16 write into the local window"}


def case_moe_layer():
    """One Qwen3-30B-A3B-shaped MoE layer, forward + backward, single GPU (all 128 experts local)."""
    from rl_engine.kernels.ops.sm100.moe import FusedMoESM100Op

    e, k, h, f, t = 128, 8, 2048, 768, 8192
    x = rand((t, h)).requires_grad_(True)
    router = rand((e, h), 1 / 45, 1).requires_grad_(True)
    w1 = rand((e * 2 * f, h), 0.02, 2).requires_grad_(True)
    w2 = rand((e * h, f), 0.02, 3).requires_grad_(True)
    do = rand((t, h), 1.0, 4)
    op = FusedMoESM100Op()

    def run():
        x.grad = router.grad = w1.grad = w2.grad = None
        op(x, router, w1, w2, k).backward(do)

    ms = timed(run)
    return {"flops": 3.0 * 2.0 * t * k * (h * 2 * f + f * h), "bytes": 0.0, "ms": ms, "shape": [t, h, e, k, f],
            "note": "router + top-8 + plan kernels + gather + grouped GEMMs + SwiGLU + combine, forward and backward"}


def case_linear_logp():
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    n, d, v = 8192, 4096, 128256  # weight 1.05 GB
    h, w = rand((n, d)), rand((v, d), 0.02, 1)
    t = torch.randint(0, v, (n,), device="cuda")
    op = FusedLinearLogpSM100Op(check_targets=False)
    ms = timed(lambda: op(h, w, t))
    return {"flops": 2.0 * n * d * v, "bytes": 2.0 * (n * d + v * d), "ms": ms, "shape": [n, d, v]}


def case_linear_logp_bwd():
    from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op

    n, d, v = 4096, 4096, 128256
    h, w = rand((n, d)).requires_grad_(True), rand((v, d), 0.02, 1).requires_grad_(True)
    t = torch.randint(0, v, (n,), device="cuda")
    op = FusedLinearLogpSM100Op(check_targets=False)

    def run():
        h.grad = w.grad = None
        op(h, w, t).sum().backward()

    ms = timed(run, launches=2)
    return {"flops": 8.0 * n * d * v, "bytes": 0.0, "ms": ms, "shape": [n, d, v], "note": "forward + recompute backward"}


def _attn_inputs(prompt=1024, group=32, length=512, hq=32, hkv=8):  # Q + O = 285 MB > L2
    t = prompt + group * length
    return rand((t, hq, 128)), rand((t, hkv, 128), 1.0, 1), rand((t, hkv, 128), 1.0, 2), prompt, group, length


def _attn_flops(prompt, group, length, hq):
    keys = group * length * prompt + group * length * (length + 1) / 2 + prompt * (prompt + 1) / 2
    return 4.0 * hq * 128 * keys


def case_attention_fwd():
    from rl_engine.kernels.ops.sm100.attention import grpo_group_layout, packed_attention_forward

    q, k, v, p, g, l = _attn_inputs()
    layout = grpo_group_layout(p, g, l, "cuda")
    ms = timed(lambda: packed_attention_forward(q, k, v, layout))
    return {"flops": _attn_flops(p, g, l, 32), "bytes": 2.0 * (2 * q.numel() + 2 * k.numel()), "ms": ms, "shape": [p, g, l]}


def case_attention_bwd():
    from rl_engine.kernels.ops.sm100.attention import grpo_group_layout, packed_attention_forward
    from rl_engine.kernels.ops.sm100.attention_bwd_kernels import fused_backward

    q, k, v, p, g, l = _attn_inputs()
    layout = grpo_group_layout(p, g, l, "cuda")
    out, lse = packed_attention_forward(q, k, v, layout)
    dout = rand(tuple(q.shape), 1.0, 3)
    ms = timed(lambda: fused_backward(q, k, v, out, lse, dout, layout, 128**-0.5))
    return {"flops": 3.5 * _attn_flops(p, g, l, 32), "bytes": 0.0, "ms": ms, "shape": [p, g, l],
            "note": "dQ kernel (3 GEMMs / tile) + dK,dV kernel (4 GEMMs / tile)"}


def case_logp_rows():
    from rl_engine.kernels.ops.sm100.logp import FusedLogpSM100Op

    rows, v = 4096, 128256  # 1.05 GB of bf16 logits
    logits = rand((rows, v))
    ids = torch.randint(0, v, (rows,), device="cuda")
    op = FusedLogpSM100Op()
    ms = timed(lambda: op.apply_fp32(logits, ids))
    return {"flops": 0.0, "bytes": 2.0 * rows * v, "ms": ms, "shape": [rows, v]}


def case_swiglu():
    from rl_engine.kernels.ops.sm100.model_ops import swiglu_packed

    rows, f = 16384, 14336
    gu = rand((rows, 2 * f))
    ms = timed(lambda: swiglu_packed(gu))
    return {"flops": 0.0, "bytes": 2.0 * rows * 3 * f, "ms": ms, "shape": [rows, f]}


def case_rmsnorm():
    from rl_engine.kernels.ops.sm100.model_ops import FusedRMSNormSM100Op

    rows, d = 65536, 4096
    x, w = rand((rows, d)), rand((d,), 1.0, 1)
    op = FusedRMSNormSM100Op()
    ms = timed(lambda: op(x, w))
    return {"flops": 0.0, "bytes": 2.0 * rows * d * 2, "ms": ms, "shape": [rows, d]}


def case_sampler():
    from rl_engine.kernels.ops.sm100.sampler import sample_topk_topp

    logits = rand((256, 151936)).float()
    ms = timed(lambda: sample_topk_topp(logits, top_k=50, top_p=0.9, temperature=0.7, seed=1, offset=0))
    return {"flops": 0.0, "bytes": 4.0 * 256 * 151936, "ms": ms, "shape": [256, 151936],
            "note": "bytes = one pass over the logits; the kernel reads each row twice (thread maxima from DRAM, gather "
                    "from L2)"}


def case_adamw():
    """Fused AdamW on bf16 parameters with fp32 masters kept as 16-bit residuals (one GPU's optimiser step)."""
    from rl_engine.kernels.ops.base import require_ext

    n = 1 << 28  # 0.27 G parameters: 0.5 GB of weights, 3.8 GB touched per step
    p, g = rand((n,), 0.02), rand((n,), 1.0, 1)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    residual = torch.zeros(n, dtype=torch.int16, device="cuda")
    step = [0]

    def run():
        step[0] += 1
        require_ext().adamw(p, residual, g, m, v, 1e-6, 0.9, 0.95, 1e-8, 0.0, step[0], 1.0)

    ms = timed(run)
    # read p, g, residual (2 B each) and m, v (4 B each); write p, residual, m, v
    return {"flops": 0.0, "bytes": n * (2.0 + 2 + 2 + 4 + 4 + 2 + 2 + 4 + 4), "ms": ms, "shape": [n],
            "note": "bf16 parameter + int16 residual = exact fp32 master; bytes = all reads and writes"}


def case_weight_digest():
    """One-pass integrity digest of a weight tensor (64-bit position-weighted sum)."""
    from rl_engine.kernels.ops.base import require_ext

    n = 1 << 29  # 1 GB of bf16
    t = rand((n,), 0.02)
    out = torch.zeros(4, dtype=torch.int64, device="cuda")
    ms = timed(lambda: require_ext().weight_digest(t, out, 0))
    return {"flops": 0.0, "bytes": 2.0 * n, "ms": ms, "shape": [n]}


def case_ratio_kl():
    """Policy and reference logits streamed side by side (ratio / KL front end)."""
    from rl_engine.kernels.registry import kernel_registry

    b, t, v = 16, 512, 131072
    pol, ref = rand((b, t, v)), rand((b, t, v), 1.0, 1)
    ids = torch.randint(0, v, (b, t), device="cuda")
    mask = torch.ones(b, t, dtype=torch.bool, device="cuda")
    old = torch.zeros(b, t, device="cuda")
    op = kernel_registry.get_op("ratio_kl")

    def run():
        with torch.no_grad():
            op(pol, ref, ids, mask, old)

    ms = timed(run)
    return {"flops": 0.0, "bytes": 2.0 * 2 * b * t * v, "ms": ms, "shape": [b, t, v]}


CASES = {name[5:]: fn for name, fn in globals().items() if name.startswith("case_")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel", default="all", help="one name, a comma-separated list, or 'all' of: " + ", ".join(sorted(CASES)))
    args = ap.parse_args()
    names = sorted(CASES) if args.kernel == "all" else [k.strip() for k in args.kernel.split(",") if k.strip()]
    unknown = [k for k in names if k not in CASES]
    if unknown:
        ap.error(f"unknown kernels {unknown}; choose from {sorted(CASES)}")
    pk = peaks()
    for name in names:
        r = CASES[name]()
        line = {"kernel": name, "ms": round(r["ms"], 4), "shape": r["shape"], "peaks": pk["source"]}
        if r["flops"]:
            line["tflops"] = round(r["flops"] / r["ms"] / 1e9, 1)
            line["frac_of_bf16_peak"] = round(line["tflops"] / pk["bf16_tflops"], 3)
        if r["bytes"]:
            line["gbs"] = round(r["bytes"] / r["ms"] / 1e6, 1)
            line["frac_of_hbm_peak"] = round(line["gbs"] / pk["hbm_gbs"], 3)
        if "note" in r:
            line["note"] = r["note"]
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
