"""Multi-GPU checks (skipped with fewer than two GPUs) and the single-GPU bounded-wait test."""

import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_wait_is_bounded_and_reports():
    """A barrier whose peer never arrives must return within its limit and leave the context usable."""
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")
    absent_peer = torch.zeros(64, dtype=torch.int32, device="cuda")  # nothing ever raises its flag for us
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    ext.peer_barrier([mine.data_ptr(), absent_peer.data_ptr()], 0, 1, 30.0, err)
    stop.record()
    torch.cuda.synchronize()
    assert 20.0 < start.elapsed_time(stop) < 2000.0
    code, kernel, _block, site = err.tolist()
    assert code == 2 and kernel == 300 and site == 1
    # the context is still healthy
    assert float((torch.ones(8, device="cuda") * 2).sum()) == 16.0


def test_symmetric_memory_single_rank_and_timeout_error():
    from rl_engine.parallel.symmetric import SymmetricMemory

    mem = SymmetricMemory(1 << 20)
    a = mem.alloc((256,), torch.float32)
    b = mem.alloc((3, 5), torch.bfloat16)
    assert a.local.data_ptr() % 256 == 0 and b.local.data_ptr() % 256 == 0 and b.local.shape == (3, 5)
    a.local.fill_(3.0)
    mem.barrier()
    mem.check()
    assert float(a.peer(0).sum()) == 768.0
    with pytest.raises(MemoryError):
        mem.alloc((1 << 30,), torch.float32)
    mem.close()


@pytest.mark.parametrize("dtype,numel", [(torch.bfloat16, 1), (torch.bfloat16, 3), (torch.float32, 5), (torch.uint8, 23),
                                         (torch.bfloat16, 8 * 1000 + 4), (torch.float32, 1 << 20), (torch.int64, 7)])
def test_weight_digest_kernel_matches_the_tensor_op_form(dtype, numel):
    """The one-pass digest kernel and the plain tensor-op formula give the same 64 bits, for tails of 1..7 bytes, an
    odd word count, and a size that spans many blocks; a single flipped bit or two swapped words change the digest."""
    from rl_engine.executors.weight_sync.protocol import _dev64_reference, tensor_digest, tensor_digests

    g = torch.Generator(device="cuda").manual_seed(numel)
    raw = torch.randint(0, 256, (numel * torch.empty((), dtype=dtype).element_size(),), device="cuda", generator=g,
                        dtype=torch.uint8)
    t = raw.view(dtype)
    want = _dev64_reference(t)
    got = tensor_digest(t)
    assert got == f"dev64:{want:016x}:{(raw.numel() + 7) // 8 * 8}"
    flipped = raw.clone()
    flipped[raw.numel() // 2] ^= 1
    assert tensor_digest(flipped.view(dtype)) != got
    if raw.numel() >= 24:
        swapped = raw.clone()
        swapped[:8], swapped[8:16] = raw[8:16], raw[:8]
        if not torch.equal(raw[:8], raw[8:16]):
            assert tensor_digest(swapped.view(dtype)) != got
    many = tensor_digests({"a": t, "b": flipped.view(dtype), "c": t[: max(1, numel // 2)]})   # one read-back for all
    assert many["a"] == got and many["b"] != got


@pytest.mark.parametrize("src_dtype,dst_dtype", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.bfloat16),
                                                 (torch.bfloat16, torch.float32), (torch.float16, torch.float32)])
def test_table_driven_cast_matches_per_tensor_casts(src_dtype, dst_dtype):
    """``cast_segments`` (one launch for many tensors) against ``Tensor.to``: sizes below, at and above one work unit,
    a size that is not a multiple of eight, a source that is not 16-byte aligned; bytes between the tensors stay
    untouched.  ``peer_copy`` moves plain bytes in stream order."""
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
    sizes = [1, 7, 4096, 32768, 32769, 100003, 3 * 32768]
    g = torch.Generator(device="cuda").manual_seed(5)
    pool = torch.randn(sum(sizes) + 64, device="cuda", generator=g).to(src_dtype)
    item = torch.empty((), dtype=dst_dtype).element_size()
    window = torch.full((sum((n * item + 255) // 256 * 256 + 256 for n in sizes),), 0xAB, dtype=torch.uint8, device="cuda")
    rows, units, cursor, start, expected = [], 0, 0, 1, []  # start = 1: the first source is deliberately misaligned
    for n in sizes:
        src = pool[start : start + n]
        rows.append((src.data_ptr(), cursor, n, units))
        expected.append((cursor, src.to(dst_dtype)))
        units += (n + 32767) // 32768
        cursor += (n * item + 255) // 256 * 256 + 256
        start += n + (8 if n % 2 else 0)
    ext.cast_segments(torch.tensor(rows, dtype=torch.int64).cuda(), units, code[src_dtype], code[dst_dtype], window.data_ptr())
    for (offset, want), n in zip(expected, sizes):
        got = window[offset : offset + n * item].view(dst_dtype)
        assert torch.equal(got, want)
        assert bool((window[offset + n * item : offset + n * item + 16] == 0xAB).all())  # nothing written past the tensor
    copy = torch.zeros_like(window)
    ext.peer_copy(copy.data_ptr() + 256, window[256:], window.numel() - 256)
    assert torch.equal(copy[256:], window[256:]) and int(copy[:256].sum()) == 0


@pytest.mark.parametrize("stores", ["copy-engine", "kernel"])
def test_nvlink_broadcast_bridge_single_rank_publish_import_acknowledge(stores):
    """The weight-sync transport over symmetric memory on one rank: fp32 trainer weights land in the window as bf16
    through the cast+broadcast kernel, the manifest validates, tampering is caught, a too-small window is refused."""
    from rl_engine.executors.bridge import (
        NVLinkBroadcastBridge, WeightBridgeUnavailableError, WeightManifestValidationError, make_weight_bridge,
    )
    from rl_engine.parallel.symmetric import SymmetricMemory

    mem = SymmetricMemory(8 << 20)
    bridge = make_weight_bridge("nvlink-broadcast", memory=mem, capacity_bytes=4 << 20, target_dtype=torch.bfloat16,
                                stores=stores)
    assert isinstance(bridge, NVLinkBroadcastBridge) and bridge.stores == stores
    torch.manual_seed(3)
    model = torch.nn.Sequential(torch.nn.Linear(300, 257), torch.nn.Linear(257, 19, bias=False)).cuda()
    model.register_buffer("step", torch.tensor([5], dtype=torch.int64, device="cuda"))
    manifest, tensors = bridge.sync(model, weight_version=3)
    mem.check()
    assert manifest.transport == "nvlink-broadcast" and manifest.weight_version == 3
    assert bridge.active_weight_version == 3 and bridge.update_status(manifest.update_id) == "acknowledged"
    for name, want in model.state_dict().items():
        got = tensors[name]
        if want.is_floating_point():
            assert got.dtype == torch.bfloat16 and torch.equal(got, want.to(torch.bfloat16)), name
        else:
            assert torch.equal(got, want), name
        lo, hi = bridge.window.local.data_ptr(), bridge.window.local.data_ptr() + bridge.window.local.numel()
        assert lo <= got.data_ptr() < hi and got.data_ptr() % 256 == 0       # a view of the window, 256-byte aligned
    second = bridge.publish(model, weight_version=4)
    view = bridge.import_update(second)
    view["0.weight"].view(-1)[:8].add_(1.0)
    with pytest.raises(WeightManifestValidationError, match="checksum"):
        bridge.acknowledge(second.update_id)
    assert bridge.active_weight_version == 3                                  # the previous version stays active
    tiny = NVLinkBroadcastBridge(mem, 1024)
    with pytest.raises(WeightBridgeUnavailableError):
        tiny.publish(model, weight_version=1)
    mem.check()
    mem.close()


@pytest.mark.parametrize("n,offset", [(8 * 4096, 0), (8 * 4096 + 5, 0), (3, 0), (8 * 1000 + 3, 1), (8 * 5000, 8)])
def test_cast_broadcast_and_peer_sum_vector_and_scalar_paths(n, offset):
    """Sizes that are not multiples of 8 take a scalar tail; an element offset that leaves the pointer off a 16-byte boundary takes the
    scalar path for everything.  Both must agree with a plain cast / sum."""
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    torch.manual_seed(n)
    src = torch.randn(n, device="cuda")
    for code, dtype in ((0, torch.float32), (1, torch.bfloat16), (2, torch.float16)):
        dst = torch.zeros(n + 64, dtype=dtype, device="cuda")
        view = dst[offset:]
        ext.cast_broadcast(src, [view.data_ptr()], code)
        torch.testing.assert_close(view[:n], src.to(dtype), rtol=0, atol=0)
        assert float(view[n:].abs().sum()) == 0.0
    a, b = src.to(torch.bfloat16), torch.randn(n, device="cuda").to(torch.bfloat16)
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(n, dtype=out_dtype, device="cuda")
        ext.peer_sum([a.data_ptr(), b.data_ptr()], n, False, out)
        torch.testing.assert_close(out, (a.float() + b.float()).to(out_dtype), rtol=0, atol=0)
    out = torch.zeros(n, device="cuda")
    ext.peer_sum([src.data_ptr(), src.data_ptr(), src.data_ptr()], n, True, out)
    torch.testing.assert_close(out, src + src + src, rtol=0, atol=1e-6)


def test_fused_tp_linears_single_rank_match_plain_gemm():
    """World size 1: the copy warps feed this GPU's own gathered buffer and the reduce phase sums a single
    slab, so both fused kernels must reproduce the plain GEMM (three rounds reuse both buffer parities)."""
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.parallel.tp_linear import TensorParallelLinears, pick_chunks

    assert pick_chunks(1024, 4096) == 8 and pick_chunks(128, 512) == 1 and pick_chunks(16384, 4096) == 2
    tp = TensorParallelLinears()
    for it in range(3):
        g = torch.Generator(device="cuda").manual_seed(40 + it)
        x = torch.randn(640, 1024, device="cuda", generator=g).to(torch.bfloat16).requires_grad_(True)
        w = (torch.randn(712, 1024, device="cuda", generator=g) * 0.05).to(torch.bfloat16).requires_grad_(True)
        dy = torch.randn(640, 712, device="cuda", generator=g).to(torch.bfloat16)
        for layer in (tp.column_parallel, tp.row_parallel):
            x.grad = w.grad = None
            y = layer(x, w)
            y.backward(dy)
            ref = x.detach().float() @ w.detach().float().t()
            assert (y.float() - ref).abs().max() / ref.abs().max() < 1e-2
            dx = dy.float() @ w.detach().float()
            dw = dy.float().t() @ x.detach().float()
            assert (x.grad.float() - dx).abs().max() / dx.abs().max() < 1e-2
            assert (w.grad.float() - dw).abs().max() / dw.abs().max() < 1e-2
    check_device_errors(0)


def test_tensor_parallel_layer_single_rank_matches_model_layer():
    from rl_engine.kernels.ops.sm100.attention import make_layout
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.tp_linear import TensorParallelLinears
    from rl_engine.parallel.tp_transformer import TensorParallelLlamaLayer, shard_layer_weights

    cfg = ModelConfig("tp-check", 1024, 512, 1, 4, 2, 128, 768)
    model = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=4, activation_checkpointing=False)
    t = 384
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(t, 512, device="cuda", generator=g).to(torch.bfloat16)
    dout = torch.randn(t, 512, device="cuda", generator=g).to(torch.bfloat16)
    pos = torch.arange(t, device="cuda")
    layout = make_layout([(0, 128, 0, 0, 0, 128), (128, 256, 0, 0, 128, 256)], True, "cuda")
    xf = x.clone().requires_grad_(True)
    yf = model._layer(xf, 0, pos, layout)
    yf.backward(dout)
    w = {k: v.requires_grad_(True) for k, v in shard_layer_weights(model, 0, 0, 1).items()}
    layer = TensorParallelLlamaLayer(cfg, w, TensorParallelLinears(), model.rope_cos, model.rope_sin)
    xl = x.clone().requires_grad_(True)
    yl = layer(xl, pos, layout)
    yl.backward(dout)
    assert torch.allclose(yl.float(), yf.float(), atol=3e-2, rtol=3e-2)
    assert (xl.grad.float() - xf.grad.float()).abs().max() / xf.grad.float().abs().max() < 3e-2
    gw = model.params[model._index["l0.w_down"]].grad
    assert (w["w_down"].grad.float() - gw.float()).abs().max() / gw.float().abs().max() < 3e-2


def test_tensor_parallel_model_single_rank_trains_like_the_plain_model():
    """World size 1: the tensor-parallel model / trainer (fused TP kernels, flat local optimiser) must follow the plain
    single-GPU trainer on the same weights and batch."""
    from rl_engine.models.config import ModelConfig
    from rl_engine.models.grpo import GRPOTrainer, synthetic_batch
    from rl_engine.models.llama import LlamaModel
    from rl_engine.parallel.tp_linear import TensorParallelLinears
    from rl_engine.parallel.tp_model import TensorParallelGRPOTrainer, TensorParallelLlama

    cfg = ModelConfig("tp-model", 2048, 512, 2, 4, 2, 128, 1024)
    plain = LlamaModel(cfg, dtype=torch.bfloat16, device="cuda", seed=21)
    tp_model = TensorParallelLlama(plain, TensorParallelLinears())
    batch = synthetic_batch(cfg.vocab_size, prompt_len=128, group=4, completion_len=96, seed=3)
    a, b = GRPOTrainer(plain, lr=1e-3), TensorParallelGRPOTrainer(tp_model, lr=1e-3)
    la = [a.step(batch) for _ in range(3)]
    lb = [b.step(batch) for _ in range(3)]
    assert abs(la[0] - lb[0]) < 2e-2 * max(1.0, abs(la[0])), (la, lb)
    assert lb[-1] < lb[0], lb
    diff = (tp_model.params["final_norm"].detach().float() - plain.view("final_norm").detach().float()).abs().max()
    assert float(diff) < 5e-2


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_parallel_checks_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
        "--master-port", "29731", os.path.join(ROOT, "tests", "multigpu", "run_parallel_checks.py"),
    ]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0 and "ALL OK" in out.stdout, out.stdout[-3000:] + out.stderr[-3000:]
