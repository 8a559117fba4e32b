"""tcgen05 GEMM vs an fp32 PyTorch reference: every operand layout, ragged shapes, accumulate."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(a, b, a_mn, b_mn):
    af = a.float().t() if a_mn else a.float()
    bf = b.float().t() if b_mn else b.float()
    return af @ bf.t()


def _rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, device="cuda", generator=g) * 0.5).to(torch.bfloat16)


SHAPES = [(128, 256, 64), (256, 512, 128), (384, 768, 512), (200, 328, 136), (1, 8, 8), (129, 257, 72), (1000, 1000, 1000)]


@pytest.mark.parametrize("pair", [False, True], ids=["single_cta", "cta_pair"])
@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_gemm_layouts(M, N, K, a_mn, b_mn, pair):
    from functools import partial

    from rl_engine.kernels.ops.sm100 import gemm as gemm_module

    gemm = partial(gemm_module.gemm, pair=pair)

    if (a_mn and M % 8) or (b_mn and N % 8):
        pytest.skip("MN-major operands need a 16-byte row pitch")
    a = _rand((K, M) if a_mn else (M, K), 1)
    b = _rand((K, N) if b_mn else (N, K), 2)
    if (not a_mn and K % 8) or (not b_mn and K % 8):
        pytest.skip("row pitch must be a multiple of 8")
    want = _ref(a, b, a_mn, b_mn)
    got32 = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    torch.cuda.synchronize()
    scale = want.abs().max().item() + 1e-6
    assert (got32 - want).abs().max().item() / scale < 2e-3
    got16 = gemm(a, b, a_mn=a_mn, b_mn=b_mn)
    assert (got16.float() - want).abs().max().item() / scale < 1e-2
    # run-to-run bitwise determinism
    again = gemm(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32)
    assert torch.equal(got32, again)


@pytest.mark.parametrize("pair", [False, True], ids=["single_cta", "cta_pair"])
def test_gemm_accumulate_and_alpha(pair):
    from rl_engine.kernels.ops.sm100.gemm import gemm

    a, b = _rand((300, 192), 3), _rand((520, 192), 4)
    base = torch.randn(300, 520, device="cuda")
    out = base.clone()
    gemm(a, b, out=out, out_dtype=torch.float32, accumulate=True, alpha=0.5, pair=pair)
    want = base + 0.5 * (a.float() @ b.float().t())
    assert torch.allclose(out, want, atol=2e-2, rtol=2e-3)


def test_linear_autograd_matches_torch():
    from rl_engine.kernels.ops.sm100.gemm import matmul_nt

    x = _rand((4, 96, 256), 5).requires_grad_(True)
    w = _rand((384, 256), 6).requires_grad_(True)
    y = matmul_nt(x, w)
    dy = _rand((4, 96, 384), 7)
    y.backward(dy)
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yf = xf @ wf.t()
    yf.backward(dy.float())
    for got, want in ((y, yf), (x.grad, xf.grad), (w.grad, wf.grad)):
        scale = want.abs().max().item()
        assert (got.float() - want).abs().max().item() / scale < 1e-2


def test_cta_pair_gemm_matches_single_cta_bitwise_on_a_large_problem():
    """Both tile engines accumulate every output element over k in the same order, so they must agree bitwise."""
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.kernels.ops.sm100.gemm import gemm

    a, b = _rand((4096 + 128, 2048), 7), _rand((3000, 2048), 8)
    one = gemm(a, b, pair=False)
    two = gemm(a, b, pair=True)
    assert torch.equal(one, two)
    w = _rand((2048, 1536), 9)
    assert torch.equal(gemm(a, w, b_mn=True, pair=False), gemm(a, w, b_mn=True, pair=True))
    check_device_errors(0)


@pytest.mark.parametrize("m,n,k", [(256, 512, 256), (300, 1000, 1168), (1024, 4096, 4096), (77, 264, 144)])
def test_fp8_gemm_matches_the_dequantised_fp32_product(m, n, k):
    """The kernel multiplies e4m3 codes exactly (fp32 accumulation) and applies the row / channel scales in the
    epilogue, so it must agree with the fp32 product of the dequantised operands to bf16 output rounding; the
    quantiser must agree with a PyTorch restatement code for code."""
    from rl_engine.kernels.ops.base import check_device_errors
    from rl_engine.kernels.ops.sm100.gemm_fp8 import (Fp8Linear, gemm_fp8, matmul_nt_fp8, quantize_rows,
                                                      quantize_rows_reference)

    g = torch.Generator(device="cuda").manual_seed(m + n + k)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(n, k, device="cuda", generator=g)).to(torch.bfloat16)
    x[3] = 0  # an all-zero row gets scale 1 and zero codes
    xq, xs = quantize_rows(x)
    wq, ws = quantize_rows(w)
    xq_ref, xs_ref = quantize_rows_reference(x)
    assert torch.allclose(xs, xs_ref, rtol=2e-7, atol=0)
    same = xq.view(torch.float8_e4m3fn).float() == xq_ref.float()
    assert float(same.float().mean()) > 0.999  # a scale that differs in its last bit may move a code at a rounding tie
    ref = (xq.view(torch.float8_e4m3fn).float() * xs[:, None]) @ (wq.view(torch.float8_e4m3fn).float() * ws[:, None]).t()
    out = gemm_fp8(xq, xs, wq, ws)
    assert out.dtype == torch.bfloat16 and out.shape == (m, n)
    assert (out.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
    assert torch.equal(out, gemm_fp8(xq, xs, wq, ws))  # run to run
    assert torch.equal(gemm_fp8(xq, xs, wq, ws, pair=True), gemm_fp8(xq, xs, wq, ws, pair=False))  # both tile engines
    # against the unquantised product: e4m3 has a 3-bit mantissa, errors average out over K
    full = x.float() @ w.float().t()
    rel = (out.float() - full).norm() / full.norm()
    assert float(rel) < 6e-2
    assert torch.equal(matmul_nt_fp8(x, wq, ws), out) and torch.equal(Fp8Linear(w)(x), out)
    check_device_errors(0)


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (32, 4096, 14336), (128, 1000, 520), (77, 28672, 4096)])
def test_skinny_gemm_rows_equal_the_same_rows_of_a_tall_gemm(m, n, k):
    """At most 128 rows of A take the 64-column-tile engine (more CTAs to stream the weight matrix); every output
    element accumulates over K in the same order as on the other engines, so the rows must be the bits that a taller
    problem containing them produces."""
    from rl_engine.kernels.ops.sm100.gemm import gemm

    g = torch.Generator(device="cuda").manual_seed(m + n)
    x = torch.randn(256, k, device="cuda", generator=g).to(torch.bfloat16)
    w = (0.05 * torch.randn(n, k, device="cuda", generator=g)).to(torch.bfloat16)
    tall = gemm(x, w, pair=False)
    skinny = gemm(x[:m], w)
    assert torch.equal(skinny, tall[:m])
    ref = x[:m].float() @ w.float().t()
    assert (skinny.float() - ref).abs().max() <= 1e-2 * ref.abs().max()
