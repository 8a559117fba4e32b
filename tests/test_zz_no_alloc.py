"""The allocation-free RMSNorm backward, called through its exported C symbol.

Callers that cannot allocate (code under stream capture, a frozen memory pool, a non-PyTorch host
runtime) use ``rlk_rmsnorm_backward_noalloc``; its scratch is a fixed device array inside the
library.  This test loads the built extension with ctypes, calls the symbol twice in a row on
different inputs (the shared scratch keeps the first call's contents) and compares both results with
the regular entry point, which takes scratch from PyTorch's allocator.  It also checks the size
limit.  The file name sorts last so that a ``-x`` run has already executed every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20


def _lib():
    from rl_engine.kernels.ops.base import require_ext

    lib = ctypes.CDLL(require_ext().__file__)
    fn = lib.rlk_rmsnorm_backward_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_longlong, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p]
    lib.rlk_noalloc_last_error.restype = ctypes.c_char_p
    lib.rlk_rmsnorm_backward_noalloc_scratch_floats.restype = ctypes.c_longlong
    lib.rlk_rmsnorm_backward_noalloc_scratch_floats.argtypes = [ctypes.c_longlong, ctypes.c_int]
    return lib


CODES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def _close(got, want):
    scale = want.float().abs().max().item() + 1e-6
    tol = 2e-2 if got.dtype in (torch.bfloat16, torch.float16) else 1e-5
    return (got.float() - want.float()).abs().max().item() / scale < tol


def _call(lib, x, w, dy, rstd, dx, dw):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.rlk_rmsnorm_backward_noalloc(
        x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), x.shape[0], x.shape[1],
        x.stride(0), CODES[x.dtype], CODES[w.dtype], ctypes.c_void_p(stream),
    )


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_regular_entry_point_twice(dtype):
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    lib = _lib()
    gen = torch.Generator(device="cuda").manual_seed(3)
    for rows, dim in [(777, 512), (300, 1024)]:  # two calls in a row share the library's scratch array
        x = torch.randn(rows, dim, device="cuda", generator=gen).to(dtype)
        w = torch.randn(dim, device="cuda", generator=gen).to(dtype)
        dy = torch.randn(rows, dim, device="cuda", generator=gen).to(dtype)
        _, rstd = ext.rmsnorm_fwd(x, w, 1e-6, False, True)
        want_dx, want_dw = ext.rmsnorm_bwd(x, w, dy, rstd)
        dx = torch.full_like(x, float("nan"))
        dw = torch.full_like(w, float("nan"))
        rc = _call(lib, x, w, dy, rstd, dx, dw)
        assert rc == 0, lib.rlk_noalloc_last_error()
        torch.cuda.synchronize()
        # same kernels: dx is computed row by row and agrees bitwise; the weight gradient is a sum over rows that the
        # two entry points cut into chunks of different length, so it agrees to rounding (the tolerance of the other
        # RMSNorm tests)
        assert torch.equal(dx, want_dx)
        assert _close(dw, want_dw)


@pytest.mark.parametrize("case", ["fp16", "fp32_wide_rows", "mixed_dtypes", "row_pitch"])
def test_noalloc_other_paths_match_regular_entry_point(case):
    """The generic kernel (fp16, mixed x / weight types), rows wider than 48 KB of shared memory, and a row pitch
    larger than the row, each called twice in a row."""
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    lib = _lib()
    gen = torch.Generator(device="cuda").manual_seed(11)
    xdt, wdt, dim, pitch = {
        "fp16": (torch.float16, torch.float16, 640, 640),
        "fp32_wide_rows": (torch.float32, torch.float32, 16384, 16384),
        "mixed_dtypes": (torch.bfloat16, torch.float32, 768, 768),
        "row_pitch": (torch.bfloat16, torch.bfloat16, 512, 640),
    }[case]
    for rows in (130, 65):
        x = torch.randn(rows, pitch, device="cuda", generator=gen).to(xdt)[:, :dim]
        dy = torch.randn(rows, pitch, device="cuda", generator=gen).to(xdt)[:, :dim]
        w = torch.randn(dim, device="cuda", generator=gen).to(wdt)
        _, rstd = ext.rmsnorm_fwd(x.contiguous(), w, 1e-6, False, True)
        want_dx, want_dw = ext.rmsnorm_bwd(x.contiguous(), w, dy.contiguous(), rstd)
        dx = torch.full((rows, pitch), float("nan"), device="cuda", dtype=xdt)[:, :dim]
        dw = torch.full_like(w, float("nan"))
        rc = _call(lib, x, w, dy, rstd, dx, dw)
        assert rc == 0, lib.rlk_noalloc_last_error()
        torch.cuda.synchronize()
        assert torch.equal(dx, want_dx)
        assert _close(dw, want_dw)


def test_noalloc_rejects_oversized_and_bad_arguments():
    lib = _lib()
    rows, dim = 64 * 300, 4096  # 300 chunks x 4096 floats > 2^20
    assert lib.rlk_rmsnorm_backward_noalloc_scratch_floats(rows, dim) > SCRATCH_FLOATS
    x = torch.zeros(rows, dim, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(dim, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(rows, device="cuda")
    dx, dw = torch.zeros_like(x), torch.zeros_like(w)
    assert _call(lib, x, w, x, rstd, dx, dw) == 1
    assert b"scratch" in lib.rlk_noalloc_last_error()
    assert lib.rlk_rmsnorm_backward_noalloc(0, 0, 0, 0, 0, 0, 1, 1, 1, 0, 0, None) == 2
    # a row that cannot fit the kernel's shared-memory buffer is refused before any launch
    wide = 60000
    xw = torch.zeros(1, wide, device="cuda")
    ww = torch.ones(wide, device="cuda")
    assert _call(lib, xw, ww, xw, torch.ones(1, device="cuda"), torch.zeros_like(xw), torch.zeros_like(ww)) == 2
    assert b"shared-memory" in lib.rlk_noalloc_last_error()
    torch.cuda.synchronize()
    assert torch.zeros(1, device="cuda").item() == 0.0  # the context is intact and no error was left behind
