"""Cases for the debug-bounds build, run as a script with ``RLK_DEBUG_BOUNDS=1`` (by ``test_gpu_debug_bounds.py``).

Part 1: ordinary small workloads of the kernels that take caller-supplied indices must leave the device error word
clean.  Part 2: one out-of-range index per kernel; the checked build records ``index out of range`` with the kernel's id
and SKIPS the access, so nothing is read or written outside a buffer.  Prints ``DEBUG-BOUNDS OK`` at the end.
"""

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
assert os.environ.get("RLK_DEBUG_BOUNDS") == "1", "run with RLK_DEBUG_BOUNDS=1"

from rl_engine.kernels.ops.base import _C, check_device_errors  # noqa: E402

assert _C.__name__.endswith("_C_dbg"), f"the debug-bounds extension was not loaded: {_C.__name__}"
dev = torch.device("cuda", 0)
g = torch.Generator(device=dev).manual_seed(0)


def clean():
    check_device_errors(0)


def expect_bad_index(kernel_ids):
    code, kernel, _block, _site = _C.error_state(0)
    assert code == 4 and kernel in kernel_ids, f"expected a bad-index report from kernel {kernel_ids}, got {(code, kernel)}"
    _C.reset_error(0)


# ---- part 1: valid inputs ------------------------------------------------------------------------------
from rl_engine.kernels.registry import kernel_registry  # noqa: E402

table = torch.randn(50, 64, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
ids = torch.randint(0, 50, (33,), device=dev, generator=g)
emb = kernel_registry.get_op("embedding")(ids, table)
emb.float().sum().backward()
clean()

x = torch.randn(40, 4, 128, device=dev, generator=g).to(torch.bfloat16)
pos = torch.randint(0, 16, (40,), device=dev, generator=g)
from rl_engine.kernels.ops.pytorch.linear.rope import rope_cos_sin  # noqa: E402

cos, sin = rope_cos_sin(torch.arange(16, device=dev), 128, 10000.0)
cos, sin = cos.contiguous(), sin.contiguous()
_C.rope(x, pos, cos, sin, False, None)
_C.rope(x.float(), pos, cos, sin, True, None)
clean()

logits = torch.randn(12, 300, device=dev, generator=g)
tok = torch.randint(0, 300, (12,), device=dev, generator=g)
out = torch.zeros(12, device=dev)
_C.logp_rows(logits, tok, torch.tensor([0, 5, 11], device=dev), out)
want = torch.log_softmax(logits, -1).gather(-1, tok[:, None]).squeeze(-1)
assert torch.allclose(out[[0, 5, 11]], want[[0, 5, 11]], atol=1e-4)
clean()

rewards = torch.randn(10, device=dev, generator=g)
adv = _C.group_advantages(rewards, torch.tensor([0, 3, 10], device=dev), 0, 1e-6)
assert torch.isfinite(adv).all()
clean()

from rl_engine.kernels.ops.sm100.linear_logp import FusedLinearLogpSM100Op  # noqa: E402
from rl_engine.kernels.ops.sm100.moe import FusedMoESM100Op  # noqa: E402

h = torch.randn(70, 128, device=dev, generator=g).to(torch.bfloat16)
w = (torch.randn(520, 128, device=dev, generator=g) * 0.05).to(torch.bfloat16)
FusedLinearLogpSM100Op()(h, w, torch.randint(0, 520, (70,), device=dev, generator=g))
xm = torch.randn(96, 256, device=dev, generator=g).to(torch.bfloat16)
router = (torch.randn(8, 256, device=dev, generator=g) * 0.3).to(torch.bfloat16)
w1 = (torch.randn(8 * 2 * 128, 256, device=dev, generator=g) * 0.06).to(torch.bfloat16)
w2 = (torch.randn(8 * 256, 128, device=dev, generator=g) * 0.09).to(torch.bfloat16)
FusedMoESM100Op()(xm, router, w1, w2, 2)
from rl_engine.kernels.sampling import SamplerBackend  # noqa: E402

SamplerBackend(seed=1).sample(torch.randn(4, 1000, device=dev, generator=g), top_k=20, top_p=0.9, temperature=0.8)
from rl_engine.kernels.ops.sm100.attention import make_layout, packed_attention_forward  # noqa: E402

qa = torch.randn(256, 4, 128, device=dev, generator=g).to(torch.bfloat16)
ka = torch.randn(384, 2, 128, device=dev, generator=g).to(torch.bfloat16)
va = torch.randn(384, 2, 128, device=dev, generator=g).to(torch.bfloat16)
good_layout = make_layout([(0, 128, 0, 128, 128, 128), (128, 128, 0, 128, 256, 128)], True, dev)
packed_attention_forward(qa, ka, va, good_layout, 128 ** -0.5, True)
clean()

# ---- part 2: one bad index per kernel; the checked access is skipped and reported --------------------------------
bad_ids = ids.clone()
bad_ids[4] = 50
_C.embedding_fwd(bad_ids, table.detach())
expect_bad_index({620})

bad_pos = pos.clone()
bad_pos[7] = 16                                   # one past the cos / sin tables
_C.rope(x, bad_pos, cos, sin, False, None)
expect_bad_index({611})
_C.rope(x.float(), bad_pos, cos, sin, False, None)
expect_bad_index({610})

_C.logp_rows(logits, tok, torch.tensor([0, 12], device=dev), out)      # gathered row 12 of 12
expect_bad_index({630})

_C.group_advantages(rewards, torch.tensor([0, 3, 11], device=dev), 0, 1e-6)  # the last group ends past the rewards
expect_bad_index({640})

bad_layout = make_layout([(0, 128, 0, 128, 128, 128), (128, 128, 0, 128, 320, 128)], True, dev)  # keys 320..447 of 384
packed_attention_forward(qa, ka, va, bad_layout, 128 ** -0.5, True)
expect_bad_index({200})

torch.cuda.synchronize()
assert float(torch.ones(4, device=dev).sum()) == 4.0    # the context is intact
clean()
print("DEBUG-BOUNDS OK")
