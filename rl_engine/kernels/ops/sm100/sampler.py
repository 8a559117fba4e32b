"""Temperature / top-k / top-p sampling on the sm_100a kernel (one CTA per row).

The draw is a pure function of ``(logits row, top_k, top_p, temperature, seed, offset, row)``;
``philox_uniform`` below restates the kernel's random stream on the host so tests can predict it.
Reference: FlashInfer calls in ``rl_engine/kernels/sampling.py:41-78``.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from rl_engine.kernels.ops.base import require_ext

TOPK_LIMIT = 1024
_M32 = 0xFFFFFFFF


def philox_uniform(seed: int, offset: int, row: int) -> float:
    """Host restatement of the kernel's Philox4x32-10 draw -> uniform in (0, 1)."""
    c = [offset & _M32, (offset >> 32) & _M32, row & _M32, 0]
    k = [seed & _M32, (seed >> 32) & _M32]
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        c = [((p1 >> 32) ^ c[1] ^ k[0]) & _M32, p1 & _M32, ((p0 >> 32) ^ c[3] ^ k[1]) & _M32, p0 & _M32]
        k = [(k[0] + 0x9E3779B9) & _M32, (k[1] + 0xBB67AE85) & _M32]
    return ((c[0] >> 8) + 0.5) / 16777216.0


def sample_reference(logits: torch.Tensor, top_k: int, top_p: float, temperature: float, seed: int, offset: int):
    """CPU oracle with the kernel's exact tie-breaking and cut rule (fp32 math)."""
    out = []
    z = logits.float().cpu()
    for row in range(z.shape[0]):
        order = sorted(range(z.shape[1]), key=lambda i: (-float(z[row, i]), i))
        kth = float(z[row, order[min(top_k, z.shape[1]) - 1]])
        cand = [i for i in order if float(z[row, i]) >= kth]
        e = torch.exp((z[row, cand] - z[row, cand[0]]) / temperature)
        cum = torch.cumsum(e, 0)
        total = float(cum[-1])
        nkeep = 1
        for i in range(1, len(cand)):
            if float(cum[i - 1]) <= top_p * total:
                nkeep = i + 1
            else:
                break
        target = philox_uniform(seed, offset, row) * float(cum[nkeep - 1])
        pick = nkeep - 1
        for i in range(nkeep):
            if float(cum[i]) > target:
                pick = i
                break
        out.append(cand[pick])
    return torch.tensor(out, dtype=torch.long)


def nucleus_reference(logits: torch.Tensor, top_p: float, temperature: float, seed: int, offset: int):
    """CPU oracle of the full-vocabulary nucleus kernel: 40-bit fixed-point masses, cut = smallest value v such
    that the mass of tokens >= v reaches ``top_p`` of the total (ties kept), inverse CDF in index order."""
    out = []
    z = logits.float().cpu()
    for row in range(z.shape[0]):
        m = float(z[row].max())
        # float32 arithmetic as in the kernel; __expf differs from exp by a few ulp, so tests compare the kept
        # set and the drawn token's cumulative interval with a tolerance instead of bit-exact masses
        e = torch.exp((z[row] - m) / temperature).double()
        mass = torch.floor(e * float(1 << 40)).to(torch.int64)
        total = int(mass.sum())
        want = max(1, int(top_p * total))
        order = torch.argsort(z[row], descending=True, stable=True)
        cum = torch.cumsum(mass[order], 0)
        first = int(torch.searchsorted(cum, torch.tensor(want), right=False))
        first = min(first, z.shape[1] - 1)
        cut = float(z[row, order[first]])
        keep = z[row] >= cut
        kept_mass = torch.where(keep, mass, torch.zeros_like(mass))
        kept = int(kept_mass.sum())
        t = min(int(philox_uniform(seed, offset, row) * kept), max(kept - 1, 0))
        c = torch.cumsum(kept_mass, 0)
        out.append(int(torch.searchsorted(c, torch.tensor(t), right=True)))
    return torch.tensor(out, dtype=torch.long)


def sample_topk_topp(
    logits: torch.Tensor, *, top_k: Optional[int], top_p: Optional[float], temperature: float = 1.0,
    seed: int = 0, offset: int = 0, return_logprob: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    v = logits.shape[-1]
    rows = logits.reshape(-1, v)
    if rows.stride(1) != 1:
        rows = rows.contiguous()
    # top_k None (or >= vocab): the full-vocabulary nucleus kernel (k = 0 in the native call); its kept set is the
    # smallest set of most probable tokens reaching top_p, drawn in index order -- see ``nucleus_reference``.
    k = 0 if (top_k is None or int(top_k) >= v) else int(top_k)
    if k > TOPK_LIMIT:
        raise ValueError(f"top_k must be <= {TOPK_LIMIT} (or None / >= vocab) for the fused sampler, got {k}")
    p = 1.0 if top_p is None else float(top_p)
    ids, lp = require_ext().sample(rows, k, p, float(temperature), int(seed), int(offset), bool(return_logprob))
    return ids.reshape(logits.shape[:-1]), (lp.reshape(logits.shape[:-1]) if return_logprob else None)
