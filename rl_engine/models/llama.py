"""Llama-style decoder over packed tokens, assembled from registry operators.

Token layout: one flat axis ``[T]`` with a ``PackedLayout`` describing which key ranges every
sequence attends (``rl_engine.kernels.ops.sm100.attention``), so a GRPO group is stored as
``[prompt | completion_0 | ... ]`` and the prompt is embedded, projected and attended exactly once.

On a Blackwell GPU with bf16 weights every matmul is the tcgen05 GEMM, attention is the tcgen05
flash kernel and the elementwise ops are the sm_100a kernels; on CPU (or fp32) the PyTorch oracles
run, which is the fp32 reference configuration.  All parameters are views into ONE flat buffer so
the optimizer and any gradient collective work on a single contiguous range.

The reference ships no model (only ``Embedding -> Linear`` toys:
``rl_engine/executors/deepspeed_trainer.py:54-70``, ``examples/grpo_single_gpu.py:47-56``).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple, Union

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from rl_engine.kernels.ops.pytorch.linear.rope import rope_cos_sin
from rl_engine.models.activation_plan import ActivationPlanner
from rl_engine.models.config import ModelConfig


def _fused_path(x: torch.Tensor) -> bool:
    return x.is_cuda and x.dtype == torch.bfloat16


def linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    if _fused_path(x) and x.shape[-1] % 8 == 0:
        from rl_engine.kernels.ops.sm100.gemm import matmul_nt

        return matmul_nt(x, w)
    return x @ w.t()


def rms_norm(x, w, eps):
    from rl_engine.kernels.registry import kernel_registry

    return kernel_registry.get_op("rms_norm")(x, w, eps=eps)


def swiglu(gate, up):
    from rl_engine.kernels.registry import kernel_registry

    return kernel_registry.get_op("swiglu")(gate, up)


def swiglu_packed(gate_up):
    from rl_engine.kernels.ops.sm100.model_ops import swiglu_packed as fused

    return fused(gate_up)


def reference_packed_attention(q, k, v, host_seqs, causal: bool, scale: float) -> torch.Tensor:
    """Differentiable PyTorch restatement of packed attention (CPU path / oracle)."""
    hq, hkv = q.shape[1], k.shape[1]
    rep = hq // hkv
    outs: List[Tuple[int, torch.Tensor]] = []
    for (q_start, q_len, pk_start, pk_len, sk_start, sk_len) in host_seqs:
        qs = q[q_start : q_start + q_len].transpose(0, 1)  # Hq, L, D
        keys, vals, masks = [], [], []
        for (k0, klen, masked) in ((pk_start, pk_len, False), (sk_start, sk_len, causal)):
            if klen == 0:
                continue
            keys.append(k[k0 : k0 + klen].transpose(0, 1).repeat_interleave(rep, 0))
            vals.append(v[k0 : k0 + klen].transpose(0, 1).repeat_interleave(rep, 0))
            allow = torch.ones(q_len, klen, dtype=torch.bool, device=q.device)
            masks.append(allow.tril() if masked else allow)
        kk, vv, mm = torch.cat(keys, 1), torch.cat(vals, 1), torch.cat(masks, 1)
        s = torch.einsum("hqd,hkd->hqk", qs.float(), kk.float()) * scale
        p = torch.softmax(s.masked_fill(~mm, float("-inf")), dim=-1)
        outs.append((q_start, torch.einsum("hqk,hkd->hqd", p, vv.float()).transpose(0, 1).to(q.dtype)))
    outs.sort(key=lambda t: t[0])
    return torch.cat([o for _, o in outs], 0)


class _FusedAttentionBlock(torch.autograd.Function):
    """qkv [T, Hq+2Hkv, 128] -> RoPE(q), RoPE(k) -> packed flash attention -> [T, Hq, 128]."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_t, sin_t, layout, hq, hkv, scale):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        ext = require_ext()
        # q and k are rotated in place: the projection that produced ``qkv`` does not need its output for its own
        # backward pass, and this block's backward un-rotates the gradients, so the unrotated values are never read
        # again.  One [T, Hq + 2 Hkv, 128] tensor is kept instead of that plus rotated copies of q and k.
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        ext.rope(q, positions, cos_t, sin_t, False, q)
        ext.rope(k, positions, cos_t, sin_t, False, k)
        out, lse = packed_attention_forward(q, k, v, layout, scale, True)
        ctx.save_for_backward(qkv, out, lse, positions, cos_t, sin_t)
        ctx.meta = (layout, hq, hkv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention_bwd import packed_attention_backward

        qkv, out, lse, positions, cos_t, sin_t = ctx.saved_tensors
        layout, hq, hkv, scale = ctx.meta
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        dq, dk, dv = packed_attention_backward(q, k, v, out, lse, dout.contiguous(), layout, scale)
        dqkv = torch.empty_like(qkv)
        ext = require_ext()
        ext.rope(dq, positions, cos_t, sin_t, True, dqkv[:, :hq])
        ext.rope(dk, positions, cos_t, sin_t, True, dqkv[:, hq : hq + hkv])
        dqkv[:, hq + hkv :].copy_(dv)
        return dqkv, None, None, None, None, None, None, None


def _unrotate_into(dqkv, dq, dk, dv, positions, cos_t, sin_t, hq, hkv):
    """Gradients w.r.t. rotated q / k (and v) -> gradient of the packed, unrotated qkv projection output."""
    from rl_engine.kernels.ops.base import require_ext

    ext = require_ext()
    ext.rope(dq, positions, cos_t, sin_t, True, dqkv[:, :hq])
    ext.rope(dk, positions, cos_t, sin_t, True, dqkv[:, hq : hq + hkv])
    dqkv[:, hq + hkv :].copy_(dv)
    return dqkv


class _FusedAttentionBlockKV(torch.autograd.Function):
    """``_FusedAttentionBlock`` that also returns copies of the rotated k and v, for a prefix (prompt) whose keys and
    values later passes attend to.  Their gradients come back as extra inputs of the backward pass."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_t, sin_t, layout, hq, hkv, scale):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        ext = require_ext()
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        ext.rope(q, positions, cos_t, sin_t, False, q)
        ext.rope(k, positions, cos_t, sin_t, False, k)
        out, lse = packed_attention_forward(q, k, v, layout, scale, True)
        ctx.save_for_backward(qkv, out, lse, positions, cos_t, sin_t)
        ctx.meta = (layout, hq, hkv, scale)
        return out, k.contiguous(), v.contiguous()

    @staticmethod
    def backward(ctx, dout, dk_later, dv_later):
        from rl_engine.kernels.ops.sm100.attention_bwd import packed_attention_backward

        qkv, out, lse, positions, cos_t, sin_t = ctx.saved_tensors
        layout, hq, hkv, scale = ctx.meta
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        dq, dk, dv = packed_attention_backward(q, k, v, out, lse, dout.contiguous(), layout, scale)
        if dk_later is not None:
            dk = (dk.float() + dk_later.float()).to(dk.dtype)
        if dv_later is not None:
            dv = (dv.float() + dv_later.float()).to(dv.dtype)
        dqkv = _unrotate_into(torch.empty_like(qkv), dq, dk, dv, positions, cos_t, sin_t, hq, hkv)
        return dqkv, None, None, None, None, None, None, None


class _FusedAttentionBlockPrefix(torch.autograd.Function):
    """Attention of a pass that holds only suffix tokens: keys / values are ``[prefix | this pass]``, the prefix part
    (already rotated) coming from ``_FusedAttentionBlockKV`` of an earlier pass.  ``layout`` indexes queries in this
    pass's rows and keys in the concatenation."""

    @staticmethod
    def forward(ctx, qkv, k_prefix, v_prefix, positions, cos_t, sin_t, layout, hq, hkv, scale):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        ext = require_ext()
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        ext.rope(q, positions, cos_t, sin_t, False, q)
        ext.rope(k, positions, cos_t, sin_t, False, k)
        out, lse = packed_attention_forward(q, torch.cat([k_prefix, k]), torch.cat([v_prefix, v]), layout, scale, True)
        ctx.save_for_backward(qkv, k_prefix, v_prefix, out, lse, positions, cos_t, sin_t)
        ctx.meta = (layout, hq, hkv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_engine.kernels.ops.sm100.attention_bwd import packed_attention_backward

        qkv, k_prefix, v_prefix, out, lse, positions, cos_t, sin_t = ctx.saved_tensors
        layout, hq, hkv, scale = ctx.meta
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        n = k_prefix.shape[0]
        dq, dk, dv = packed_attention_backward(q, torch.cat([k_prefix, k]), torch.cat([v_prefix, v]), out, lse,
                                               dout.contiguous(), layout, scale)
        dqkv = _unrotate_into(torch.empty_like(qkv), dq, dk[n:], dv[n:], positions, cos_t, sin_t, hq, hkv)
        return dqkv, dk[:n], dv[:n], None, None, None, None, None, None, None


class _FusedAttentionBlockCP(torch.autograd.Function):
    """``_FusedAttentionBlock`` for a sequence that is sharded over the ranks of a context-parallel group: ``cp`` (a
    ``rl_engine.parallel.context_parallel.ContextParallelAttention``) gathers every rank's rotated keys / values through
    peer stores before the flash kernel runs on the local queries, and in backward sums the ranks' contributions to the
    locally owned keys / values in rank order.  ``positions`` are the global positions of the local (zig-zag) rows."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_t, sin_t, cp, hq, hkv, scale):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        ext = require_ext()
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        ext.rope(q, positions, cos_t, sin_t, False, q)
        ext.rope(k, positions, cos_t, sin_t, False, k)
        k_all, v_all = cp.gather_kv(k, v)
        out, lse = packed_attention_forward(q, k_all, v_all, cp.layout(q.device), scale, True)
        ctx.save_for_backward(qkv, out, lse, positions, cos_t, sin_t)
        ctx.meta = (cp, hq, hkv, scale)
        return out

    @staticmethod
    def backward(ctx, dout):
        from rl_engine.kernels.ops.sm100.attention_bwd_kernels import fused_backward

        qkv, out, lse, positions, cos_t, sin_t = ctx.saved_tensors
        cp, hq, hkv, scale = ctx.meta
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        k_all, v_all = cp.gather_kv(k, v)  # gathered again: cheaper than keeping the whole sequence's keys per layer
        dq, dk_full, dv_full = fused_backward(q, k_all, v_all, out, lse, dout.contiguous(), cp.layout(q.device), scale)
        dk, dv = cp.reduce_dkv(dk_full, dv_full)
        dqkv = _unrotate_into(torch.empty_like(qkv), dq, dk, dv, positions, cos_t, sin_t, hq, hkv)
        return dqkv, None, None, None, None, None, None, None


class _QKHeadNorm(torch.autograd.Function):
    """Per-head RMSNorm (head_dim 128) of the q and k heads of a packed ``qkv [T, (Hq + 2 Hkv) * 128]``; v is copied.
    One kernel forward and one backward instead of two strided copies, two generic RMSNorm launches and a
    concatenation (and their five backward kernels)."""

    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, hq, hkv, eps):
        from rl_engine.kernels.ops.base import require_ext

        wq, wk = q_weight.contiguous(), k_weight.contiguous()
        ctx.save_for_backward(qkv, wq, wk)
        ctx.meta = (int(hq), int(hkv), float(eps))
        return require_ext().qk_norm_fwd(qkv, wq, wk, int(hq), int(hkv), float(eps))

    @staticmethod
    def backward(ctx, dout):
        from rl_engine.kernels.ops.base import require_ext

        qkv, wq, wk = ctx.saved_tensors
        hq, hkv, eps = ctx.meta
        dqkv, dwq, dwk = require_ext().qk_norm_bwd(qkv, dout.contiguous(), wq, wk, hq, hkv, eps)
        return dqkv, dwq, dwk, None, None, None


class _FusedAttentionBlockCPKV(torch.autograd.Function):
    """``_FusedAttentionBlockCP`` that also returns the gathered rotated keys / values ``[S, Hkv, 128]`` of the whole
    sequence (natural order) as differentiable outputs: later passes attend to them as a cached prefix, and whatever
    gradient reaches them on this rank is added to this rank's contribution before the ranks' contributions are
    summed, so the owner of each chunk receives the gradient of every rank's later passes as well."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_t, sin_t, cp, hq, hkv, scale):
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward

        ext = require_ext()
        q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
        ext.rope(q, positions, cos_t, sin_t, False, q)
        ext.rope(k, positions, cos_t, sin_t, False, k)
        k_all, v_all = cp.gather_kv(k, v)
        k_all, v_all = k_all.clone(), v_all.clone()  # the symmetric buffers are reused by the next layer
        out, lse = packed_attention_forward(q, k_all, v_all, cp.layout(q.device), scale, True)
        ctx.save_for_backward(qkv, out, lse, positions, cos_t, sin_t, k_all, v_all)
        ctx.meta = (cp, hq, hkv, scale)
        return out, k_all, v_all

    @staticmethod
    def backward(ctx, dout, dk_later, dv_later):
        from rl_engine.kernels.ops.sm100.attention_bwd_kernels import fused_backward

        qkv, out, lse, positions, cos_t, sin_t, k_all, v_all = ctx.saved_tensors
        cp, hq, hkv, scale = ctx.meta
        q = qkv[:, :hq]
        dq, dk_full, dv_full = fused_backward(q, k_all, v_all, out, lse, dout.contiguous(), cp.layout(q.device), scale)
        if dk_later is not None:
            dk_full = dk_full + dk_later.to(dk_full.dtype)
        if dv_later is not None:
            dv_full = dv_full + dv_later.to(dv_full.dtype)
        dk, dv = cp.reduce_dkv(dk_full, dv_full)
        dqkv = _unrotate_into(torch.empty_like(qkv), dq, dk, dv, positions, cos_t, sin_t, hq, hkv)
        return dqkv, None, None, None, None, None, None, None


class LlamaModel(nn.Module):
    def __init__(self, cfg: ModelConfig, *, dtype: torch.dtype = torch.bfloat16, device="cpu", seed: int = 0,
                 activation_checkpointing: Union[bool, str] = "auto", max_positions: int = 8192,
                 expert_shard: Optional[Tuple[int, int]] = None) -> None:
        """``activation_checkpointing``: ``True`` recomputes every layer in the backward pass, ``False`` keeps every
        layer's activations, ``"auto"`` (default) keeps as many trailing layers as the free device memory allows at the
        first training forward and recomputes the rest (``plan_checkpointing``).

        ``expert_shard = (rank, world)`` (mixture-of-experts models): this instance stores only experts
        ``[rank * E / world, (rank + 1) * E / world)`` of every layer; the router still scores all ``E`` experts and
        ``self.moe_op`` must be set to an expert-parallel operator (``rl_engine.parallel.expert_parallel``) that sends
        every token to the ranks owning its experts.  All other parameters are replicated."""
        super().__init__()
        self.cfg = cfg
        self.expert_shard = expert_shard
        self.moe_op = None  # None: the single-GPU fused MoE from the registry
        self._planner = ActivationPlanner(cfg.num_layers, activation_checkpointing)
        # Optional ``callable(layer_index)``: while it is set, every training forward registers gradient hooks that
        # call it from inside backward when the backward pass has left layer ``layer_index`` (``num_layers`` = the
        # final norm), i.e. when nothing of this pass touches the parameters of layers >= ``layer_index`` again.
        self.layer_grad_hook = None
        self._fp8_linears: Dict[str, object] = {}
        h, f = cfg.hidden_size, cfg.ffn_size
        qkv_rows = cfg.q_dim + 2 * cfg.kv_dim
        shapes: List[Tuple[str, Tuple[int, ...]]] = [("embed", (cfg.vocab_size, h))]
        e, fe = cfg.num_experts, cfg.moe_ffn_size
        e_local = e
        if expert_shard is not None:
            shard_rank, shard_world = expert_shard
            if not e or e % shard_world or not 0 <= shard_rank < shard_world:
                raise ValueError(f"expert_shard={expert_shard} does not divide the {e} experts of this model")
            e_local = e // shard_world
        for i in range(cfg.num_layers):
            shapes += [(f"l{i}.attn_norm", (h,)), (f"l{i}.wqkv", (qkv_rows, h))]
            if cfg.qkv_bias:
                shapes += [(f"l{i}.bqkv", (qkv_rows,))]
            shapes += [(f"l{i}.wo", (h, cfg.q_dim))]
            if cfg.qk_norm:
                shapes += [(f"l{i}.q_norm", (cfg.head_dim,)), (f"l{i}.k_norm", (cfg.head_dim,))]
            shapes += [(f"l{i}.mlp_norm", (h,))]
            if e:  # mixture of experts: router + per-expert [gate | up] and down projections, stacked by expert
                shapes += [(f"l{i}.router", (e, h)), (f"l{i}.w_gate_up", (e_local * 2 * fe, h)),
                           (f"l{i}.w_down", (e_local * h, fe))]
            else:
                shapes += [(f"l{i}.w_gate_up", (2 * f, h)), (f"l{i}.w_down", (h, f))]
        shapes += [("final_norm", (h,)), ("lm_head", (cfg.vocab_size, h))]
        # every parameter starts on a 16-byte boundary of ONE flat buffer
        offsets, total = {}, 0
        for name, shape in shapes:
            offsets[name] = total
            total += (math.prod(shape) + 127) // 128 * 128
        # ``flat`` owns the storage; every nn.Parameter is a view into it, and ``flat_grad`` (allocated by
        # ``ensure_flat_grad``) plays the same role for the gradients, so autograd accumulates straight
        # into one contiguous buffer.
        self.register_buffer("flat", torch.empty(total, dtype=dtype, device=device), persistent=False)
        self.flat_grad: Optional[torch.Tensor] = None
        self._shapes = dict(shapes)
        self._offsets = offsets
        self._names = [name for name, _ in shapes]
        self.params = nn.ParameterList(
            [nn.Parameter(self._slice(self.flat, name), requires_grad=True) for name in self._names]
        )
        self._index = {name: i for i, name in enumerate(self._names)}
        self.reset_parameters(seed)
        cos, sin = rope_cos_sin(torch.arange(max_positions, device=device), cfg.head_dim, cfg.rope_theta, cfg.rope_scaling)
        self.register_buffer("rope_cos", cos.contiguous(), persistent=False)
        self.register_buffer("rope_sin", sin.contiguous(), persistent=False)

    # -- parameters -------------------------------------------------------------------------
    def _slice(self, flat: torch.Tensor, name: str) -> torch.Tensor:
        shape = self._shapes[name]
        off = self._offsets[name]
        return flat[off : off + math.prod(shape)].view(shape)

    def view(self, name: str) -> torch.Tensor:
        """The trainable parameter ``name`` (a view of the flat buffer)."""
        return self.params[self._index[name]]

    def named_views(self) -> Dict[str, torch.Tensor]:
        return {name: self.view(name) for name in self._names}

    @torch.no_grad()
    def rebind_storage(self, flat: torch.Tensor, flat_grad: Optional[torch.Tensor] = None) -> None:
        """Move parameters (and gradients) onto caller-provided flat buffers, e.g. symmetric memory.

        ``flat`` must already hold the parameter values."""
        if flat.numel() != self.flat.numel() or flat.dtype != self.flat.dtype:
            raise ValueError("replacement storage must match the flat parameter buffer")
        self.flat = flat
        for name in self._names:
            self.view(name).data = self._slice(flat, name)
        if flat_grad is not None:
            flat_grad.zero_()
            self.flat_grad = flat_grad
            for name in self._names:
                self.view(name).grad = self._slice(flat_grad, name)

    def ensure_flat_grad(self) -> torch.Tensor:
        """Allocate the flat gradient buffer once and point every ``param.grad`` into it."""
        if self.flat_grad is None:
            self.flat_grad = torch.zeros_like(self.flat)
            for name in self._names:
                self.view(name).grad = self._slice(self.flat_grad, name)
        return self.flat_grad

    @torch.no_grad()
    def reset_parameters(self, seed: int = 0) -> None:
        dev = self.flat.device
        gen = torch.Generator(device=dev).manual_seed(seed)
        self.flat.zero_()
        for name, shape in self._shapes.items():
            dst = self._slice(self.flat, name)
            if name.endswith("norm"):
                dst.fill_(1.0)
                continue
            if name.endswith("bqkv"):
                continue                      # biases start at zero
            # chunked init (on the parameter's own device) keeps the fp32 temporary small
            flat_dst = dst.view(-1)
            step = 1 << 26
            for i in range(0, flat_dst.numel(), step):
                n = min(step, flat_dst.numel() - i)
                flat_dst[i : i + n].copy_((torch.randn(n, generator=gen, device=dev) * 0.02).to(dst.dtype))
        if self.cfg.tie_word_embeddings:
            self._slice(self.flat, "lm_head").copy_(self._slice(self.flat, "embed"))

    def state_dict_views(self, names: str = "native") -> Dict[str, torch.Tensor]:
        """Checkpoint-format names -> tensors (views of the flat buffer), for the weight bridge.  ``names="hf"``: the
        names of the Hugging Face checkpoint of this architecture (``q_proj`` / ``k_proj`` / ``v_proj`` rows of the
        packed ``wqkv`` and so on), still without a copy."""
        if names == "hf":
            from rl_engine.models.hf_interop import hf_state_dict_views

            return hf_state_dict_views(self)
        if names != "native":
            raise ValueError(f"names must be 'native' or 'hf', got {names!r}")
        return {k: v.detach() for k, v in self.named_views().items()}

    # -- forward ----------------------------------------------------------------------------
    def _attention(self, qkv: torch.Tensor, positions: torch.Tensor, layout, index: int = 0, k_prefix=None,
                   v_prefix=None, return_kv: bool = False):
        cfg = self.cfg
        t = qkv.shape[0]
        qkv3 = qkv.view(t, cfg.num_heads + 2 * cfg.num_kv_heads, cfg.head_dim)
        scale = 1.0 / math.sqrt(cfg.head_dim)
        if cfg.qk_norm and _fused_path(qkv) and cfg.head_dim == 128 and qkv.stride(1) == 1 and qkv.stride(0) % 8 == 0 \
                and qkv.data_ptr() % 16 == 0:
            # Qwen3: per-head RMSNorm on q and k before the rotary embedding, one kernel over the packed buffer
            qkv3 = _QKHeadNorm.apply(qkv, self.view(f"l{index}.q_norm"), self.view(f"l{index}.k_norm"), cfg.num_heads,
                                     cfg.num_kv_heads, cfg.rms_eps).view(t, cfg.num_heads + 2 * cfg.num_kv_heads, cfg.head_dim)
        elif cfg.qk_norm:  # the same with the generic ops
            hq, hkv = cfg.num_heads, cfg.num_kv_heads
            qn = rms_norm(qkv3[:, :hq].reshape(-1, cfg.head_dim), self.view(f"l{index}.q_norm"), cfg.rms_eps)
            kn = rms_norm(qkv3[:, hq : hq + hkv].reshape(-1, cfg.head_dim), self.view(f"l{index}.k_norm"), cfg.rms_eps)
            qkv3 = torch.cat([qn.view(t, hq, -1), kn.view(t, hkv, -1), qkv3[:, hq + hkv :]], dim=1)
        if _fused_path(qkv) and cfg.head_dim == 128:
            tail = (positions, self.rope_cos, self.rope_sin, layout, cfg.num_heads, cfg.num_kv_heads, scale)
            if hasattr(layout, "gather_kv"):  # a context-parallel group: ``layout`` is its attention object
                if k_prefix is not None:
                    raise RuntimeError("context-parallel passes do not take a cached prefix")
                if return_kv:
                    out, k_all, v_all = _FusedAttentionBlockCPKV.apply(qkv3, *tail)
                    return out.reshape(t, cfg.q_dim), k_all, v_all
                return _FusedAttentionBlockCP.apply(qkv3, *tail).reshape(t, cfg.q_dim)
            if return_kv:
                out, k_rot, v_rot = _FusedAttentionBlockKV.apply(qkv3, *tail)
                return out.reshape(t, cfg.q_dim), k_rot, v_rot
            if k_prefix is not None:
                return _FusedAttentionBlockPrefix.apply(qkv3, k_prefix, v_prefix, *tail).reshape(t, cfg.q_dim)
            return _FusedAttentionBlock.apply(qkv3, *tail).reshape(t, cfg.q_dim)
        if return_kv or k_prefix is not None:
            raise RuntimeError("prefix-cached passes need the fused attention path (CUDA, bf16, head_dim 128)")
        from rl_engine.kernels.registry import kernel_registry

        rope = kernel_registry.get_op("rope")
        q = rope(qkv3[:, : cfg.num_heads], positions, theta=cfg.rope_theta, scaling=cfg.rope_scaling)
        k = rope(qkv3[:, cfg.num_heads : cfg.num_heads + cfg.num_kv_heads], positions, theta=cfg.rope_theta,
                 scaling=cfg.rope_scaling)
        v = qkv3[:, cfg.num_heads + cfg.num_kv_heads :]
        out = reference_packed_attention(q, k, v, layout.host_seqs, layout.causal, scale)
        return out.reshape(t, cfg.q_dim)

    def _layer(self, x: torch.Tensor, index: int, positions: torch.Tensor, layout, k_prefix=None, v_prefix=None,
               return_kv: bool = False):
        """One decoder layer.  ``k_prefix`` / ``v_prefix``: rotated keys / values of a prefix that is not part of ``x``;
        ``return_kv``: also return this pass's rotated keys and values (``(x, k, v)``)."""
        cfg = self.cfg
        p = lambda n: self.view(f"l{index}.{n}")
        lean = _fused_path(x)  # recompute normalised inputs and the SwiGLU output in backward instead of keeping them
        if lean:
            from rl_engine.kernels.ops.sm100.lean_blocks import norm_linear

            qkv = norm_linear(x, p("attn_norm"), p("wqkv"), cfg.rms_eps)
        else:
            qkv = linear(rms_norm(x, p("attn_norm"), cfg.rms_eps), p("wqkv"))
        if cfg.qkv_bias:
            qkv = qkv + p("bqkv")
        attn = self._attention(qkv, positions, layout, index, k_prefix, v_prefix, return_kv)
        if return_kv:
            attn, k_rot, v_rot = attn
        x = x + linear(attn, p("wo"))
        x = self._ffn(x, index, lean)
        return (x, k_rot, v_rot) if return_kv else x

    def _ffn(self, x: torch.Tensor, index: int, lean: bool) -> torch.Tensor:
        cfg = self.cfg
        p = lambda n: self.view(f"l{index}.{n}")
        if lean:
            from rl_engine.kernels.ops.sm100.lean_blocks import norm_linear, swiglu_linear
        if cfg.num_experts:
            from rl_engine.kernels.registry import kernel_registry

            h = rms_norm(x, p("mlp_norm"), cfg.rms_eps)
            if self.expert_shard is not None and self.moe_op is None:
                raise RuntimeError("a model built with expert_shard needs model.moe_op (an expert-parallel MoE operator)")
            moe = self.moe_op if self.moe_op is not None else kernel_registry.get_op("moe")
            return x + moe(h, p("router"), p("w_gate_up"), p("w_down"), cfg.experts_per_token)
        if lean:
            return x + swiglu_linear(norm_linear(x, p("mlp_norm"), p("w_gate_up"), cfg.rms_eps), p("w_down"))
        gu = linear(rms_norm(x, p("mlp_norm"), cfg.rms_eps), p("w_gate_up"))
        return x + linear(swiglu_packed(gu), p("w_down"))

    # -- activation memory ------------------------------------------------------------------
    def activation_bytes_per_layer(self, tokens: int) -> int:
        """Bytes autograd keeps alive for one dense layer that is not recomputed: the layer input, the mid-layer
        residual, qkv (q and k rotated in place), the attention output and the packed gate/up projection; plus the
        fp32 softmax statistics per head and the two RMSNorm ``rstd`` values."""
        cfg = self.cfg
        per_token = 2 * cfg.hidden_size + (cfg.q_dim + 2 * cfg.kv_dim) + cfg.q_dim + 2 * cfg.ffn_size
        return tokens * (per_token * self.flat.element_size() + 4 * cfg.num_heads + 8)

    def plan_checkpointing(self, tokens: int) -> int:
        """Number of trailing layers whose activations are kept for the backward pass (the others are recomputed);
        see ``ActivationPlanner``.  Mixture-of-experts layers are always recomputed (their activation size depends on
        the routing)."""
        if self.cfg.num_experts and self._planner.mode == "auto":
            return 0
        layer_input = tokens * self.cfg.hidden_size * self.flat.element_size()
        return self._planner.kept(tokens, self.activation_bytes_per_layer(tokens), layer_input, self.flat.device)

    def estimate_kept_layers(self, tokens: int) -> int:
        """What ``plan_checkpointing`` would answer for a packed length of ``tokens`` right now, without fixing it."""
        if self.cfg.num_experts and self._planner.mode == "auto":
            return 0
        layer_input = tokens * self.cfg.hidden_size * self.flat.element_size()
        return self._planner.estimate(self.activation_bytes_per_layer(tokens), layer_input, self.flat.device)

    def kept_layers(self) -> int:
        return self._planner.current()

    def reduce_kept_layers(self, by: int = 4) -> int:
        """After an out-of-memory error: recompute ``by`` more layers from now on.  Returns the new number kept."""
        return self._planner.reduce(by)

    def _watch(self, x: torch.Tensor, layer: int) -> torch.Tensor:
        """Registers the ``layer_grad_hook`` notification on ``x``, the input of layer ``layer``."""
        hook = self.layer_grad_hook
        if hook is not None and x.requires_grad:
            def fire(_grad, layer=layer, hook=hook):
                hook(layer)

            x.register_hook(fire)
        return x

    def hidden_states(self, token_ids: torch.Tensor, positions: torch.Tensor, layout) -> torch.Tensor:
        """Packed ``token_ids [T]`` -> final-norm hidden states ``[T, H]``."""
        from rl_engine.kernels.registry import kernel_registry

        x = kernel_registry.get_op("embedding")(token_ids, self.view("embed"))
        training = torch.is_grad_enabled()
        first_kept = self.cfg.num_layers - (self.plan_checkpointing(token_ids.numel()) if training else 0)
        for i in range(self.cfg.num_layers):
            self._watch(x, i)
            if training and i < first_kept:
                x = checkpoint(self._layer, x, i, positions, layout, use_reentrant=False)
            else:
                x = self._layer(x, i, positions, layout)
        self._watch(x, self.cfg.num_layers)
        return rms_norm(x, self.view("final_norm"), self.cfg.rms_eps)

    # -- prefix-cached passes: the shared prompt runs once, later passes hold only completion tokens ------------
    def supports_prefix_cache(self) -> bool:
        cfg = self.cfg
        return (self.flat.is_cuda and self.flat.dtype == torch.bfloat16 and cfg.head_dim == 128 and not cfg.num_experts)

    def prefix_states(self, prompt_ids: torch.Tensor, cp=None, share_row=None):
        """One pass over the prompt alone: ``(final-norm hidden state of its last token [1, H], [(k, v)] per layer)``
        with the rotated keys / values ``[P, Hkv, 128]`` every later pass attends to.  All outputs carry the
        autograd graph of the prompt pass.

        ``cp`` (a ``ContextParallelAttention`` for ``P`` tokens) shards the pass over the ranks of its group: every
        rank runs only its zig-zag rows, the keys / values it returns are the gathered ones, and ``share_row`` (a
        ``SharedRow`` of that group whose owner holds the last token) hands the last token's state to every rank.
        Back-propagating through the outputs then sums the ranks' gradients onto the rows' owners; together with
        the data-parallel gradient sum this equals every rank running the whole prompt."""
        from rl_engine.kernels.ops.sm100.attention import make_layout
        from rl_engine.kernels.registry import kernel_registry

        n = prompt_ids.numel()
        positions = torch.arange(n, device=prompt_ids.device)
        if cp is None:
            layout = make_layout([(0, n, 0, 0, 0, n)], True, prompt_ids.device)
        else:
            from rl_engine.parallel.context_parallel import shard_sequence

            if cp.seq_len != n or share_row is None:
                raise ValueError("a sharded prompt pass needs a context-parallel object of the prompt's length and a shared row")
            layout = cp
            prompt_ids = shard_sequence(prompt_ids.reshape(-1), cp.rank, cp.world)
            positions = shard_sequence(positions, cp.rank, cp.world)
        x = kernel_registry.get_op("embedding")(prompt_ids, self.view("embed"))
        kv = []
        for i in range(self.cfg.num_layers):
            self._watch(x, i)
            x, k_rot, v_rot = self._layer(x, i, positions, layout, return_kv=True)
            kv.append((k_rot, v_rot))
        self._watch(x, self.cfg.num_layers)
        last = rms_norm(x[-1:], self.view("final_norm"), self.cfg.rms_eps)
        return (last if cp is None else share_row(last)), kv

    def hidden_states_after_prefix(self, token_ids: torch.Tensor, positions: torch.Tensor, layout, kv) -> torch.Tensor:
        """Final-norm hidden states ``[T, H]`` of tokens that follow a prefix given by its per-layer ``kv``.
        ``layout`` indexes queries in ``token_ids`` and keys in ``[prefix | token_ids]``."""
        from rl_engine.kernels.registry import kernel_registry

        x = kernel_registry.get_op("embedding")(token_ids, self.view("embed"))
        training = torch.is_grad_enabled()
        first_kept = self.cfg.num_layers - (self.plan_checkpointing(token_ids.numel()) if training else 0)
        for i, (k_prefix, v_prefix) in enumerate(kv):
            if training and i < first_kept:
                x = checkpoint(self._layer, x, i, positions, layout, k_prefix, v_prefix, use_reentrant=False)
            else:
                x = self._layer(x, i, positions, layout, k_prefix, v_prefix)
        return rms_norm(x, self.view("final_norm"), self.cfg.rms_eps)

    # -- incremental decoding with a key / value cache (rollout side, no autograd) -------------------------
    @torch.no_grad()
    def new_kv_cache(self, rows: int):
        """Per-layer ``(k, v)`` buffers ``[rows, Hkv, 128]`` for ``decode_step``."""
        cfg = self.cfg
        make = lambda: torch.empty(rows, cfg.num_kv_heads, cfg.head_dim, dtype=self.flat.dtype, device=self.flat.device)
        return [(make(), make()) for _ in range(cfg.num_layers)]

    @torch.no_grad()
    def decode_step(self, token_ids: torch.Tensor, positions: torch.Tensor, cache, slots: torch.Tensor, prefix_layout,
                    self_layout) -> torch.Tensor:
        """One new token for each of ``n`` sequences: final-norm hidden states ``[n, H]``.

        The rotated key and value of token ``i`` are written to row ``slots[i]`` of every layer's cache before the
        attention of that layer runs.  Attention packs the queries so that rows which read the same keys share a tile:
        the ``Hq / Hkv`` query heads of a key / value head become rows (``n * Hq / Hkv`` rows, ``Hkv`` heads).
        ``prefix_layout`` is ONE sequence of all those rows against the shared prefix rows of the cache (for 32
        completions of a 4:1 grouped-query model exactly one 128-row tile per key / value head, instead of 1024
        one-row tiles); ``self_layout`` has one sequence per completion: its ``Hq / Hkv`` rows against its own cache rows
        up to and including ``slots[i]``.  Both are non-causal; the two partial results are merged by their
        log-sum-exp (``decode_layouts`` builds the pair)."""
        from rl_engine.kernels.ops.base import require_ext
        from rl_engine.kernels.ops.sm100.attention import packed_attention_forward
        from rl_engine.kernels.registry import kernel_registry

        if not self.supports_prefix_cache():
            raise RuntimeError("decode_step needs the fused path (CUDA, bf16, head_dim 128, dense FFN)")
        cfg, ext = self.cfg, require_ext()
        hq, hkv = cfg.num_heads, cfg.num_kv_heads
        scale = 1.0 / math.sqrt(cfg.head_dim)
        n = token_ids.numel()
        x = kernel_registry.get_op("embedding")(token_ids, self.view("embed"))
        for i in range(cfg.num_layers):
            p = lambda name: self.view(f"l{i}.{name}")
            qkv = self._project(rms_norm(x, p("attn_norm"), cfg.rms_eps), f"l{i}.wqkv")
            if cfg.qkv_bias:
                qkv = qkv + p("bqkv")
            qkv = qkv.view(n, hq + 2 * hkv, cfg.head_dim)
            q, k, v = qkv[:, :hq], qkv[:, hq : hq + hkv], qkv[:, hq + hkv :]
            ext.rope(q, positions, self.rope_cos, self.rope_sin, False, q)
            ext.rope(k, positions, self.rope_cos, self.rope_sin, False, k)
            cache[i][0].index_copy_(0, slots, k)
            cache[i][1].index_copy_(0, slots, v)
            rep = hq // hkv
            rows = q.reshape(n, hkv, rep, cfg.head_dim).permute(0, 2, 1, 3).reshape(n * rep, hkv, cfg.head_dim)
            o1, l1 = packed_attention_forward(rows, cache[i][0], cache[i][1], prefix_layout, scale, True)
            o2, l2 = packed_attention_forward(rows, cache[i][0], cache[i][1], self_layout, scale, True)
            out = ext.attn_merge2(o1, l1, o2, l2, rep)  # [n, Hq * 128] in the model's head order
            x = x + self._project(out, f"l{i}.wo")
            gu = self._project(rms_norm(x, p("mlp_norm"), cfg.rms_eps), f"l{i}.w_gate_up")
            x = x + self._project(swiglu_packed(gu), f"l{i}.w_down")
        return rms_norm(x, self.view("final_norm"), cfg.rms_eps)

    def decode_layouts(self, n: int, prefix_len: int, rows_per_sequence: int, own_len: int = 1):
        """The two layouts of ``decode_step`` for ``n`` sequences whose cache rows are ``[prefix | n x rows_per_sequence]``
        when every sequence holds ``own_len`` tokens including the new one.  Column 5 of ``self_layout.seqs`` is that
        length: a caller that decodes step by step adds one to it in place (the tables are private copies)."""
        from dataclasses import replace

        from rl_engine.kernels.ops.sm100.attention import make_layout

        dev = self.flat.device
        rep = self.cfg.num_heads // self.cfg.num_kv_heads
        prefix = make_layout([(0, n * rep, 0, prefix_len, 0, 0)], False, dev)
        own = make_layout([(i * rep, rep, 0, 0, prefix_len + i * rows_per_sequence, own_len) for i in range(n)], False, dev)
        return prefix, replace(own, seqs=own.seqs.clone())

    def _project(self, x: torch.Tensor, name: str) -> torch.Tensor:
        """``x @ W[name].T`` for inference-only passes: the fp8 copy of the weight if ``enable_fp8_inference`` made one."""
        fp8 = self._fp8_linears.get(name) if self._fp8_linears else None
        return fp8(x) if fp8 is not None else linear(x, self.view(name))

    @torch.no_grad()
    def enable_fp8_inference(self, enabled: bool = True) -> None:
        """Quantise the layer projections to e4m3 codes with one scale per output channel (8 bits per weight more
        memory) for ``decode_step``; training and scoring passes keep using the bf16 weights.  Call again after an
        optimiser step to refresh the copies."""
        self._fp8_linears = {}
        if not enabled:
            return
        from rl_engine.kernels.ops.sm100.gemm_fp8 import Fp8Linear

        for i in range(self.cfg.num_layers):
            for n in ("wqkv", "wo", "w_gate_up", "w_down"):
                self._fp8_linears[f"l{i}.{n}"] = Fp8Linear(self.view(f"l{i}.{n}"))

    def lm_head_weight(self) -> torch.Tensor:
        return self.view("lm_head")

    def forward(self, token_ids: torch.Tensor, positions: torch.Tensor, layout) -> torch.Tensor:
        """Logits ``[T, V]`` (materialised; use ``hidden_states`` + ``linear_logp`` for training)."""
        return linear(self.hidden_states(token_ids, positions, layout), self.lm_head_weight())
