"""Native rollout engine: G completions of one prompt with prefix-shared attention and the fused sampler.

On the fused path the prompt is processed once and every decoding step runs the model on the G new tokens against a
per-layer key / value cache (``LlamaModel.decode_step``, optionally with fp8 copies of the layer projections); the
fallback keeps no state and re-runs the packed forward ``[prompt | completion_0 | ...]`` every step (the same
"stateless" trade the scoring executor makes).  Both draw the next token of every completion with the
``sample_topk_topp`` kernel.  Rollout log-probs come from ``linear_logp``, the kernel the trainer
differentiates, so training-time and rollout-time log-probs of the same tokens agree bitwise.
The reference has no rollout engine of its own (it delegates to vLLM).
"""

from __future__ import annotations

from typing import Any, Dict, Optional

import torch


class NativeRolloutEngine:
    """``use_kv_cache`` (default: whenever the model supports it): the prompt is processed once, every decoding step
    runs the model on the G new tokens only and attends to per-layer key / value buffers ``[prompt | G x max_new]``.
    ``fp8_linears``: the cached path multiplies with e4m3 copies of the layer projections (refresh them with
    ``model.enable_fp8_inference()`` after weight updates).  Without the cache every step re-runs the packed forward."""

    def __init__(self, model: torch.nn.Module, seed: int = 0, use_kv_cache: Optional[bool] = None,
                 fp8_linears: bool = False, use_cuda_graph: bool = True) -> None:
        self.model = model
        self.seed = seed
        self._offset = 0
        self.use_cuda_graph = use_cuda_graph
        supported = getattr(model, "supports_prefix_cache", None)
        can_cache = bool(supported is not None and supported())
        self.use_kv_cache = can_cache if use_kv_cache is None else bool(use_kv_cache)
        if self.use_kv_cache and not can_cache:
            raise ValueError("this model does not support key / value cached decoding")
        if fp8_linears:
            if not self.use_kv_cache:
                raise ValueError("fp8_linears needs the key / value cached path")
            model.enable_fp8_inference()

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, *, num_generations: int, max_new_tokens: int, temperature: float = 1.0,
                 top_k: Optional[int] = 50, top_p: Optional[float] = 1.0) -> Dict[str, Any]:
        if self.use_kv_cache:
            return self._generate_cached(prompt_ids, num_generations, max_new_tokens, temperature, top_k, top_p)
        return self._generate_stateless(prompt_ids, num_generations, max_new_tokens, temperature, top_k, top_p)

    def _generate_cached(self, prompt_ids, g: int, max_new_tokens: int, temperature, top_k, top_p) -> Dict[str, Any]:
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.kernels.sampling import SamplerBackend

        model = self.model
        dev = model.flat.device
        prompt = prompt_ids.to(dev).long().reshape(-1)
        p = prompt.numel()
        sampler = SamplerBackend(seed=self.seed)
        sampler._offset = self._offset
        head = model.lm_head_weight()
        lm_head = kernel_registry.get_op("lm_head")
        draw = lambda hidden: sampler.sample(lm_head(hidden, head), top_k=top_k, top_p=top_p, temperature=temperature)
        # prompt pass: last hidden state (predicts the first token of every completion) and per-layer keys / values
        last_state, prompt_kv = model.prefix_states(prompt)
        cache = model.new_kv_cache(p + g * max_new_tokens)
        for (ck, cv), (pk, pv) in zip(cache, prompt_kv):
            ck[:p].copy_(pk)
            cv[:p].copy_(pv)
        del prompt_kv
        completions = torch.empty(g, max_new_tokens, dtype=torch.long, device=dev)
        tokens = draw(last_state.expand(g, -1).contiguous()).reshape(g)
        # Step state lives in fixed device tensors that are advanced in place, so that one decoding step (some 14
        # launches per layer, launch-bound at G tokens) can be captured once as a CUDA graph and replayed per token:
        # the token drawn at `step` sits at position p + step and in cache row base + step; its one-token query sees
        # the prompt rows and its own rows so far (sk_len = step + 1, column 5 of the layout table).
        step_tokens = tokens.clone()
        positions = torch.full((g,), p, dtype=torch.long, device=dev)
        slots = p + torch.arange(g, device=dev) * max_new_tokens
        prefix_layout, layout = model.decode_layouts(g, p, max_new_tokens)
        run_step = lambda: model.decode_step(step_tokens, positions, cache, slots, prefix_layout, layout)
        graph, hidden = None, None
        for step in range(max_new_tokens):
            completions[:, step] = tokens
            if step + 1 == max_new_tokens:
                break
            step_tokens.copy_(tokens)
            if graph is None and self.use_cuda_graph and step == 1:
                # step 0 ran eagerly (it also warmed up every kernel); capture from step 1 on
                graph, hidden = self._capture(run_step)
            if graph is not None:
                graph.replay()
            else:
                hidden = run_step()
            tokens = draw(hidden).reshape(g)
            positions += 1
            slots += 1
            layout.seqs[:, 5] += 1
        self._offset = sampler._offset
        logps = self.score(prompt, completions)
        return {"prompt_ids": prompt, "completion_ids": completions, "rollout_logps": logps}

    @staticmethod
    def _capture(run_step):
        """Capture one decoding step; ``(None, None)`` if capture is not possible here (the caller then runs eagerly)."""
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                hidden = run_step()
            return graph, hidden
        except RuntimeError:
            torch.cuda.synchronize()
            return None, None

    def _generate_stateless(self, prompt_ids, num_generations: int, max_new_tokens: int, temperature, top_k,
                            top_p) -> Dict[str, Any]:
        from rl_engine.kernels.ops.sm100.attention import grpo_group_layout
        from rl_engine.kernels.registry import kernel_registry
        from rl_engine.kernels.sampling import SamplerBackend

        model = self.model
        dev = model.flat.device
        prompt = prompt_ids.to(dev).long().reshape(-1)
        p, g = prompt.numel(), num_generations
        sampler = SamplerBackend(seed=self.seed)
        sampler._offset = self._offset
        completions = torch.zeros(g, 0, dtype=torch.long, device=dev)
        head = model.lm_head_weight()
        for step in range(max_new_tokens):
            l = completions.shape[1]
            if l == 0:
                layout = grpo_group_layout(p, 0, 1, dev)
                tokens, positions = prompt, torch.arange(p, device=dev)
                rows = torch.full((g,), p - 1, device=dev)
            else:
                layout = grpo_group_layout(p, g, l, dev)
                tokens = torch.cat([prompt, completions.reshape(-1)])
                positions = torch.cat([torch.arange(p, device=dev), (p + torch.arange(l, device=dev)).repeat(g)])
                rows = p + torch.arange(g, device=dev) * l + (l - 1)
            hidden = model.hidden_states(tokens, positions, layout)
            last = hidden.index_select(0, rows)
            logits = kernel_registry.get_op("lm_head")(last, head)
            nxt = sampler.sample(logits, top_k=top_k, top_p=top_p, temperature=temperature)
            completions = torch.cat([completions, nxt.reshape(g, 1)], dim=1)
        self._offset = sampler._offset
        logps = self.score(prompt, completions)
        return {"prompt_ids": prompt, "completion_ids": completions, "rollout_logps": logps}

    @torch.no_grad()
    def score(self, prompt: torch.Tensor, completions: torch.Tensor) -> torch.Tensor:
        """Log-probs of ``completions [G, L]`` under the current weights, via the training-path kernels."""
        from rl_engine.models.grpo import GRPOBatch, policy_logps

        g, l = completions.shape
        zeros = torch.zeros(g, l, device=prompt.device)
        batch = GRPOBatch(prompt, completions, torch.zeros(g, device=prompt.device), zeros, zeros,
                          torch.ones(g, l, dtype=torch.bool, device=prompt.device))
        return policy_logps(self.model, batch)
