"""Hugging Face checkpoints <-> ``LlamaModel``.

The reference has no model of its own: its executors and trainers run Hugging Face modules, and its weight bridge ships
``state_dict`` keys ("checkpoint-format names") to vLLM (``rl_engine/executors/bridge.py:206,345``).  The native model of
this library keeps packed parameters in one flat buffer (``wqkv`` = q, k and v rows stacked, ``w_gate_up`` = gate and up
rows stacked, experts stacked by expert), so two things are needed to stand in for a Hugging Face module:

* ``config_from_hf`` / ``load_hf_state_dict``: build the matching ``ModelConfig`` and copy a Llama / Mistral / Mixtral /
  Qwen2 / Qwen3 / Qwen3-MoE ``state_dict`` into the flat buffer (only the local experts of an expert-sharded model);
* ``hf_state_dict_views``: the parameters under their Hugging Face names as zero-copy views (row ranges of the packed
  matrices are contiguous), which is what a weight bridge publishes to a vLLM engine;
* ``save_hf_checkpoint`` / ``load_hf_checkpoint`` / ``model_from_hf_checkpoint``: the same for directories of
  ``config.json`` + (sharded) safetensors files, streamed tensor by tensor.

Rotary embedding (half-split rotation; linear, llama3 and YaRN scaling), RMSNorm (plain weight, eps inside the root),
attention scale, the Qwen2 q/k/v biases, the Qwen3 head norms and the router of both MoE families (softmax over all
experts, top-k, renormalised) follow the Hugging Face implementations, so logits agree (tested
against ``transformers`` on CPU in fp32).
"""

from __future__ import annotations

from typing import Any, Dict, Iterator, List, Mapping, Optional, Tuple

import torch

from rl_engine.models.config import ModelConfig


# a mapping without ``model_type`` is read as the Llama architecture
_MODEL_TYPES = {"", "llama", "mistral", "mixtral", "qwen2", "qwen3", "qwen3_moe"}


def config_from_hf(hf_config: Any, name: str = "") -> ModelConfig:
    """``ModelConfig`` of a Hugging Face configuration object (or mapping) of one of the supported decoder families:
    ``llama`` (Llama-2 / 3 / 3.x), ``mistral`` (no sliding window), ``mixtral``, ``qwen2`` (Qwen2 / 2.5), ``qwen3``,
    ``qwen3_moe``.  Anything this model cannot reproduce exactly raises ``ValueError``: another ``model_type``, an
    unknown rotary scaling, biases outside q/k/v, sliding windows, mixed dense / MoE stacks."""
    get = (lambda k, d=None: hf_config.get(k, d)) if isinstance(hf_config, Mapping) else (lambda k, d=None: getattr(hf_config, k, d))
    hidden, heads = int(get("hidden_size")), int(get("num_attention_heads"))
    head_dim = int(get("head_dim") or hidden // heads)
    scaling = get("rope_scaling") or (get("rope_parameters") if isinstance(get("rope_parameters"), Mapping) else None)
    rope_scaling = None
    kind = (scaling.get("rope_type", scaling.get("type")) if scaling else None) or "default"
    if kind == "linear":
        rope_scaling = ("linear", float(scaling["factor"]), 1.0, 1.0, 0)
    elif kind == "llama3":
        rope_scaling = ("llama3", float(scaling["factor"]), float(scaling.get("low_freq_factor", 1.0)),
                        float(scaling.get("high_freq_factor", 4.0)), int(scaling["original_max_position_embeddings"]))
    elif kind == "yarn":
        if any(scaling.get(k) is not None for k in ("attention_factor", "mscale", "mscale_all_dim")) or scaling.get("truncate") is False:
            raise ValueError(f"YaRN with an explicit attention factor, mscale or without truncation is not supported: {scaling}")
        rope_scaling = ("yarn", float(scaling["factor"]), float(scaling.get("beta_fast") or 32.0),
                        float(scaling.get("beta_slow") or 1.0),
                        int(scaling.get("original_max_position_embeddings") or get("max_position_embeddings")))
    elif kind != "default":
        raise ValueError(f"rope scaling {scaling} is not supported (known: default, linear, llama3, yarn)")
    model_type = str(get("model_type", "") or "")
    if model_type not in _MODEL_TYPES:
        raise ValueError(f"model_type {model_type!r} is not one of the supported decoder families {sorted(_MODEL_TYPES - {''})}")
    qkv_bias = model_type == "qwen2"          # Qwen2 / Qwen2.5: biased q, k, v; no bias on the output projection
    if get("attention_bias", False) or get("mlp_bias", False):
        raise ValueError("biases on the output projection or the FFN are not supported (Qwen2-style q/k/v biases are)")
    window = get("sliding_window")
    if get("use_sliding_window", model_type == "mistral") and window and int(window) < int(get("max_position_embeddings", 0) or 0):
        raise ValueError(f"sliding-window attention (window {window}) is not supported")
    experts = int(get("num_experts", 0) or get("num_local_experts", 0) or 0)
    renormalises = get("norm_topk_prob")
    if experts and not (True if renormalises is None else renormalises):      # Mixtral has no switch: it always does
        raise ValueError("routers that do not renormalise the top-k weights are not supported")
    if experts and (int(get("decoder_sparse_step", 1) or 1) != 1 or get("mlp_only_layers")):
        raise ValueError("models that mix dense and mixture-of-experts layers are not supported")
    rope_theta = get("rope_theta")
    if rope_theta is None and isinstance(get("rope_parameters"), Mapping):
        rope_theta = get("rope_parameters").get("rope_theta")
    return ModelConfig(
        name or model_type or "hf-model", int(get("vocab_size")), hidden, int(get("num_hidden_layers")), heads,
        int(get("num_key_value_heads") or heads), head_dim, int(get("intermediate_size")),
        rms_eps=float(get("rms_norm_eps", 1e-5)), rope_theta=float(rope_theta if rope_theta is not None else 10000.0),
        num_experts=experts, experts_per_token=int(get("num_experts_per_tok", 0) or 0) if experts else 0,
        moe_ffn_size=int(get("moe_intermediate_size", 0) or get("intermediate_size")) if experts else 0,
        qk_norm=model_type.startswith("qwen3"), rope_scaling=rope_scaling,
        tie_word_embeddings=bool(get("tie_word_embeddings", False)), qkv_bias=qkv_bias,
    )


def hf_parameter_map(model) -> Iterator[Tuple[str, List[Tuple[str, int, int]]]]:
    """``(native name, [(hf name, first row, one past the last row)])`` for every parameter of ``model`` (a
    ``LlamaModel``): which rows of the native tensor hold which Hugging Face tensor.  Vectors use element ranges."""
    cfg = model.cfg
    q, kv, f, h = cfg.q_dim, cfg.kv_dim, cfg.ffn_size, cfg.hidden_size
    yield "embed", [("model.embed_tokens.weight", 0, cfg.vocab_size)]
    shard_rank, shard_world = model.expert_shard if model.expert_shard is not None else (0, 1)
    e_local = cfg.num_experts // shard_world if cfg.num_experts else 0
    for i in range(cfg.num_layers):
        p = f"model.layers.{i}."
        yield f"l{i}.attn_norm", [(p + "input_layernorm.weight", 0, h)]
        yield f"l{i}.wqkv", [(p + "self_attn.q_proj.weight", 0, q), (p + "self_attn.k_proj.weight", q, q + kv),
                             (p + "self_attn.v_proj.weight", q + kv, q + 2 * kv)]
        if cfg.qkv_bias:
            yield f"l{i}.bqkv", [(p + "self_attn.q_proj.bias", 0, q), (p + "self_attn.k_proj.bias", q, q + kv),
                                 (p + "self_attn.v_proj.bias", q + kv, q + 2 * kv)]
        yield f"l{i}.wo", [(p + "self_attn.o_proj.weight", 0, h)]
        if cfg.qk_norm:
            yield f"l{i}.q_norm", [(p + "self_attn.q_norm.weight", 0, cfg.head_dim)]
            yield f"l{i}.k_norm", [(p + "self_attn.k_norm.weight", 0, cfg.head_dim)]
        yield f"l{i}.mlp_norm", [(p + "post_attention_layernorm.weight", 0, h)]
        if cfg.num_experts:
            fe = cfg.moe_ffn_size
            # checkpoint names of the two MoE families: Qwen3-MoE (q/k norms) and Mixtral (none)
            block, gate_n, up_n, down_n = (("mlp", "gate_proj", "up_proj", "down_proj") if cfg.qk_norm
                                           else ("block_sparse_moe", "w1", "w3", "w2"))
            yield f"l{i}.router", [(f"{p}{block}.gate.weight", 0, cfg.num_experts)]
            gate_up, down = [], []
            for e in range(e_local):
                ep = f"{p}{block}.experts.{shard_rank * e_local + e}."
                gate_up += [(ep + f"{gate_n}.weight", e * 2 * fe, e * 2 * fe + fe),
                            (ep + f"{up_n}.weight", e * 2 * fe + fe, (e + 1) * 2 * fe)]
                down.append((ep + f"{down_n}.weight", e * h, (e + 1) * h))
            yield f"l{i}.w_gate_up", gate_up
            yield f"l{i}.w_down", down
        else:
            yield f"l{i}.w_gate_up", [(p + "mlp.gate_proj.weight", 0, f), (p + "mlp.up_proj.weight", f, 2 * f)]
            yield f"l{i}.w_down", [(p + "mlp.down_proj.weight", 0, h)]
    yield "final_norm", [("model.norm.weight", 0, h)]
    yield "lm_head", [("lm_head.weight", 0, cfg.vocab_size)]


def hf_state_dict_views(model) -> Dict[str, torch.Tensor]:
    """The parameters of ``model`` under their Hugging Face names, as views of the flat buffer (no copies)."""
    out: Dict[str, torch.Tensor] = {}
    for native, pieces in hf_parameter_map(model):
        tensor = model.view(native).detach()
        for hf_name, lo, hi in pieces:
            out[hf_name] = tensor[lo:hi]
    return out


@torch.no_grad()
def load_hf_state_dict(model, state_dict: Mapping[str, torch.Tensor], *, strict: bool = True) -> List[str]:
    """Copies a Hugging Face ``state_dict`` into ``model`` (cast to its dtype).  A missing ``lm_head.weight`` is taken from
    the embedding (tied weights).  Returns the Hugging Face names that were not used (experts of other shards, buffers);
    with ``strict`` a missing or mis-shaped tensor raises ``KeyError`` / ``ValueError``."""
    used = set()
    cfg = model.cfg
    shard_rank, shard_world = model.expert_shard if model.expert_shard is not None else (0, 1)
    e_local = cfg.num_experts // shard_world if cfg.num_experts else 0
    for native, pieces in hf_parameter_map(model):
        dst = model.view(native)
        if cfg.num_experts and native.endswith((".w_gate_up", ".w_down")):
            # newer ``transformers`` keep a layer's experts as two stacked tensors, ``experts.gate_up_proj [E, 2F, H]``
            # and ``experts.down_proj [E, H, F]``: the native layout, expert by expert
            layer = native.split(".")[0][1:]
            fused = f"model.layers.{layer}.mlp.experts." + ("gate_up_proj" if native.endswith("w_gate_up") else "down_proj")
            if fused in state_dict:
                src = state_dict[fused][shard_rank * e_local : (shard_rank + 1) * e_local]
                src = src.reshape(-1, src.shape[-1])
                if tuple(src.shape) != tuple(dst.shape):
                    raise ValueError(f"{fused} gives {tuple(src.shape)} for this shard, {native} needs {tuple(dst.shape)}")
                dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
                used.add(fused)
                continue
        for hf_name, lo, hi in pieces:
            src = state_dict.get(hf_name)
            if src is None and ".block_sparse_moe.gate." in hf_name:     # newer transformers rename Mixtral's block
                hf_name = hf_name.replace(".block_sparse_moe.", ".mlp.")
                src = state_dict.get(hf_name)
            if src is None and hf_name == "lm_head.weight":
                src = state_dict.get("model.embed_tokens.weight")
            if src is None:
                if strict:
                    raise KeyError(f"{hf_name} is missing from the state dict (needed for {native})")
                continue
            part = dst[lo:hi]
            if tuple(src.shape) != tuple(part.shape):
                raise ValueError(f"{hf_name} has shape {tuple(src.shape)}, {native}[{lo}:{hi}] needs {tuple(part.shape)}")
            part.copy_(src.to(device=part.device, dtype=part.dtype))
            used.add(hf_name)
    return sorted(k for k in state_dict if k not in used)


def model_from_hf(hf_model, *, dtype: torch.dtype = torch.bfloat16, device="cuda", expert_shard=None, **model_kwargs):
    """A ``LlamaModel`` with the architecture and the weights of a Hugging Face causal LM (``LlamaForCausalLM``,
    ``Qwen3ForCausalLM``, ``Qwen3MoeForCausalLM``).  ``model_kwargs`` go to ``LlamaModel`` (``max_positions``, ...)."""
    from rl_engine.models.llama import LlamaModel

    cfg = config_from_hf(hf_model.config)
    model_kwargs.setdefault("max_positions", int(getattr(hf_model.config, "max_position_embeddings", 0) or 8192))
    model = LlamaModel(cfg, dtype=dtype, device=device, expert_shard=expert_shard, **model_kwargs)
    load_hf_state_dict(model, hf_model.state_dict())
    return model


# ---- checkpoints on disk (``config.json`` + ``*.safetensors``, optionally sharded with an index) -------------------
_INDEX_NAME = "model.safetensors.index.json"


def hf_config_dict(cfg: ModelConfig, *, dtype: torch.dtype = torch.bfloat16, max_position_embeddings: int = 8192,
                   tie_word_embeddings: Optional[bool] = None) -> Dict[str, Any]:
    """The ``config.json`` of ``cfg``: the inverse of ``config_from_hf`` (Llama, Qwen3 and Qwen3-MoE architectures).
    ``tie_word_embeddings`` defaults to the configuration's own flag."""
    if tie_word_embeddings is None:
        tie_word_embeddings = cfg.tie_word_embeddings
    moe, qwen = bool(cfg.num_experts), bool(cfg.qk_norm)
    if cfg.qkv_bias and (moe or qwen or cfg.head_dim * cfg.num_heads != cfg.hidden_size):
        raise ValueError("biased q/k/v projections are written as Qwen2, which has neither experts nor q/k norms and "
                         "takes head_dim = hidden_size / heads")
    arch, kind = (("Qwen3MoeForCausalLM", "qwen3_moe") if moe and qwen else ("MixtralForCausalLM", "mixtral") if moe
                  else ("Qwen3ForCausalLM", "qwen3") if qwen
                  else ("Qwen2ForCausalLM", "qwen2") if cfg.qkv_bias else ("LlamaForCausalLM", "llama"))
    out: Dict[str, Any] = {
        "architectures": [arch], "model_type": kind, "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
        "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads,
        "head_dim": cfg.head_dim, "intermediate_size": cfg.ffn_size, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta,
        "hidden_act": "silu", "max_position_embeddings": int(max_position_embeddings),
        "tie_word_embeddings": bool(tie_word_embeddings), "torch_dtype": str(dtype).replace("torch.", ""),
        "dtype": str(dtype).replace("torch.", ""),
    }
    if kind == "llama":
        out["mlp_bias"] = False
    if kind != "qwen2":
        out["attention_bias"] = False
    else:
        out.pop("head_dim")
        out["use_sliding_window"] = False
    if cfg.rope_scaling is not None:
        how, factor, low, high, original = cfg.rope_scaling
        block = {"rope_type": how, "factor": factor}
        if how == "llama3":
            block.update(low_freq_factor=low, high_freq_factor=high, original_max_position_embeddings=original)
        if how == "yarn":
            block.update(beta_fast=low, beta_slow=high, original_max_position_embeddings=original)
        out["rope_scaling"] = dict(block)
        out["rope_parameters"] = dict(block, rope_theta=cfg.rope_theta)      # the spelling of newer transformers
    if kind == "qwen3_moe":
        out.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.experts_per_token, moe_intermediate_size=cfg.moe_ffn_size,
                   norm_topk_prob=True, decoder_sparse_step=1, mlp_only_layers=[])
    if kind == "mixtral":
        out.update(num_local_experts=cfg.num_experts, num_experts_per_tok=cfg.experts_per_token,
                   intermediate_size=cfg.moe_ffn_size, sliding_window=None)
    return out


def save_hf_checkpoint(model, directory, *, max_shard_bytes: int = 5 << 30, tie_word_embeddings: Optional[bool] = None,
                       max_position_embeddings: int = 0) -> List[str]:
    """Writes ``model`` (all experts local) as a Hugging Face checkpoint: ``config.json`` plus one or more
    ``model-xxxxx-of-yyyyy.safetensors`` files cut at ``max_shard_bytes`` and the index that maps names to files.
    Tensors are the zero-copy checkpoint-name views, so one shard at a time is staged on the host.  Returns the
    file names written.  ``transformers`` and vLLM load the directory directly."""
    import json
    import os

    from safetensors.torch import save_file

    if model.expert_shard is not None and model.expert_shard[1] > 1:
        raise ValueError("an expert-sharded model holds only its own experts; gather them before saving")
    os.makedirs(directory, exist_ok=True)
    views = hf_state_dict_views(model)
    if tie_word_embeddings is None:
        tie_word_embeddings = model.cfg.tie_word_embeddings
    if tie_word_embeddings:
        views.pop("lm_head.weight")
    shards: List[List[str]] = [[]]
    used = 0
    for name, t in views.items():
        nbytes = t.numel() * t.element_size()
        if shards[-1] and used + nbytes > max_shard_bytes:
            shards.append([])
            used = 0
        shards[-1].append(name)
        used += nbytes
    files, weight_map, total = [], {}, 0
    for i, names in enumerate(shards):
        fname = "model.safetensors" if len(shards) == 1 else f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        save_file({n: views[n].detach().to("cpu").contiguous() for n in names}, os.path.join(directory, fname),
                  metadata={"format": "pt"})
        files.append(fname)
        for n in names:
            weight_map[n] = fname
            total += views[n].numel() * views[n].element_size()
    if len(shards) > 1:
        with open(os.path.join(directory, _INDEX_NAME), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1, sort_keys=True)
        files.append(_INDEX_NAME)
    positions = max_position_embeddings or int(model.rope_cos.shape[0])
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(hf_config_dict(model.cfg, dtype=model.flat.dtype, max_position_embeddings=positions,
                                 tie_word_embeddings=tie_word_embeddings), f, indent=1, sort_keys=True)
    return files + ["config.json"]


def checkpoint_files(directory) -> List[str]:
    """The ``*.safetensors`` files of a checkpoint directory (from the index when there is one), sorted."""
    import json
    import os

    index = os.path.join(directory, _INDEX_NAME)
    if os.path.exists(index):
        with open(index) as f:
            return sorted(set(json.load(f)["weight_map"].values()))
    found = sorted(f for f in os.listdir(directory) if f.endswith(".safetensors"))
    if not found:
        raise FileNotFoundError(f"no .safetensors file in {directory}")
    return found


@torch.no_grad()
def load_hf_checkpoint(model, directory, *, strict: bool = True) -> List[str]:
    """Streams a checkpoint directory into ``model`` one tensor at a time (memory-mapped safetensors, no full state
    dict on the host): every name is routed to its rows of the flat buffer by ``hf_parameter_map``.  Handles tied
    embeddings, per-expert and stacked expert tensors, and expert shards like ``load_hf_state_dict``.  Returns the names
    that were not used; with ``strict`` a parameter that no file provides raises ``KeyError``."""
    import os

    from safetensors import safe_open

    cfg = model.cfg
    shard_rank, shard_world = model.expert_shard if model.expert_shard is not None else (0, 1)
    e_local = cfg.num_experts // shard_world if cfg.num_experts else 0
    route: Dict[str, Tuple[str, int, int]] = {}
    alias: Dict[str, str] = {}                  # other spellings of a routed name -> the routed name
    for native, pieces in hf_parameter_map(model):
        for hf_name, lo, hi in pieces:
            route[hf_name] = (native, lo, hi)
            if ".block_sparse_moe.gate." in hf_name:
                alias[hf_name.replace(".block_sparse_moe.", ".mlp.")] = hf_name
    stacked = {}
    if cfg.num_experts:
        for i in range(cfg.num_layers):
            stacked[f"model.layers.{i}.mlp.experts.gate_up_proj"] = f"l{i}.w_gate_up"
            stacked[f"model.layers.{i}.mlp.experts.down_proj"] = f"l{i}.w_down"
    filled, unused, embed_seen = set(), [], False
    for fname in checkpoint_files(directory):
        with safe_open(os.path.join(directory, fname), framework="pt", device="cpu") as f:
            for name in f.keys():
                if name in stacked:
                    dst = model.view(stacked[name])
                    src = f.get_slice(name)[shard_rank * e_local : (shard_rank + 1) * e_local]
                    src = src.reshape(-1, src.shape[-1])
                    if tuple(src.shape) != tuple(dst.shape):
                        raise ValueError(f"{name} gives {tuple(src.shape)} for this shard, {stacked[name]} needs {tuple(dst.shape)}")
                    dst.copy_(src.to(device=dst.device, dtype=dst.dtype))
                    filled.update(h for h, (nat, _lo, _hi) in route.items() if nat == stacked[name])
                    continue
                src_name, name = name, alias.get(name, name)
                if name not in route:
                    unused.append(name)
                    continue
                native, lo, hi = route[name]
                part = model.view(native)[lo:hi]
                src = f.get_tensor(src_name)
                if tuple(src.shape) != tuple(part.shape):
                    raise ValueError(f"{name} has shape {tuple(src.shape)}, {native}[{lo}:{hi}] needs {tuple(part.shape)}")
                part.copy_(src.to(device=part.device, dtype=part.dtype))
                filled.add(name)
                embed_seen |= name == "model.embed_tokens.weight"
    if "lm_head.weight" not in filled and embed_seen:          # tied embeddings: the head is the embedding
        model.view("lm_head").copy_(model.view("embed"))
        filled.add("lm_head.weight")
    missing = sorted(set(route) - filled)
    if missing and strict:
        raise KeyError(f"the checkpoint in {directory} lacks {missing[:4]}{' ...' if len(missing) > 4 else ''}")
    return sorted(unused)


def model_from_hf_checkpoint(directory, *, dtype: torch.dtype = torch.bfloat16, device="cuda", expert_shard=None,
                             **model_kwargs):
    """A ``LlamaModel`` built from ``config.json`` and filled from the safetensors files of ``directory``."""
    import json
    import os

    from rl_engine.models.llama import LlamaModel

    with open(os.path.join(directory, "config.json")) as f:
        raw = json.load(f)
    model_kwargs.setdefault("max_positions", int(raw.get("max_position_embeddings", 0) or 8192))
    model = LlamaModel(config_from_hf(raw), dtype=dtype, device=device, expert_shard=expert_shard, **model_kwargs)
    load_hf_checkpoint(model, directory)
    return model
