"""MiniCPM4 (``MiniCPMForCausalLM``) as data: which parts, with which constants, under
which tensor names.

Layer structure and scales follow the reference: embedding times ``scale_emb``
(src/model/embedding.cuh:49-52), residual scale ``scale_depth / sqrt(layers)`` on both
parts of every layer (src/model/layer.cuh:47-67, cpmcu/llm.py:69), head scale
``dim_model_base / hidden_size`` (cpmcu/llm.py:68).  Tensor names are those of the
reference's loader (src/model/model.cuh:122-143, src/model/attn.cuh:162-182,
src/model/ffn.cuh:61-75); fused ``qkv_proj`` / ``gate_up_proj`` tensors are split by
rows as cpmcu/llm.py:125-131 does.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.minicpm import MiniCPMConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, default_schedule

LAYER_NAMES = {
    "mixer_norm": "input_layernorm.",
    "mixer": "self_attn.",
    "feed_forward_norm": "post_attention_layernorm.",
    "feed_forward": "mlp.",
}


def position_spec(cfg: MiniCPMConfig) -> PartSpec:
    if cfg.rope_scaling is None:
        return PartSpec("rope", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta})
    rs = cfg.rope_scaling
    return PartSpec("longrope", {
        "head_dim": cfg.head_dim, "theta": cfg.rope_theta,
        "long_factor": tuple(rs.long_factor), "short_factor": tuple(rs.short_factor),
        "original_max_positions": rs.original_max_position_embeddings,
        "max_positions": cfg.max_position_embeddings,
    })


def model_spec(cfg: MiniCPMConfig) -> ModelSpec:
    norm = PartSpec("rms_norm", {"hidden_size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    mixer = PartSpec("gqa_attention", {
        "hidden_size": cfg.hidden_size, "n_heads": cfg.num_attention_heads,
        "n_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "position": position_spec(cfg),
        "sparse": cfg.sparse_config.to_json() if cfg.sparse_config else None,
    })
    ffn = PartSpec("gated_ffn", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                                 "activation": cfg.hidden_act})
    block = PartSpec("pre_norm_residual", {"residual_scale": cfg.residual_scale})
    layers = [
        LayerSpec(block=block, mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=norm,
                  prefix=f"model.layers.{i}.", names=LAYER_NAMES)
        for i in range(cfg.num_hidden_layers)
    ]
    return ModelSpec(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        embedding=PartSpec("scaled_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                                "scale": cfg.scale_emb}),
        layers=layers,
        schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=norm,
        head=PartSpec("scaled_lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size,
                                         "scale": cfg.logit_scale, "tied": cfg.tie_word_embeddings}),
        stop_token_ids=tuple(cfg.eos_token_ids),
        max_positions=cfg.max_position_embeddings,
    )


def split_fused_tensors(cfg: MiniCPMConfig, name: str, tensor: torch.Tensor) -> List[Tuple[str, torch.Tensor]]:
    """Checkpoint names this architecture also accepts, mapped to the canonical ones."""
    if name.endswith("self_attn.qkv_proj.weight"):
        base = name[: -len("qkv_proj.weight")]
        q_rows = cfg.num_attention_heads * cfg.head_dim
        kv_rows = cfg.num_key_value_heads * cfg.head_dim
        if tensor.shape[0] == q_rows + 2 * kv_rows:
            return [(base + "q_proj.weight", tensor[:q_rows]),
                    (base + "k_proj.weight", tensor[q_rows:q_rows + kv_rows]),
                    (base + "v_proj.weight", tensor[q_rows + kv_rows:])]
    if name.endswith("mlp.gate_up_proj.weight"):
        base = name[: -len("gate_up_proj.weight")]
        if tensor.shape[0] == 2 * cfg.intermediate_size:
            return [(base + "gate_proj.weight", tensor[:cfg.intermediate_size]),
                    (base + "up_proj.weight", tensor[cfg.intermediate_size:])]
    return [(name, tensor)]


def ignored_tensor(name: str) -> bool:
    """Tensors a checkpoint may carry that the model computes itself."""
    return name.endswith("rotary_emb.inv_freq")
