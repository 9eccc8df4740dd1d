"""Qwen1.5-MoE (``Qwen2MoeForCausalLM``) as a plan of parts.

A pre-norm decoder: RMSNorm -> grouped-query attention with q/k/v bias and half-split
rotary encoding -> residual -> RMSNorm -> sparse mixture of experts (with a sigmoid-gated
shared expert) or, on dense layers, a SwiGLU MLP -> residual; final RMSNorm; linear head,
optionally tied to the embedding.  The reference builds the same model as GGUF architecture
``qwen2moe`` (src/locus/model/arch.cpp:544-696, registry entry arch.cpp:854-858); tensor
names here are those of the safetensors checkpoint (``model.layers.N.self_attn.q_proj.weight``
and so on) instead of GGUF's.
"""
from __future__ import annotations

from ..config.base import ArchEntry, register_arch
from ..config.qwen2_moe import Qwen2MoeConfig
from ..parts.base import LayerCall, LayerSpec, ModelPlan, PartSpec


def build_plan(cfg: Qwen2MoeConfig) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = PartSpec("attention", {
            "hidden": cfg.hidden_size,
            "n_heads": cfg.num_attention_heads,
            "n_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim,
            "qkv_bias": cfg.qkv_bias,
            "o_bias": False,
            "window": cfg.layer_window(l),
            "position": PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta}),
        })
        if cfg.is_moe_layer(l):
            ff = PartSpec("sparse_moe", {
                "hidden": cfg.hidden_size,
                "n_experts": cfg.num_experts,
                "top_k": cfg.num_experts_per_tok,
                "norm_topk": cfg.norm_topk_prob,
                "expert_intermediate": cfg.moe_intermediate_size,
                "shared_intermediate": cfg.shared_expert_intermediate_size,
                "shared_gate": True,
            })
        else:
            ff = PartSpec("dense_mlp", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size})
        layers.append(LayerSpec(
            prefix=f"model.layers.{l}",
            arrangement=PartSpec("pre_norm", {"hidden": cfg.hidden_size}),
            norm=norm, mixer=mixer, feed_forward=ff,
        ))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        eos_token_id=cfg.eos_token_id,
        embedding=PartSpec("embedding", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size,
                                         "prefix": "model.embed_tokens"}),
        layers=layers,
        order=[LayerCall(l) for l in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps, "prefix": "model.norm"}),
        head=PartSpec("linear", {"vocab": cfg.vocab_size, "hidden": cfg.hidden_size, "prefix": "lm_head",
                                 "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else ""}),
        config=cfg,
        # checkpoints of this family may carry the rotary tables, and a copy of the head even when it is tied
        ignorable_tensors=("*.rotary_emb.inv_freq",) + (("lm_head.weight",) if cfg.tie_word_embeddings else ()),
    )


register_arch(ArchEntry(
    name="Qwen2MoeForCausalLM",
    description="Qwen1.5-MoE / Qwen2-MoE: GQA attention with q/k/v bias and rotary encoding; "
                "softmax top-k routed SwiGLU experts with a sigmoid-gated shared expert; dense layers "
                "by decoder_sparse_step / mlp_only_layers",
    parse_config=Qwen2MoeConfig.from_dict,
    build_plan=build_plan,
))
