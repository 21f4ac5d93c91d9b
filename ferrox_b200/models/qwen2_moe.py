"""Qwen2-MoE as a description made of parts.

The reference runs this architecture (GGUF name ``qwen2moe``) through its generic
decoder: crates/ferrox-models/src/capability.rs:253 (profile), decoder.rs:2054-2205
(one token) and :3224-3670 (a batch of tokens).  Per layer:

    h += Wo . attention(rope(Wq n + bq), rope(Wk n + bk), Wv n + bv),  n = rms_norm(h)
    h += ffn(rms_norm(h))

where ``ffn`` is a dense SwiGLU MLP or the expert block (softmax router over all
experts, top-k, routed SwiGLU experts, a shared SwiGLU expert scaled by a sigmoid
gate; crates/ferrox-moe/src/lib.rs:333-355,619-659,735-752; decoder.rs:2660-2681).

One ``rope_theta`` serves every layer: the reference's switch to another base on
windowed layers (loader.rs:388-399) is a rule of a different model family and is
not taken over.  Tensor names are those of the published checkpoints
(``model.layers.<l>.self_attn.q_proj.weight`` and so on).
"""
from __future__ import annotations

from ..config.qwen2_moe import ARCHITECTURE, Qwen2MoeConfig
from ..config.registry import register_architecture
from ..parts.specs import (
    AttentionSpec,
    BlockSpec,
    DenseMlpSpec,
    ModelSpec,
    MoeSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
)


def model_spec(cfg: Qwen2MoeConfig) -> ModelSpec:
    layers = []
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        mixer = AttentionSpec(
            hidden=cfg.hidden_size,
            n_heads=cfg.num_attention_heads,
            n_kv_heads=cfg.num_key_value_heads,
            head_dim=cfg.head_dim,
            qkv_bias=cfg.qkv_bias,
            position=PositionSpec(rotary_dim=cfg.head_dim, theta=cfg.rope_theta),
            window=cfg.layer_window(l),
            prefix=p + "self_attn.",
        )
        if cfg.layer_is_moe(l):
            ffn = MoeSpec(
                hidden=cfg.hidden_size,
                n_experts=cfg.num_experts,
                top_k=cfg.num_experts_per_tok,
                expert_intermediate=cfg.moe_intermediate_size,
                shared_intermediate=cfg.shared_expert_intermediate_size,
                norm_topk_prob=cfg.norm_topk_prob,
                shared_gate=cfg.shared_expert_intermediate_size > 0,
                prefix=p + "mlp.",
            )
        else:
            ffn = DenseMlpSpec(hidden=cfg.hidden_size, intermediate=cfg.intermediate_size, prefix=p + "mlp.")
        layers.append(
            BlockSpec(
                norm1=NormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "input_layernorm."),
                mixer=mixer,
                norm2=NormSpec(cfg.hidden_size, cfg.rms_norm_eps, p + "post_attention_layernorm."),
                ffn=ffn,
            )
        )
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab_size,
        hidden=cfg.hidden_size,
        max_positions=cfg.max_position_embeddings,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=l, cache=l) for l in range(cfg.num_hidden_layers)),
        final_norm=NormSpec(cfg.hidden_size, cfg.rms_norm_eps, "model.norm."),
        head_name=None if cfg.tie_word_embeddings else "lm_head.weight",
        eos_token_ids=() if cfg.eos_token_id is None else (cfg.eos_token_id,),
    )


register_architecture(ARCHITECTURE, Qwen2MoeConfig.from_json, model_spec, replace=True)
