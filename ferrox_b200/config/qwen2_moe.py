"""Typed configuration of ``Qwen2MoeForCausalLM``, read from its own config.json keys.

The reference reads the same hyper-parameters from GGUF metadata
(crates/ferrox-models/src/loader.rs:117-470; key by key: block_count :168-170,
embedding_length :171-174, head counts :175-188, key_length :189-197, vocab :211-227,
rope.freq_base :228-231, rms epsilon :232-243, expert counts :245-256, expert widths
:262-294, sliding_window :339-341).  The checkpoint convention used here is the
``config.json`` that ships with the model; the mapping of keys is one to one.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from typing import Optional, Tuple

from .schema import REQUIRED, ConfigError, Key, non_negative, positive, read_keys

ARCHITECTURE = "Qwen2MoeForCausalLM"

_SCHEMA = (
    Key("num_hidden_layers", int, check=positive),
    Key("hidden_size", int, check=positive),
    Key("num_attention_heads", int, check=positive),
    Key("num_key_value_heads", int, default=lambda v: v["num_attention_heads"], check=positive),
    Key("head_dim", int, default=lambda v: v["hidden_size"] // v["num_attention_heads"], check=positive),
    Key("vocab_size", int, check=positive),
    Key("max_position_embeddings", int, check=positive),
    Key("rope_theta", float, default=10000.0, check=positive),
    Key("rms_norm_eps", float, default=1e-6, check=positive),
    Key("num_experts", int, default=0, check=non_negative),
    Key("num_experts_per_tok", int, default=lambda v: min(2, v["num_experts"]), check=non_negative),
    Key("moe_intermediate_size", int, default=0, check=non_negative),
    Key("shared_expert_intermediate_size", int, default=0, check=non_negative),
    Key("intermediate_size", int, default=0, check=non_negative),
    Key("decoder_sparse_step", int, default=1, check=positive),
    Key("mlp_only_layers", list, default=lambda v: []),
    Key("norm_topk_prob", bool, default=False),
    Key("qkv_bias", bool, default=True),
    Key("use_sliding_window", bool, default=False),
    Key("sliding_window", int, default=None, nullable=True, check=positive),
    Key("max_window_layers", int, default=lambda v: v["num_hidden_layers"], check=non_negative),
    Key("tie_word_embeddings", bool, default=False),
    Key("hidden_act", str, default="silu"),
    Key("eos_token_id", int, default=None, nullable=True),
    Key("bos_token_id", int, default=None, nullable=True),
    # keys of this family's config.json that change the arithmetic and are implemented in one setting only
    Key("rope_scaling", object, default=None, nullable=True,
        check=lambda v: "scaled rotary positions are not implemented (only null)"),
    Key("partial_rotary_factor", float, default=1.0,
        check=lambda v: None if v == 1.0 else "a rotary width below head_dim is not implemented (only 1.0)"),
    Key("attention_bias", bool, default=None, nullable=True),   # another spelling of qkv_bias; must agree with it
    Key("attention_dropout", float, default=0.0, check=non_negative),  # training only
    Key("mlp_bias", bool, default=False, check=lambda v: "a bias in the feed-forward is not implemented" if v else None),
)

# Keys a checkpoint's config.json carries that do not concern inference.
_BOOKKEEPING = (
    "architectures", "model_type", "torch_dtype", "dtype", "transformers_version", "_name_or_path", "use_cache",
    "initializer_range", "output_router_logits", "router_aux_loss_coef", "pad_token_id", "auto_map", "id2label",
    "label2id", "return_dict", "output_attentions", "output_hidden_states", "is_decoder", "use_bfloat16",
    "tokenizer_class", "task_specific_params", "problem_type", "chunk_size_feed_forward", "tie_encoder_decoder",
    )


@dataclass(frozen=True)
class Qwen2MoeConfig:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int
    rope_theta: float
    rms_norm_eps: float
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    intermediate_size: int
    decoder_sparse_step: int
    mlp_only_layers: Tuple[int, ...]
    norm_topk_prob: bool
    qkv_bias: bool
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    tie_word_embeddings: bool
    hidden_act: str
    eos_token_id: Optional[int]
    bos_token_id: Optional[int]

    # ---- per-layer questions (reference: config.rs:247-277) ----------------
    def layer_is_moe(self, layer: int) -> bool:
        """A layer has experts unless it is listed in ``mlp_only_layers``, the model
        has no experts, or ``decoder_sparse_step`` skips it."""
        if self.num_experts == 0 or layer in self.mlp_only_layers:
            return False
        return (layer + 1) % self.decoder_sparse_step == 0

    def layer_window(self, layer: int) -> Optional[int]:
        """Layers at index >= ``max_window_layers`` see only the last
        ``sliding_window`` positions when ``use_sliding_window`` is set."""
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    # ---- JSON ---------------------------------------------------------------
    @classmethod
    def from_json(cls, obj: dict) -> "Qwen2MoeConfig":
        v = read_keys(obj, _SCHEMA, ignore=_BOOKKEEPING)
        problems = []
        if v["attention_bias"] is not None and v["attention_bias"] != v["qkv_bias"]:
            problems.append(f"attention_bias={v['attention_bias']} contradicts qkv_bias={v['qkv_bias']}")
        for k in ("rope_scaling", "partial_rotary_factor", "attention_bias", "attention_dropout", "mlp_bias"):
            v.pop(k)
        if v["head_dim"] % 2:
            problems.append("head_dim must be even (rotary pairs)")
        if v["num_attention_heads"] % v["num_key_value_heads"]:
            problems.append("num_attention_heads must be a multiple of num_key_value_heads")
        if v["hidden_act"] != "silu":
            problems.append(f"hidden_act={v['hidden_act']!r}: only 'silu' is implemented")
        for l in v["mlp_only_layers"]:
            if isinstance(l, bool) or not isinstance(l, int) or not 0 <= l < v["num_hidden_layers"]:
                problems.append(f"mlp_only_layers: {l!r} is not a layer index")
        v["mlp_only_layers"] = tuple(v["mlp_only_layers"])
        if v["use_sliding_window"] and not v["sliding_window"]:
            problems.append("use_sliding_window is true but sliding_window is not given")
        if not problems:
            cfg = cls(**v)
            any_moe = any(cfg.layer_is_moe(l) for l in range(cfg.num_hidden_layers))
            any_dense = not all(cfg.layer_is_moe(l) for l in range(cfg.num_hidden_layers))
            if any_moe:
                if cfg.moe_intermediate_size <= 0:
                    problems.append("moe_intermediate_size: required by the layers with experts")
                if not 0 < cfg.num_experts_per_tok <= cfg.num_experts:
                    problems.append("num_experts_per_tok must lie in 1..num_experts")
            if any_dense and cfg.intermediate_size <= 0:
                problems.append("intermediate_size: required by the dense layers")
        if problems:
            raise ConfigError("config.json: " + "; ".join(problems))
        return cfg

    def to_json(self) -> dict:
        d = asdict(self)
        d["mlp_only_layers"] = list(self.mlp_only_layers)
        d["architectures"] = [ARCHITECTURE]
        d["model_type"] = "qwen2_moe"
        return d

    def dumps(self) -> str:
        return json.dumps(self.to_json(), indent=2)
