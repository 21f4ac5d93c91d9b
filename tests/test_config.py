"""Typed configuration and the architecture registry."""
import copy

import pytest

from ferrox_b200 import ConfigError, known_architectures, resolve
from ferrox_b200.config.qwen2_moe import Qwen2MoeConfig
from tiny_configs import TINY_A, TINY_B, TINY_C


def test_reads_every_key_of_tiny_b():
    cfg, spec = resolve(TINY_B)
    assert isinstance(cfg, Qwen2MoeConfig)
    assert (cfg.num_hidden_layers, cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads) == (3, 128, 2, 1)
    assert cfg.head_dim == 64 and cfg.vocab_size == 384 and cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6
    assert [cfg.layer_is_moe(l) for l in range(3)] == [False, True, False]
    assert [cfg.layer_window(l) for l in range(3)] == [None, 16, 16]
    kinds = [type(b.ffn).__name__ for b in spec.layers]
    assert kinds == ["DenseMlpSpec", "MoeSpec", "DenseMlpSpec"]
    assert spec.layers[1].ffn.norm_topk_prob and spec.layers[1].ffn.top_k == 3
    assert spec.head_name is None  # tied
    assert [b.mixer.window for b in spec.layers] == [None, 16, 16]
    assert all(b.mixer.position.theta == 1e6 for b in spec.layers)  # one theta for every layer


def test_defaults():
    obj = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta", "rms_norm_eps",
                                                       "decoder_sparse_step", "mlp_only_layers", "qkv_bias")}
    cfg, _ = resolve(obj)
    assert cfg.num_key_value_heads == cfg.num_attention_heads
    assert cfg.head_dim == cfg.hidden_size // cfg.num_attention_heads
    assert cfg.rope_theta == 10000.0 and cfg.rms_norm_eps == 1e-6 and cfg.qkv_bias is True
    assert cfg.decoder_sparse_step == 1 and cfg.mlp_only_layers == ()


def test_head_dim_need_not_divide_hidden():
    cfg, spec = resolve(TINY_C)
    assert cfg.head_dim * cfg.num_attention_heads != cfg.hidden_size
    assert spec.layers[0].mixer.head_dim == 48


@pytest.mark.parametrize("key", ["num_hidden_layers", "hidden_size", "vocab_size", "num_attention_heads",
                                 "max_position_embeddings"])
def test_missing_required_key_is_named(key):
    obj = copy.deepcopy(TINY_A)
    del obj[key]
    with pytest.raises(ConfigError, match=key):
        resolve(obj)


def test_all_problems_in_one_error():
    obj = copy.deepcopy(TINY_A)
    obj["hidden_size"] = "big"
    obj["vocab_size"] = -3
    del obj["num_hidden_layers"]
    with pytest.raises(ConfigError) as e:
        resolve(obj)
    msg = str(e.value)
    assert "hidden_size" in msg and "vocab_size" in msg and "num_hidden_layers" in msg


def test_inconsistent_values():
    obj = dict(TINY_A, num_key_value_heads=3)
    with pytest.raises(ConfigError, match="multiple"):
        resolve(obj)
    obj = dict(TINY_A, use_sliding_window=True)
    with pytest.raises(ConfigError, match="sliding_window"):
        resolve(obj)
    obj = dict(TINY_B, intermediate_size=0)
    with pytest.raises(ConfigError, match="intermediate_size"):
        resolve(obj)
    obj = dict(TINY_A, num_experts_per_tok=9)
    with pytest.raises(ConfigError, match="num_experts_per_tok"):
        resolve(obj)


def test_unknown_architecture_fails_closed():
    with pytest.raises(ConfigError, match="LlamaForCausalLM") as e:
        resolve(dict(TINY_A, architectures=["LlamaForCausalLM"]))
    assert "Qwen2MoeForCausalLM" in str(e.value)
    assert "Qwen2MoeForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="architectures"):
        resolve({k: v for k, v in TINY_A.items() if k != "architectures"})


def test_round_trip_through_json():
    cfg, _ = resolve(TINY_B)
    again, _ = resolve(cfg.to_json())
    assert again == cfg


@pytest.mark.parametrize("extra,named", [
    ({"rope_scaling": {"type": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768}}, "rope_scaling"),
    ({"partial_rotary_factor": 0.5}, "partial_rotary_factor"),
    ({"attention_bias": False}, "attention_bias"),          # contradicts qkv_bias=true
    ({"mlp_bias": True}, "mlp_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"rope_parameters": {"rope_theta": 5e5}}, "rope_parameters"),   # a key this engine does not know at all
    ({"attn_logit_softcapping": 30.0}, "attn_logit_softcapping"),
])
def test_a_configuration_that_asks_for_what_is_not_implemented_is_refused(extra, named):
    """Keys that change the arithmetic and are not built, and keys the engine has never heard of, are refused by
    name instead of being ignored (wrong logits otherwise)."""
    with pytest.raises(ConfigError, match=named):
        resolve(dict(TINY_A, **extra))


def test_every_refusal_in_one_error_and_bookkeeping_keys_pass():
    with pytest.raises(ConfigError) as e:
        resolve(dict(TINY_A, rope_scaling={"type": "linear", "factor": 2.0}, partial_rotary_factor=0.25,
                     sliding_window_pattern=4))
    msg = str(e.value)
    assert "rope_scaling" in msg and "partial_rotary_factor" in msg and "sliding_window_pattern" in msg
    # what a published checkpoint's config.json carries beside the architecture's keys
    cfg, _ = resolve(dict(TINY_A, model_type="qwen2_moe", torch_dtype="bfloat16", transformers_version="4.40.0",
                          use_cache=True, initializer_range=0.02, attention_dropout=0.0, output_router_logits=False,
                          router_aux_loss_coef=0.001, rope_scaling=None, partial_rotary_factor=1.0,
                          attention_bias=True, bos_token_id=1, eos_token_id=2))
    assert cfg.eos_token_id == 2 and cfg.qkv_bias


def test_a_head_size_no_prompt_kernel_takes_in_bfloat16_still_builds():
    """head_dim 40 (no multiple of 16) is a legal configuration: the mixer is built, and its prompt path is the
    general kernel (checked on the GPU in the replay tests)."""
    cfg, spec = resolve(dict(TINY_C, head_dim=40))
    assert spec.layers[0].mixer.head_dim == 40
    with pytest.raises(ConfigError, match="head_dim"):
        resolve(dict(TINY_C, head_dim=41))
