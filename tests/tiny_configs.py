"""Two tiny Qwen2-MoE configurations that differ in every size and option, and the
helpers that make model folders for them (in temporary folders, never committed)."""
from __future__ import annotations

ARCH = "Qwen2MoeForCausalLM"

# A: every layer has experts; 2:1 grouped heads; no window; untied head.
TINY_A = dict(
    architectures=[ARCH], num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
    head_dim=16, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=32,
    shared_expert_intermediate_size=64, intermediate_size=96, decoder_sparse_step=1, mlp_only_layers=[],
    norm_topk_prob=False, qkv_bias=True, vocab_size=256, rope_theta=10000.0, rms_norm_eps=1e-6,
    use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=128,
)

# B: dense, MoE, dense layers; one kv head; window 16 from layer 1 on; tied head;
# renormalised top-3 of 8; sizes that are no power of two.
TINY_B = dict(
    architectures=[ARCH], num_hidden_layers=3, hidden_size=128, num_attention_heads=2, num_key_value_heads=1,
    head_dim=64, num_experts=8, num_experts_per_tok=3, moe_intermediate_size=48,
    shared_expert_intermediate_size=96, intermediate_size=160, decoder_sparse_step=2, mlp_only_layers=[0],
    norm_topk_prob=True, qkv_bias=True, vocab_size=384, rope_theta=1000000.0, rms_norm_eps=1e-5,
    use_sliding_window=True, sliding_window=16, max_window_layers=1, tie_word_embeddings=True,
    max_position_embeddings=256,
)

# C: odd sizes everywhere: 3 kv heads of 6 heads, head_dim 48 (hidden != heads*head_dim),
# hidden 80, vocab 331, 5 experts top-1, no shared expert, no qkv bias, window 7.
TINY_C = dict(
    architectures=[ARCH], num_hidden_layers=4, hidden_size=80, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, num_experts=5, num_experts_per_tok=1, moe_intermediate_size=24,
    shared_expert_intermediate_size=0, intermediate_size=56, decoder_sparse_step=1, mlp_only_layers=[2],
    norm_topk_prob=True, qkv_bias=False, vocab_size=331, rope_theta=50000.0, rms_norm_eps=3e-6,
    use_sliding_window=True, sliding_window=7, max_window_layers=2, tie_word_embeddings=False,
    max_position_embeddings=192,
)

CONFIGS = {"A": (TINY_A, 0, "ones"), "B": (TINY_B, 1, "around_one"), "C": (TINY_C, 2, "around_one")}


def make_folder(tmp_path, name, dtype="bfloat16", std=0.02):
    from ferrox_b200 import write_random_model

    cfg, seed, norm_init = CONFIGS[name]
    folder = str(tmp_path / f"tiny_{name}_{dtype}")
    write_random_model(folder, cfg, seed, dtype=dtype, std=std, norm_init=norm_init)
    return folder
