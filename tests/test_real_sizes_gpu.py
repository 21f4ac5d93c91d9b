"""The engine at the layer sizes of the real checkpoints (one layer, a small
vocabulary, random weights), against the plain implementation: the kernels meet
hidden 2048 / 3584, 16 x 128 heads and 28:4 grouped heads, 60 experts of width 1408,
a shared expert of width 5632, which the tiny configurations never reach."""
import random

import pytest
import torch

import plain_qwen2moe as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

# one layer with the sizes of Qwen1.5-MoE-A2.7B
A27B_LAYER = dict(
    architectures=["Qwen2MoeForCausalLM"], num_hidden_layers=1, hidden_size=2048, num_attention_heads=16,
    num_key_value_heads=16, head_dim=128, num_experts=60, num_experts_per_tok=4, moe_intermediate_size=1408,
    shared_expert_intermediate_size=5632, intermediate_size=5632, decoder_sparse_step=1, mlp_only_layers=[],
    norm_topk_prob=False, qkv_bias=True, vocab_size=3001, rope_theta=1000000.0, rms_norm_eps=1e-6,
    use_sliding_window=False, tie_word_embeddings=False, max_position_embeddings=512,
)
# one layer with the attention and expert widths of Qwen2-57B-A14B (fewer experts, narrower shared expert)
A14B_LAYER = dict(
    architectures=["Qwen2MoeForCausalLM"], num_hidden_layers=1, hidden_size=3584, num_attention_heads=28,
    num_key_value_heads=4, head_dim=128, num_experts=10, num_experts_per_tok=8, moe_intermediate_size=2560,
    shared_expert_intermediate_size=2560, intermediate_size=2560, decoder_sparse_step=1, mlp_only_layers=[],
    norm_topk_prob=False, qkv_bias=True, vocab_size=2000, rope_theta=1000000.0, rms_norm_eps=1e-6,
    use_sliding_window=True, sliding_window=48, max_window_layers=0, tie_word_embeddings=True,
    max_position_embeddings=512,
)


@pytest.fixture(scope="module", params=["a2.7b", "a14b"])
def model(request, tmp_path_factory):
    from ferrox_b200 import write_random_model

    cfg = A27B_LAYER if request.param == "a2.7b" else A14B_LAYER
    folder = write_random_model(str(tmp_path_factory.mktemp("real") / request.param), cfg, seed=5, std=0.02,
                                norm_init="around_one")
    rng = random.Random(1)
    prompts = {"p": [rng.randrange(cfg["vocab_size"]) for _ in range(150)],
               "q": [rng.randrange(cfg["vocab_size"]) for _ in range(70)]}
    return folder, prompts, ru.Expected(folder, prompts)


def check(got, want, tol, bf16):
    for rid in want:
        diff = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max()
        if bf16:
            diff = torch.where(want.margins[rid] < 2.0 ** -7, torch.zeros_like(diff), diff)
        assert float(diff.max()) < tol, (rid, int(diff.argmax()), float(diff.max()))


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 3e-2)])
def test_real_layer_sizes_under_three_cuts(model, dtype, tol):
    from ferrox_b200 import Engine

    folder, prompts, want = model
    eng = Engine.from_folder(folder, dtype=dtype, page_size=64, n_pages=8, max_slots=3)
    first = ru.run_whole(eng, prompts)
    check(first, want, tol, dtype == "bfloat16")
    for _ in range(3):   # the same steps again give the same bits (fixed order of sums, no race between kernels)
        again = ru.run_whole(eng, prompts)
        assert all(torch.equal(first[r], again[r]) for r in prompts)
    check(ru.run_tail_decode(eng, prompts, tail=24), want, tol, dtype == "bfloat16")
    check(ru.run_mixed(eng, prompts, seed=2, max_live=2, max_portion=40), want, tol, dtype == "bfloat16")
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())
