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
    prompts = {rid: [rng.randrange(cfg["vocab_size"]) for _ in range(n)]
               for rid, n in (("p", 150), ("q", 70), ("r", 200), ("s", 9))}
    return folder, prompts, ru.Expected(folder, prompts, one_layer=True)


def check(got, want, tol, bf16):
    """Every position within the tolerance of the plain logits.  In bfloat16 rounded router logits may tip a close
    choice between experts: such a position must then be within the tolerance of the plain logits under that other
    choice (one layer: a position's logits hang on its own router only), and such positions must be few.  No
    position is left out."""
    for rid in want:
        diff = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max()
        tipped = 0
        for t in (diff >= tol).nonzero().flatten().tolist() if bf16 else []:
            diff[t] = want.close_to_a_choice(rid, t, got[rid][t])
            tipped += 1
        assert tipped <= max(2, len(diff) // 20), (rid, tipped)
        assert float(diff.max()) < tol, (rid, int(diff.argmax()), float(diff.max()))


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 3e-2)])
def test_real_layer_sizes_under_three_cuts(model, dtype, tol):
    from ferrox_b200 import Engine

    folder, prompts, want = model
    eng = Engine.from_folder(folder, dtype=dtype, page_size=64, n_pages=10, max_slots=4)
    first = ru.run_whole(eng, prompts)
    check(first, want, tol, dtype == "bfloat16")
    for _ in range(3):   # the same steps again give the same bits (fixed order of sums, no race between kernels)
        again = ru.run_whole(eng, prompts)
        assert all(torch.equal(first[r], again[r]) for r in prompts)
    check(ru.run_tail_decode(eng, prompts, tail=24), want, tol, dtype == "bfloat16")
    check(ru.run_mixed(eng, prompts, seed=2, max_live=2, max_portion=40), want, tol, dtype == "bfloat16")
    # requests of 150, 70, 200 and 9 tokens decoding together (replayed graphs; key ranges of unequal length, some empty)
    check(ru.run_decode_together(eng, prompts, tail=8), want, tol, dtype == "bfloat16")
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())


def test_two_layers_one_windowed_served_in_mixed_batches_fp32(tmp_path):
    """The widths of Qwen1.5-MoE-A2.7B in true 32-bit, two layers of which the second has a sliding window (two groups
    of pages with different needs), prompts of random lengths served as portions beside decoded tokens with pages
    used again: every logit against the plain implementation."""
    from ferrox_b200 import Engine, write_random_model

    cfg = dict(A27B_LAYER, num_hidden_layers=2, use_sliding_window=True, sliding_window=96, max_window_layers=1,
               vocab_size=1500)
    folder = write_random_model(str(tmp_path / "two"), cfg, seed=9, std=0.02, norm_init="around_one")
    rng = random.Random(4)
    lens = [64, 1, 300] + [rng.randint(2, 300) for _ in range(4)]
    prompts = {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lens)}
    want = ru.Expected(folder, prompts)
    eng = Engine.from_folder(folder, dtype="float32", page_size=64, n_pages=3 * 5, max_slots=3)
    check(ru.run_mixed(eng, prompts, seed=6, max_live=3, max_portion=50), want, 3e-5, False)
    check(ru.run_decode_together(eng, dict(list(prompts.items())[2:5]), tail=20),
          {rid: want[rid] for rid in list(prompts)[2:5]}, 3e-5, False)
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())


def test_long_prompt_cut_three_ways_agrees_with_itself():
    """6,000 tokens at the real layer sizes, too long for the plain implementation: the logits at the last positions
    must not depend on whether the prompt came whole (pairs of SMs, 256-query attention tiles, 128-row expert tiles),
    in portions, or with its last tokens decoded one by one (split-key attention over 47 blocks of keys, few rows an
    expert).  The keys far back must count: the comparison would fail if a block of keys were dropped."""
    from ferrox_b200 import Engine, StepEntry, write_random_model
    import tempfile

    cfg = dict(A27B_LAYER, max_position_embeddings=8192, vocab_size=1000)
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_random_model(tmp + "/m", cfg, seed=7, std=0.02, norm_init="around_one")
        eng = Engine.from_folder(folder, dtype="bfloat16", page_size=64, n_pages=96, max_slots=2)
    rng = random.Random(3)
    toks = [rng.randrange(cfg["vocab_size"]) for _ in range(6000)]
    tail = 6

    def last_logits(cuts):
        slot = eng.open_request()
        outs, at = [], 0
        for n in cuts:
            want = [i - at for i in range(max(at, len(toks) - tail), at + n)]
            lg = eng.step([StepEntry(slot, toks[at:at + n], want=want)])
            if want:
                outs.append(lg.float().cpu())
            at += n
        eng.close_request(slot)
        assert at == len(toks)
        return torch.cat(outs)

    whole = last_logits([6000])
    portions = last_logits([2048, 1000, 2500, 452])
    decoded = last_logits([6000 - tail] + [1] * tail)
    assert whole.shape == portions.shape == decoded.shape == (tail, cfg["vocab_size"])
    scale = float(whole.abs().max())
    assert float((whole - portions).abs().max()) / scale < 3e-2
    assert float((whole - decoded).abs().max()) / scale < 3e-2
    # and the far keys matter: the same tail after a different first half gives other logits
    other = [rng.randrange(cfg["vocab_size"]) for _ in range(3000)] + toks[3000:]
    slot = eng.open_request()
    lg = eng.step([StepEntry(slot, other, want=list(range(6000 - tail, 6000)))]).float().cpu()
    eng.close_request(slot)
    assert float((whole - lg).abs().max()) / scale > 1e-2
