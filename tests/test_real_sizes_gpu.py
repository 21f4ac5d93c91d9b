"""The engine at the layer sizes of the real checkpoints (a small vocabulary, random
weights), against the plain implementation: the kernels meet hidden 2048 / 3584,
16 x 128 heads and 28:4 grouped heads, 60 experts of width 1408, a shared expert of
width 5632, which the tiny configurations never reach; and the schedules that the
benchmark times: decode batches of 8, 33 and 64 through the replayed graphs, prompts
of more than 2,048 tokens, a window of 2,048 that is crossed.

The reference checks the same equalities on its own decoder: a batch of tokens
equals token by token, N sequences together equal each alone
(crates/ferrox-models/src/decoder.rs:4168-4203, 4266-4351), and a real checkpoint's
continuation (crates/ferrox-models/tests/qwen2moe_paris.rs:16-103).

Weights are drawn on the device by the random-weights rule and handed to the plain
implementation as copies (``replay_util.drawn_model``): no folder of gigabytes."""
import os
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
    choice (one layer: a position's logits hang on its own router only), and such positions must be few: at most a
    tenth of a request's (two of a short one) and a twentieth of all the run's.  No position is left out."""
    all_tipped = all_positions = 0
    for rid in want:
        diff = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max()
        tipped = 0
        for t in (diff >= tol).nonzero().flatten().tolist() if bf16 else []:
            diff[t] = want.close_to_a_choice(rid, t, got[rid][t])
            tipped += 1
        assert tipped <= max(2, len(diff) // 10), (rid, tipped)
        assert float(diff.max()) < tol, (rid, int(diff.argmax()), float(diff.max()))
        all_tipped += tipped
        all_positions += len(diff)
    assert all_tipped <= max(2, all_positions // 20), (all_tipped, all_positions)


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


# ------------------------------------------------------------------ the schedules the benchmark times
DECODE_BATCHES = (8, 33, 64)


@pytest.fixture(scope="module", params=["a2.7b", "a14b"])
def many_requests(request):
    """64 requests of 20 to 130 tokens at one layer of the real widths, their plain logits computed once."""
    cfg = dict(A27B_LAYER if request.param == "a2.7b" else A14B_LAYER, vocab_size=1201)
    rng = random.Random(8)
    prompts = {f"d{i:02d}": [rng.randrange(cfg["vocab_size"]) for _ in range(rng.randint(20, 130))] for i in range(64)}
    return cfg, prompts, ru.Expected(ru.drawn_model(cfg, seed=12), prompts, one_layer=True)


@pytest.mark.parametrize("dtype,tol", [("float32", 3e-5), ("bfloat16", 3e-2)])
@pytest.mark.parametrize("batch", DECODE_BATCHES)
def test_decode_batches_through_the_graphs(many_requests, batch, dtype, tol):
    """8, 33 and 64 requests of different lengths decoding together for 10 steps (the first runs eagerly, the second
    is captured, the rest replay the graph): from 8 tokens on the step uses other kernels than the smaller batches
    of the tests above (experts by the swapped-role tcgen05 kernel, the head by it too, K cut over CTAs from 17 and 33
    tokens, the in-kernel merge of key ranges only while all blocks run at once).  Every logit against plain."""
    from ferrox_b200 import Engine

    cfg, prompts, want = many_requests
    some = dict(list(prompts.items())[:batch])
    eng = Engine.from_random(cfg, seed=12, norm_init="around_one", dtype=dtype, on_device=True, page_size=64,
                             n_pages=3 * batch, max_slots=batch)
    got = ru.run_decode_together(eng, some, tail=10)
    assert eng.graphs is not None and batch in eng.graphs.graphs     # the steps did go through a captured graph
    check(got, _Subset(want, some), tol, dtype == "bfloat16")
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())


class _Subset:
    """Some requests of an Expected (what `check` reads of it)."""

    def __init__(self, want, rids):
        self._want, self._rids = want, list(rids)

    def __iter__(self):
        return iter(self._rids)

    def __getitem__(self, rid):
        return self._want[rid]

    def close_to_a_choice(self, *a, **k):
        return self._want.close_to_a_choice(*a, **k)


@pytest.mark.parametrize("shape", ["a2.7b", "a14b"])
def test_prompt_beyond_2048_tokens_whole_in_portions_and_with_a_decoded_tail(shape):
    """One prompt of 2,400 tokens at the real widths against plain, in 32-bit and in bfloat16: whole (the dense
    products on pairs of SMs, a tenth 256-query tile, 160 rows an expert and so a second 128-row tile for most
    experts, routing in two kernels), as 2,048 tokens and the rest (the second portion reads a cached prefix), and
    with its last 12 tokens decoded one by one (split-key attention over 38 blocks of keys)."""
    from ferrox_b200 import Engine

    cfg = dict(A27B_LAYER if shape == "a2.7b" else A14B_LAYER, vocab_size=1201, max_position_embeddings=2560)
    rng = random.Random(21)
    prompts = {"long": [rng.randrange(cfg["vocab_size"]) for _ in range(2400)]}
    want = ru.Expected(ru.drawn_model(cfg, seed=3), prompts, one_layer=True)
    for dtype, tol in (("float32", 3e-5), ("bfloat16", 3e-2)):
        eng = Engine.from_random(cfg, seed=3, norm_init="around_one", dtype=dtype, on_device=True, page_size=64,
                                 n_pages=40, max_slots=2)
        bf = dtype == "bfloat16"
        check(ru.run_whole(eng, prompts), want, tol, bf)
        check(ru.run_portions(eng, prompts, sizes=(2048, 352)), want, tol, bf)
        check(ru.run_tail_decode(eng, prompts, tail=12), want, tol, bf)
        assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())


def test_four_layers_a_window_of_2048_crossed_served_mixed_fp32():
    """The widths of Qwen1.5-MoE-A2.7B in true 32-bit: four layers, the last two with a sliding window of 2,048, five
    prompts of which one has 2,300 tokens (its window is crossed by 252 positions, so the windowed group gives pages
    back while the request runs), served as portions of up to 600 tokens beside decoded tokens of the others, two
    requests live at a time, with fewer pages than the prompts need together so that pages are used again.  Every
    logit against the plain implementation."""
    from ferrox_b200 import Engine

    W = 2048
    cfg = dict(A27B_LAYER, num_hidden_layers=4, use_sliding_window=True, sliding_window=W, max_window_layers=2,
               vocab_size=1500, max_position_embeddings=2560)
    rng = random.Random(14)
    lens = [2300, 64, 700, 300, 1]
    prompts = {f"w{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lens)}
    want = ru.Expected(ru.drawn_model(cfg, seed=2), prompts)
    # pages of 64: the longest request holds 36 in the full group and at most (2048 + 600) / 64 + 1 in the windowed one;
    # beside it one other request of at most 700 tokens (11 pages)
    pools = {None: 36 + 11, W: 43 + 11}
    assert sum(-(-n // 64) for n in lens) > pools[None]
    eng = Engine.from_random(cfg, seed=2, norm_init="around_one", dtype="float32", on_device=True, page_size=64,
                             n_pages=pools, max_slots=2)
    got = ru.run_mixed(eng, prompts, seed=9, max_live=2, max_portion=300)
    check(got, want, 3e-5, False)
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())
    assert eng.cache.peak_pages[None] >= 36
    # the windowed group lets go of what the window has passed: the book-keeping of a request of 2,300 positions
    slot = eng.open_request()
    for n in (600, 1200, 1800, 2300):
        assert eng.cache.reserve(slot, n)
        eng.cache.commit(slot, n)
    held = eng.cache.held_pages(slot)
    assert len(held[None]) == 36 and len(held[W]) == 36 - (2300 - W + 1) // 64
    eng.close_request(slot)


def test_6000_tokens_cut_three_ways():
    """6,000 tokens at the real layer sizes in bfloat16 against plain: whole (pairs of SMs, 24 tiles of 256 queries,
    400 rows an expert), in four portions, and with its last tokens decoded one by one (split-key attention over 94
    blocks of keys).  The keys far back count: another first half gives other logits."""
    from ferrox_b200 import Engine, StepEntry

    cfg = dict(A27B_LAYER, max_position_embeddings=8192, vocab_size=1000)
    rng = random.Random(3)
    toks = [rng.randrange(cfg["vocab_size"]) for _ in range(6000)]
    tail = 6
    cfg_w = ru.drawn_model(cfg, seed=7)
    want = ru.Expected(cfg_w, {"p": toks}, one_layer=True)
    eng = Engine.from_random(cfg, seed=7, norm_init="around_one", dtype="bfloat16", on_device=True, page_size=64,
                             n_pages=96, max_slots=2)

    def last_logits(cuts):
        slot = eng.open_request()
        outs, at = [], 0
        for n in cuts:
            rows = [i - at for i in range(max(at, len(toks) - tail), at + n)]
            lg = eng.step([StepEntry(slot, toks[at:at + n], want=rows)])
            if rows:
                outs.append(lg.float().cpu())
            at += n
        eng.close_request(slot)
        assert at == len(toks)
        return torch.cat(outs)

    scale = float(want["p"].abs().max())
    for cuts in ([6000], [2048, 1000, 2500, 452], [6000 - tail] + [1] * tail):
        got = last_logits(cuts)
        assert got.shape == (tail, cfg["vocab_size"])
        for i in range(tail):
            t = 6000 - tail + i
            err = float((got[i] - want["p"][t]).abs().max()) / scale
            if err >= 3e-2:    # a close choice between experts tipped by rounding: right under that other choice
                err = want.close_to_a_choice("p", t, got[i])
            assert err < 3e-2, (cuts[:2], t, err)
    # and the far keys matter: the same tail after a different first half gives other logits
    other = [rng.randrange(cfg["vocab_size"]) for _ in range(3000)] + toks[3000:]
    slot = eng.open_request()
    lg = eng.step([StepEntry(slot, other, want=list(range(6000 - tail, 6000)))]).float().cpu()
    eng.close_request(slot)
    assert float((want["p"][6000 - tail:] - lg).abs().max()) / scale > 1e-2


@pytest.mark.skipif(os.environ.get("FERROX_FULL_SIZE") != "1",
                    reason="the full-size check takes minutes and 60 GB: set FERROX_FULL_SIZE=1")
def test_full_size_fp32_window_2048_sixteen_prompts_served_mixed():
    """All 24 layers at the widths of Qwen1.5-MoE-A2.7B in true 32-bit (57 GB of weights), a sliding window of 2,048
    from layer 12 on, context 8,192: 16 prompts of 64 to 3,000 tokens served as portions beside decoded tokens, four
    live at a time, against the plain implementation at every position.  The vocabulary is cut to 8,192 rows to keep
    the logits of 24,000 positions in memory; every other size is the checkpoint's."""
    from ferrox_b200 import Engine

    W = 2048
    cfg = dict(A27B_LAYER, num_hidden_layers=24, use_sliding_window=True, sliding_window=W, max_window_layers=12,
               vocab_size=8192, max_position_embeddings=8192)
    rng = random.Random(40)
    lens = [64, 3000, 2111] + [rng.randint(64, 3000) for _ in range(13)]
    prompts = {f"f{i:02d}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(lens)}
    want = ru.Expected(ru.drawn_model(cfg, seed=1), prompts)
    eng = Engine.from_random(cfg, seed=1, norm_init="around_one", dtype="float32", on_device=True, page_size=64,
                             n_pages={None: 4 * 47 + 4, W: 4 * 43 + 4}, max_slots=4)
    got = ru.run_mixed(eng, prompts, seed=17, max_live=4, max_portion=300)
    # Every position is compared.  Among 26,000 positions x 24 routers a few separate the fourth expert from the
    # fifth by less than 32-bit sums taken in another order differ (the logits of long requests differ by 2e-5 at
    # the end of 24 layers): there either choice is right, and the logits of that one position differ by parts in a
    # thousand.  A position beyond the tolerance is excused only if plain's own router gap there is under 1e-4 of the
    # token's largest router logit, and at most one position in a thousand may need the excuse.
    tol, floor, tipped, total, worst, wrong = 1e-4, 1e-4, 0, 0, 0.0, []
    for rid in prompts:
        diff = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max()
        total += diff.numel()
        for t in (diff >= tol).nonzero().flatten().tolist():
            if float(want.margins[rid][t]) < floor:
                tipped += 1
                diff[t] = 0.0
            else:
                wrong.append((rid, t, f"{float(diff[t]):.2e}", f"margin {float(want.margins[rid][t]):.2e}"))
        worst = max(worst, float(diff.max()))
    assert not wrong, (len(wrong), wrong[:40])
    assert tipped <= total // 1000, (tipped, total)
    left_out = tipped
    print(f"full size: {total} positions, {left_out} excused for an undecided router, worst relative error {worst:.2e}")
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())
