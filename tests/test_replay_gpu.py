"""The engine against the plain implementation under every way of cutting the work:
whole prompts, a decoded tail, portions of changing size, mixed batches with pages
used again; in 32-bit and in bfloat16; on tiny configurations that differ in every
size and option."""
import random

import pytest
import torch

import replay_util as ru
from tiny_configs import CONFIGS, make_folder

pytestmark = pytest.mark.gpu

# Largest |difference| allowed, relative to the largest |logit| of the request.
# 32-bit: both sides round 32-bit sums in different orders.  bfloat16: activations
# between kernels are rounded to 8 bits of mantissa.
TOL = {"float32": 2e-5, "bfloat16": 3e-2}
# In bfloat16 a router choice is not comparable where the plain implementation itself
# separates the experts at the cut by less than a few roundings: the gap between the
# two logits is under 2^-7 of the token's largest |logit| (bfloat16 spaces values
# 2^-8 apart).  The engine may then take the other expert and the logits of that
# position differ by whole percents.  Such positions are left out of the bfloat16
# comparison (never of the 32-bit one); they must stay few.
BF16_ROUTER_MARGIN = 2.0 ** -7

def prompts_for(name, n=5, lo=1, hi=96, seed=0):
    cfg = CONFIGS[name][0]
    rng = random.Random(seed)
    hi = min(hi, cfg["max_position_embeddings"])
    lens = [lo, 2, hi] + [rng.randint(lo, hi) for _ in range(max(0, n - 3))]
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(L)] for i, L in enumerate(lens)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("models")
    return {name: make_folder(tmp, name) for name in CONFIGS}


@pytest.fixture(scope="module")
def expected(folders):
    return {name: ru.Expected(folders[name], prompts_for(name)) for name in CONFIGS}


def engine(folder, dtype, **kw):
    from ferrox_b200 import Engine

    return Engine.from_folder(folder, dtype=dtype, **kw)


def compare(got, want, tol, what):
    worst, left_out, total = 0.0, 0, 0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        assert torch.isfinite(got[rid]).all(), (what, rid)
        diff = (got[rid] - want[rid]).abs().max(dim=1).values / want[rid].abs().max()
        total += diff.numel()
        if "bfloat16" in what:
            undecided = want.margins[rid] < BF16_ROUTER_MARGIN
            left_out += int(undecided.sum())
            diff = torch.where(undecided, torch.zeros_like(diff), diff)
        if float(diff.max()) > tol:
            first = int((diff > tol).nonzero()[0])
            raise AssertionError(f"{what}: request {rid} (length {want[rid].shape[0]}): relative error "
                                 f"{float(diff.max()):.3e} > {tol}; first wrong position {first}")
        worst = max(worst, float(diff.max()))
    assert left_out <= 0.1 * total, f"{what}: {left_out} of {total} positions have undecided routing"
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts(folders, expected, name, dtype):
    eng = engine(folders[name], dtype, page_size=16, n_pages=16, max_slots=4)
    got = ru.run_whole(eng, prompts_for(name))
    compare(got, expected[name], TOL[dtype], f"whole/{name}/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_tail_decoded_one_by_one(folders, expected, name, dtype):
    eng = engine(folders[name], dtype, page_size=16, n_pages=16, max_slots=4)
    got = ru.run_tail_decode(eng, prompts_for(name), tail=32)
    compare(got, expected[name], TOL[dtype], f"tail/{name}/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size", [4, 16, 64])
def test_portions_of_changing_size(folders, expected, name, dtype, page_size):
    eng = engine(folders[name], dtype, page_size=page_size, n_pages=max(2, 128 // page_size), max_slots=4)
    got = ru.run_portions(eng, prompts_for(name))
    compare(got, expected[name], TOL[dtype], f"portions/{name}/{dtype}/ps{page_size}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
@pytest.mark.parametrize("page_size", [4, 16])
def test_mixed_batches_reuse_pages(folders, name, dtype, page_size):
    prompts = prompts_for(name, n=9, seed=3)
    want = ru.Expected(folders[name], prompts)
    # four live requests of at most 96 tokens: exactly enough pages, so that every
    # page a finished request gives back is taken again by a later one
    eng = engine(folders[name], dtype, page_size=page_size, n_pages=4 * (96 // page_size), max_slots=4)
    got = ru.run_mixed(eng, prompts, seed=5)
    compare(got, want, TOL[dtype], f"mixed/{name}/{dtype}/ps{page_size}")
    assert all(n == eng.cache.groups[k].pool.n_pages for k, n in eng.cache.free_pages().items())


@pytest.mark.parametrize("name", list(CONFIGS))
def test_cutting_changes_nothing_beyond_rounding_fp32(folders, name):
    """The same positions through different cuts agree far more tightly than either
    agrees with another implementation: the sums run in the same order."""
    prompts = prompts_for(name)
    a = ru.run_whole(engine(folders[name], "float32", page_size=16, n_pages=16, max_slots=4), prompts)
    b = ru.run_portions(engine(folders[name], "float32", page_size=4, n_pages=64, max_slots=4), prompts)
    c = ru.run_mixed(engine(folders[name], "float32", page_size=16, n_pages=24, max_slots=4), prompts, seed=1)
    for rid in prompts:
        assert ru.max_rel_err(b[rid], a[rid]) < 2e-6
        assert ru.max_rel_err(c[rid], a[rid]) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_token_decoded_one_by_one(folders, expected, dtype):
    """Long decoding: pages roll over, and on B the window leaves pages behind many times."""
    for name in ("A", "B"):
        eng = engine(folders[name], dtype, page_size=4, n_pages=32, max_slots=2)
        got = ru.run_tail_decode(eng, prompts_for(name), tail=10 ** 6)
        compare(got, expected[name], TOL[dtype], f"decode-all/{name}/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_tensors_stored_in_32_bits_stay_so(tmp_path, dtype):
    """A folder whose tensors are float32: the bfloat16 engine keeps them in 32 bits
    (products then run on the CUDA-core kernel with 32-bit weights)."""
    folder = make_folder(tmp_path, "B", dtype="float32")
    prompts = prompts_for("B", n=4)
    want = ru.Expected(folder, prompts)
    eng = engine(folder, dtype, page_size=16, n_pages=16, max_slots=4)
    if dtype == "bfloat16":
        assert eng.model.layers[1].ffn.w_gu.dtype == torch.float32 and eng.model.embedding.dtype == torch.float32
    compare(ru.run_portions(eng, prompts), want, TOL[dtype], f"stored32/B/{dtype}")


def test_dense_only_model_and_first_tokens(tmp_path):
    """No experts at all; and the very first positions of a sequence, one token at a time from position 0."""
    from ferrox_b200 import write_random_model
    from tiny_configs import TINY_A

    cfg = dict(TINY_A, num_experts=0, num_experts_per_tok=0, moe_intermediate_size=0, shared_expert_intermediate_size=0,
               intermediate_size=72, hidden_size=48, num_attention_heads=3, num_key_value_heads=3, head_dim=16)
    folder = write_random_model(str(tmp_path / "dense"), cfg, seed=9, norm_init="around_one")
    prompts = {"a": [7, 3, 250, 9, 11, 2, 5], "b": [1]}
    want = ru.Expected(folder, prompts)
    for dtype in ("float32", "bfloat16"):
        eng = engine(folder, dtype, page_size=4, n_pages=8, max_slots=2)
        assert all(type(l.ffn).__name__ == "SwigluMlp" for l in eng.model.layers)
        compare(ru.run_tail_decode(eng, prompts, tail=10 ** 6), want, TOL[dtype], f"dense/first-tokens/{dtype}")
        compare(ru.run_whole(eng, prompts), want, TOL[dtype], f"dense/whole/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_same_trace_twice_gives_the_same_bits(folders, dtype):
    """Every sum has a fixed order and no kernel reads what an earlier one has not finished writing:
    a replayed trace reproduces its logits exactly."""
    prompts = prompts_for("B", n=6, seed=11)
    runs = []
    for _ in range(3):
        eng = engine(folders["B"], dtype, page_size=16, n_pages=24, max_slots=4)
        runs.append(ru.run_mixed(eng, prompts, seed=4))
    for rid in prompts:
        assert torch.equal(runs[0][rid], runs[1][rid]) and torch.equal(runs[0][rid], runs[2][rid])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_logits_of_a_step_outlive_the_steps_after_it(folders, expected, dtype):
    """Small eager steps keep their buffers from one step to the next; what a step returns is not one of them: the
    logits of every step, kept on the device without a copy and read only at the end, are the plain ones."""
    from ferrox_b200 import StepEntry

    eng = engine(folders["A"], dtype, page_size=16, n_pages=12, max_slots=2)
    toks = prompts_for("A")["r2"]
    slot = eng.open_request()
    kept = []
    for i in range(0, len(toks), 3):                 # the same shapes step after step
        part = toks[i:i + 3]
        kept.append(eng.step([StepEntry(slot, part, want=list(range(len(part))))]))
    assert len({t.data_ptr() for t in kept}) == len(kept)
    got = {"r2": torch.cat([t.cpu() for t in kept])}
    compare(got, _Only(expected["A"], "r2"), TOL[dtype], f"kept-logits/A/{dtype}")
    eng.close_request(slot)
    eng.cache.check_invariants()


def test_a_fault_leaves_the_requests_where_they_were(folders, expected):
    """A step whose kernels raised the status word (here: set by hand, no kernel is made to fault) counts as not
    run: StepFault, the requests' lengths unchanged, the decode attention's merge counters zeroed again, and the
    same tokens fed once more give the plain logits."""
    from ferrox_b200 import StepEntry
    from ferrox_b200.engine import step as stepmod

    eng = engine(folders["A"], "bfloat16", page_size=64, n_pages=8, max_slots=2)
    toks = prompts_for("A")["r2"]
    slot = eng.open_request()
    first = eng.step([StepEntry(slot, toks[:40], want=list(range(40)))]).cpu()
    status = stepmod._status(eng.rt.device)
    counters = eng.model.layers[0].mixer._range_counters
    counters[:3] = 1          # what blocks that gave up half-way would leave behind
    status.fill_(3)
    with pytest.raises(stepmod.StepFault, match="bounded wait"):
        eng.step([StepEntry(slot, toks[40:42], want=[0, 1])])
    assert eng.cache.seq_len[slot] == 40 and int(status) == 0 and int(counters.abs().sum()) == 0
    rest = [eng.step([StepEntry(slot, toks[i:i + 1], want=[0])]).cpu().clone() for i in range(40, len(toks))]
    got = {"r2": torch.cat([first] + rest)}
    compare(got, _Only(expected["A"], "r2"), TOL["bfloat16"], "after-fault/A/bfloat16")
    eng.close_request(slot)
    eng.cache.check_invariants()


class _Only:
    def __init__(self, want, rid):
        self._want, self._rid, self.margins = want, rid, want.margins

    def __iter__(self):
        return iter([self._rid])

    def __getitem__(self, rid):
        return self._want[rid]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_head_size_that_is_no_multiple_of_16(tmp_path, dtype):
    """head_dim 40: in bfloat16 neither tensor-core attention kernel takes it; prompts go through the general kernel
    and decoding through the CUDA-core split-key kernel, against plain under mixed cuts."""
    from ferrox_b200 import write_random_model
    from tiny_configs import TINY_C

    cfg = dict(TINY_C, head_dim=40)
    folder = write_random_model(str(tmp_path / "c40"), cfg, seed=4, norm_init="around_one")
    rng = random.Random(2)
    prompts = {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate((70, 2, 33, 96, 17))}
    want = ru.Expected(folder, prompts)
    eng = engine(folder, dtype, page_size=16, n_pages=4 * 6, max_slots=4)
    compare(ru.run_mixed(eng, prompts, seed=8), want, TOL[dtype], f"mixed/head40/{dtype}")
    compare(ru.run_tail_decode(eng, prompts, tail=20), want, TOL[dtype], f"tail/head40/{dtype}")
