"""Generation through the public entry point, sampling, and the command line."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen2moe as plain
from tiny_configs import CONFIGS, make_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    tmp = tmp_path_factory.mktemp("gen")
    # std 0.2: logits far enough apart that greedy choices survive 32-bit rounding
    return {name: make_folder(tmp, name, std=0.2) for name in CONFIGS}


def engine(folder, dtype="float32", **kw):
    from ferrox_b200 import Engine

    kw.setdefault("page_size", 16)
    kw.setdefault("n_pages", 32)
    kw.setdefault("max_slots", 4)
    return Engine.from_folder(folder, dtype=dtype, **kw)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_greedy_generation_matches_plain(folders, name):
    cfg, w = plain.load_model(folders[name])
    prompts = [[5, 9, 200, 31], [7], list(range(40, 75))]
    want = [plain.greedy(cfg, w, p, 12) for p in prompts]
    eng = engine(folders[name])
    assert eng.generate(prompts, max_new_tokens=12) == want
    assert eng.generate(prompts[0], max_new_tokens=12) == want[0]  # a single prompt
    # small budget: prompts cut into portions, decodes beside them
    assert eng.generate(prompts, max_new_tokens=12, max_batch_tokens=5) == want
    eng.cache.check_invariants()
    assert eng.cache.n_free_slots == 4


def test_generation_with_preemption_gives_the_same_tokens(folders):
    cfg, w = plain.load_model(folders["A"])
    prompts = [[i + 1, i + 3, i + 7, 99, 4, 8, 15, 16] for i in range(4)]
    want = [plain.greedy(cfg, w, p, 20) for p in prompts]
    eng = engine(folders["A"], page_size=4, n_pages=14, max_slots=4)  # 4 x 27 positions do not fit 56
    outs, stats = eng.generate(prompts, max_new_tokens=20, return_stats=True)
    assert stats["preemptions"] >= 1
    assert outs == want


def test_decoding_issued_ahead_gives_the_same_tokens(folders):
    """Greedy decode steps run one ahead of the host once a graph of the batch size exists: same tokens; an
    end-of-sequence token that shows one step late ends its request at the right place; limits that differ."""
    cfg, w = plain.load_model(folders["A"])
    prompts = [[5, 9, 200, 31], [7, 8], list(range(40, 60))]
    free = [plain.greedy(cfg, w, p, 24) for p in prompts]
    eng = engine(folders["A"])
    outs, stats = eng.generate(prompts, max_new_tokens=24, return_stats=True)
    assert outs == free and stats["ahead_steps"] >= 10
    eos = free[1][15]
    want = [f[:f.index(eos)] if eos in f else f for f in free]
    outs, stats = eng.generate(prompts, max_new_tokens=24, eos_token_id=eos, return_stats=True)
    assert outs == want and stats["ahead_steps"] >= 5
    eng.cache.check_invariants()
    assert eng.cache.n_free_slots == 4
    # few pages: the run ends where a page is missing and the ordinary step preempts
    small = engine(folders["A"], page_size=4, n_pages=16, max_slots=4)
    outs, stats = small.generate(prompts, max_new_tokens=24, return_stats=True)
    assert outs == free and stats["preemptions"] >= 1
    small.cache.check_invariants()
    # bfloat16 through the same path: as many tokens as asked for
    outs, stats = engine(folders["A"], "bfloat16").generate(prompts, max_new_tokens=24, return_stats=True)
    assert [len(o) for o in outs] == [24, 24, 24] and stats["ahead_steps"] >= 10
    for p, o in zip(prompts, outs):
        assert_greedy_within_rounding(cfg, w, p, o)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sampled_decoding_issued_ahead_gives_the_same_tokens(folders, dtype):
    """Temperature, top-k and top-p sampling chosen inside the replayed graph, one step ahead of the host: the same
    tokens as the engine without graphs draws with the same seeds (the same kernels give the same logits bit for
    bit; each request's uniform draws come from its own generator in both)."""
    prompts = [[5, 9, 200, 31], [7, 8], list(range(40, 60))]
    for kw in (dict(temperature=0.9), dict(temperature=1.3, top_k=7), dict(temperature=0.8, top_p=0.6),
               dict(temperature=1.0, top_k=12, top_p=0.9)):
        plain_eng = engine(folders["B"], dtype, cuda_graphs=False)
        want, st0 = plain_eng.generate(prompts, max_new_tokens=30, seed=11, return_stats=True, **kw)
        assert st0["ahead_steps"] == 0
        eng = engine(folders["B"], dtype)
        got, st = eng.generate(prompts, max_new_tokens=30, seed=11, return_stats=True, **kw)
        assert got == want and st["ahead_steps"] >= 10, kw
        again = eng.generate(prompts, max_new_tokens=30, seed=11, **kw)        # the sampling graph a second time
        other = eng.generate(prompts, max_new_tokens=30, seed=12, **kw)
        assert again == want and other != want
        eng.cache.check_invariants()
    # an end-of-sequence token that shows one step late; a repetition penalty keeps the ordinary path
    eng = engine(folders["B"], dtype)
    free = eng.generate(prompts, max_new_tokens=30, seed=3, temperature=1.1, top_k=20)
    eos = free[2][12]
    want = [f[:f.index(eos)] if eos in f else f for f in free]
    assert eng.generate(prompts, max_new_tokens=30, seed=3, temperature=1.1, top_k=20, eos_token_id=eos) == want
    outs, st = eng.generate(prompts, max_new_tokens=12, seed=3, temperature=1.1, repetition_penalty=1.2, return_stats=True)
    assert st["ahead_steps"] == 0 and [len(o) for o in outs] == [12, 12, 12]


def test_long_decoding_stays_on_the_plain_implementation(folders):
    """One token at a time up to the context's end (pages and, for B, the window roll over many times)."""
    for name in ("A", "B"):
        cfg, w = plain.load_model(folders[name])
        n = cfg["max_position_embeddings"] - 4
        got = engine(folders[name], page_size=4, n_pages=64).generate([[1, 2, 3]], max_new_tokens=n)[0]
        seq = [1, 2, 3] + got
        logits = plain.forward(cfg, w, seq[:-1])
        # every generated token is the plain implementation's choice given the same history
        want = logits[2:].argmax(dim=-1).tolist()
        assert got == want


BF16_LOGIT_TOL = 3e-2   # the replay tests' bound on a bfloat16 logit's error, relative to the request's largest |logit|


def assert_greedy_within_rounding(cfg, w, prompt, generated, tol=BF16_LOGIT_TOL):
    """Every generated token must be the plain implementation's choice given the same history, or a token whose
    plain logit is within twice the bfloat16 logit tolerance of the best one (an engine whose logits are off by at
    most the tolerance can prefer no other token).  The history is the engine's own, so every token is checked, not
    only those before the first legitimate difference.  As in the replay tests, a position where plain itself
    separates the experts at the router's cut by less than a few bfloat16 roundings is not comparable (the engine
    may rightly take the other expert); at least half of the tokens must be comparable."""
    seq = list(prompt) + list(generated)
    logits, margins = plain.forward(cfg, w, seq[:-1], return_margins=True)
    scale = float(logits.abs().max())
    undecided = 0
    for i, tok in enumerate(generated):
        at = len(prompt) - 1 + i
        if float(margins[at]) < 2.0 ** -7:
            undecided += 1
            continue
        row = logits[at]
        gap = float(row.max() - row[tok])
        assert gap <= 2 * tol * scale, (i, tok, int(row.argmax()), gap / scale, float(margins[at]))
    assert undecided <= len(generated) // 2, undecided    # (a generated sequence that repeats a token repeats its margin)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_bfloat16_generation_stays_within_rounding_of_plain(tmp_path, name):
    # (weights of the usual spread, for which the replay tests establish the bfloat16 logit tolerance; with the ten
    # times larger weights of this file's other tests a deep model amplifies roundings beyond it)
    folder = make_folder(tmp_path, name)
    cfg, w = plain.load_model(folder)
    prompts = [[5, 9, 200, 31], [7], list(range(40, 75))]
    eng = engine(folder, "bfloat16")
    outs = eng.generate(prompts, max_new_tokens=12)
    assert [len(o) for o in outs] == [12, 12, 12]
    for p, o in zip(prompts, outs):
        assert_greedy_within_rounding(cfg, w, p, o)
    # and the check can fail: a sequence with one token swapped for an unlikely one does not pass it
    for at in range(12):
        bad = list(outs[0])
        logits, margins = plain.forward(cfg, w, prompts[0] + bad[:at], return_margins=True)
        if float(margins[-1]) < 2.0 ** -7:
            continue
        bad[at] = int(logits[-1].argmin())
        with pytest.raises(AssertionError):
            assert_greedy_within_rounding(cfg, w, prompts[0], bad)
        break
    else:
        raise AssertionError("no comparable position among 12")


def test_eos_and_string_prompts(folders):
    eng = engine(folders["A"])
    free = eng.generate([[5, 9, 200, 31]], max_new_tokens=10)[0]
    eos = free[4]
    stopped = eng.generate([[5, 9, 200, 31]], max_new_tokens=10, eos_token_id=eos)[0]
    assert stopped == free[:free.index(eos)]
    assert eng.generate([[5, 9, 200, 31]], max_new_tokens=10, eos_token_id=eos, ignore_eos=True)[0] == free
    assert eng.generate(["hi"], max_new_tokens=3) == eng.generate([[104, 105]], max_new_tokens=3)
    with pytest.raises(ValueError, match="vocab"):
        eng.generate([[5, 999]], max_new_tokens=1)


def plain_sample(row, p, rng, h, detail=False):
    """One row by the reference's procedure, crates/ferrox-models/src/sampling.rs:93-189, in plain torch.
    ``detail``: the cumulative sums in 64 bits, returned with the token and the draw."""
    V = row.numel()
    s = row.clone()
    if p.repetition_penalty != 1.0:
        for t in h:
            s[t] = s[t] / p.repetition_penalty if s[t] > 0 else s[t] * p.repetition_penalty
    if p.temperature <= 0:
        return int(torch.argmax(s))
    pr = torch.softmax(s / p.temperature, dim=0)
    if 0 < p.top_k < V:
        kth = torch.topk(pr, p.top_k).values[-1]
        pr = torch.where(pr >= kth, pr, torch.zeros_like(pr))
    if p.top_p < 1.0:
        order = torch.argsort(pr, descending=True)
        c = torch.cumsum(pr[order], 0)
        cut = int((c >= p.top_p).nonzero()[0]) + 1 if bool((c >= p.top_p).any()) else V
        keep = torch.zeros(V, dtype=torch.bool)
        keep[order[:cut]] = True
        pr = torch.where(keep, pr, torch.zeros_like(pr))
    pr = pr / pr.sum()
    draw = rng.next_f32()
    c = torch.cumsum(pr.double() if detail else pr, 0)
    idx = (draw < c).nonzero()
    tok = int(idx[0]) if len(idx) else int((pr > 0).nonzero()[-1])
    return (tok, c, draw) if detail else tok



def test_sampling_follows_the_reference_procedure(folders):
    """Device sampling against a plain restatement of sampling.rs:93-189."""
    from ferrox_b200.sampling.sampler import Sampler, SamplingParams, XorShift64

    torch.manual_seed(0)
    V = 331
    logits = (torch.randn(6, V) * 3).cuda()
    hist = [[], [1, 2, 2, 5], [7], [], [3, 3, 3], [9]]
    params = [
        SamplingParams(temperature=0.0),
        SamplingParams(temperature=0.0, repetition_penalty=1.5),
        SamplingParams(temperature=0.7, seed=11),
        SamplingParams(temperature=1.3, top_k=5, seed=12),
        SamplingParams(temperature=0.9, top_p=0.6, repetition_penalty=1.2, seed=13),
        SamplingParams(temperature=1.0, top_k=40, top_p=0.95, seed=14),
    ]

    sampler = Sampler("cuda:0")
    rngs_a = [XorShift64(p.seed) for p in params]
    rngs_b = [XorShift64(p.seed) for p in params]
    cpu = logits.cpu()
    for _ in range(20):
        got = sampler.sample(logits, params, rngs_a, hist)
        want = [plain_sample(cpu[i], params[i], rngs_b[i], hist[i]) for i in range(6)]
        assert got == want
    # temperature -> 0+ and top_k = 1 both reduce to greedy (sampling.rs:241-380)
    g = sampler.sample(logits, [SamplingParams()] * 6, rngs_a, hist)
    k1 = sampler.sample(logits, [SamplingParams(temperature=1.0, top_k=1, seed=3)] * 6, [XorShift64(3) for _ in range(6)], hist)
    p0 = sampler.sample(logits, [SamplingParams(temperature=1.0, top_p=1e-6, seed=3)] * 6, [XorShift64(3) for _ in range(6)], hist)
    assert g == k1 == p0 == cpu.argmax(dim=1).tolist()


@pytest.mark.parametrize("V", [151936, 151936 - 371, 4099])
def test_sampling_at_the_real_vocabulary(V):
    """The sampling kernels at the vocabulary the served model has (their chunking and the radix selection of the
    top-k threshold depend on it) and at sizes that are no multiple of anything: neither filter, top-k 40,
    top-p 0.95 and both, 20 draws each, against the plain restatement; then the form that runs inside the decode
    graph (fx_sample_or: scores untouched, a fallback where a request is greedy) against the plain form."""
    from ferrox_b200.kernels import ops
    from ferrox_b200.sampling.sampler import Sampler, SamplingParams, XorShift64

    g = torch.Generator().manual_seed(V)
    logits = (torch.randn(4, V, generator=g) * 2.5).cuda()
    params = [
        SamplingParams(temperature=0.8, seed=21),
        SamplingParams(temperature=0.8, top_k=40, seed=22),
        SamplingParams(temperature=0.8, top_p=0.95, seed=23),
        SamplingParams(temperature=0.8, top_k=40, top_p=0.95, seed=24),
    ]
    hist = [[] for _ in params]
    sampler = Sampler("cuda:0")
    rngs_a = [XorShift64(p.seed) for p in params]
    rngs_b = [XorShift64(p.seed) for p in params]
    rngs_c = [XorShift64(p.seed) for p in params]
    cpu = logits.cpu()
    dev = dict(device="cuda:0")
    temp = torch.tensor([p.temperature for p in params], **dev)
    top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32, **dev)
    top_p = torch.tensor([p.top_p for p in params], **dev)
    use = torch.tensor([1, 1, 0, 1], dtype=torch.int32, **dev)          # request 2 is "greedy" in the graph form
    best = ops.argmax(logits, torch.empty(4, dtype=torch.int32, **dev))
    seen, exact = set(), 0
    for _ in range(20):
        got = sampler.sample(logits, params, rngs_a, hist)
        for i in range(4):
            want, c, draw = plain_sample(cpu[i], params[i], rngs_b[i], hist[i], detail=True)
            exact += got[i] == want
            # Over 150,000 probabilities of some 1e-5 each, 32-bit running sums differ from exact ones by about
            # 1e-6: a draw that lands that close to a border between two tokens may rightly give the neighbour.  The
            # token must have mass and its interval of the exact cumulative sums must hold the draw within 1e-5.
            lo = float(c[got[i] - 1]) if got[i] > 0 else 0.0
            assert float(c[got[i]]) > lo and lo - 1e-5 <= draw < float(c[got[i]]) + 1e-5, (i, got[i], want, draw)
        seen.update(got)
        draw = torch.tensor([r.next_f32() for r in rngs_c], **dev)
        before = logits.clone()
        out = torch.empty(4, dtype=torch.int32, **dev)
        ops.sample_or(logits, torch.empty_like(logits), temp, top_k, top_p, draw, use, best, out)
        assert torch.equal(logits, before)
        assert out.tolist() == [got[0], got[1], int(best[2]), got[3]]
    assert len(seen) > 20      # draws, not one token over and over
    assert exact >= 72         # and nearly always the very token of the plain procedure


def test_sampled_generation_is_seeded_and_batch_independent(folders):
    eng = engine(folders["A"])
    a = eng.generate([[5, 9, 200, 31]], max_new_tokens=16, temperature=0.9, top_k=20, seed=5)[0]
    b = eng.generate([[5, 9, 200, 31]], max_new_tokens=16, temperature=0.9, top_k=20, seed=5)[0]
    c = eng.generate([[5, 9, 200, 31]], max_new_tokens=16, temperature=0.9, top_k=20, seed=6)[0]
    both = eng.generate([[5, 9, 200, 31], [8, 8, 8]], max_new_tokens=16, temperature=0.9, top_k=20, seed=5)
    assert a == b and a != c and both[0] == a


def test_command_line(folders, tmp_path):
    env = dict(os.environ, PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ferrox"), "-m", folders["A"], "--tokens", "5,9,200,31",
                        "-n", "6", "--temp", "0", "--dtype", "float32", "--repeat-penalty", "1.0"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr
    cfg, w = plain.load_model(folders["A"])
    assert [int(t) for t in r.stdout.split()] == plain.greedy(cfg, w, [5, 9, 200, 31], 6)
    assert "ferrox: prompt 4 tokens" in r.stderr and "predict 6 tokens" in r.stderr
    r = subprocess.run([sys.executable, "-m", "ferrox_b200", "run", "-m", folders["A"], "-p", "ab", "-n", "3", "--temp", "0.8",
                        "-s", "1", "--print-ids"], capture_output=True, text=True, env=env, timeout=600, cwd=ROOT)
    assert r.returncode == 0 and len(r.stdout.split()) == 3, r.stderr


def test_trace_run_tool(folders, tmp_path):
    cfg, w = plain.load_model(folders["B"])
    toks = {"a": [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5], "b": [2, 7, 1, 8, 2, 8]}
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": toks["a"][:5], "want": [4]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": toks["a"][5:7], "want": []},
                                {"id": "b", "tokens": toks["b"], "want": [0, 5]}], "end": ["b"]},
        {"step": 2, "entries": [{"id": "a", "tokens": toks["a"][7:], "want": [0, 3]}], "end": ["a"]},
    ]
    out = tmp_path / "out"
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["B"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", "128"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    assert r.stdout.split("\n")[:3] == ["done 0", "done 1", "done 2"]
    import numpy as np

    la, lb = plain.forward(cfg, w, toks["a"]), plain.forward(cfg, w, toks["b"])
    V = cfg["vocab_size"]
    s0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, V)
    s1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, V)
    s2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, V)
    assert s0.shape[0] == 1 and s1.shape[0] == 2 and s2.shape[0] == 2
    for got, want in ((s0[0], la[4]), (s1[0], lb[0]), (s1[1], lb[5]), (s2[0], la[7]), (s2[1], la[10])):
        assert float(np.abs(got - want.numpy()).max()) < 2e-5 * float(want.abs().max())


def test_trace_run_from_a_configuration_and_a_seed(folders, tmp_path):
    """--random CONFIG --seed S runs the model a folder written by the random-weights mode holds: the same logits, bit
    for bit, as --model on that folder."""
    from tiny_configs import TINY_B
    import numpy as np

    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(TINY_B))
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [3, 1, 4, 1, 5, 9, 2, 6], "want": [0, 7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [5, 3], "want": [1]}], "end": ["a"]}]
    outs = []
    # (the fixture's folder of B: seed 1, norm weights around one, but std 0.2)
    for i, src in enumerate((["--model", folders["B"]],
                             ["--random", str(cfg_path), "--seed", "1", "--std", "0.2", "--norm-init", "around_one"])):
        out = tmp_path / f"out{i}"
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), *src, "--dtype", "bfloat16", "--out", str(out),
                            "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stderr
        outs.append([np.fromfile(out / f"{k}.f32", dtype="<f4") for k in (0, 1)])
    assert all(np.array_equal(a, b) for a, b in zip(*outs)) and outs[0][0].size == 2 * TINY_B["vocab_size"]


def test_kernel_trace_behind_its_switch(folders):
    """With the switch on, device time is summed per part and entry point and generation gives the same tokens
    (without graphs); with it off nothing is recorded."""
    from ferrox_b200 import Engine
    from ferrox_b200.kernels import ops

    prompt = [5, 9, 200, 31]
    want = engine(folders["A"]).generate([prompt], max_new_tokens=6)[0]
    assert not ops.trace_enabled()
    Engine.trace_start()
    try:
        eng = engine(folders["A"])
        assert eng.graphs is None
        got = eng.generate([prompt], max_new_tokens=6)[0]
    finally:
        times = Engine.trace_stop()
    assert got == want and not ops.trace_enabled()
    assert any(k.startswith("mixer:fx_decode_attention") for k in times) and "head:fx_rmsnorm" in times
    assert all(n > 0 and ms > 0.0 for n, ms in times.values())
    assert engine(folders["A"]).graphs is not None
