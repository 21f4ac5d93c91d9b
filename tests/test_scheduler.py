"""The scheduler's decisions, with the real cache manager on the CPU and a stand-in
for the model: the 'model' answers with logits that make the next token a function
of the request's whole history, so any mix-up of requests, positions or
recomputation after a preemption changes the output."""
import random

import pytest
import torch

from ferrox_b200.cache.manager import CacheManager
from ferrox_b200.cache.specs import CacheSpec, KvCacheSpec
from ferrox_b200.engine.scheduler import AdmissionError, Scheduler
from ferrox_b200.sampling.sampler import SamplingParams

VOCAB = 50


def next_token(history):
    h = 7
    for t in history:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


class FakeEngine:
    """Keeps each slot's token history as the cache would keep keys and values."""

    def __init__(self, n_pages=8, page_size=4, max_slots=3, max_positions=64, window=None):
        specs = [CacheSpec(kv=KvCacheSpec(1, 2, None)), CacheSpec(kv=KvCacheSpec(1, 2, window))]
        self.cache = CacheManager(specs, page_size=page_size, n_pages=n_pages, max_slots=max_slots,
                                  max_positions=max_positions, device="cpu", dtype=torch.float32)
        self.history = {}
        self.steps = []

    def step(self, entries):
        rows = []
        self.steps.append([(e.slot, len(e.tokens), len(e.want)) for e in entries])
        wanted = {}
        for e in entries:
            for key, n in self.cache.pages_needed(e.slot, self.cache.seq_len[e.slot] + len(e.tokens)).items():
                wanted[key] = wanted.get(key, 0) + n
        assert self.cache.can_reserve(wanted), "the scheduler planned a step that does not fit"
        for e in entries:
            start = self.cache.seq_len[e.slot]
            if start == 0:
                self.history[e.slot] = []
            assert len(self.history[e.slot]) == start
            assert self.cache.reserve(e.slot, start + len(e.tokens))
            for i, t in enumerate(e.tokens):
                self.history[e.slot].append(t)
                if i in e.want:
                    row = torch.zeros(VOCAB)
                    row[next_token(self.history[e.slot])] = 1.0
                    rows.append(row)
            self.cache.commit(e.slot, start + len(e.tokens))
        self.cache.check_invariants()
        return torch.stack(rows) if rows else torch.zeros(0, VOCAB)


class ArgmaxSampler:
    def sample(self, logits, params, rngs, histories):
        return [int(torch.argmax(r)) for r in logits]


def alone(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        out.append(next_token(seq))
        seq.append(out[-1])
    return out


def make(engine, budget=16):
    return Scheduler(engine, max_batch_tokens=budget, sampler=ArgmaxSampler())


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    eng = FakeEngine(n_pages=16, page_size=4, max_slots=3)
    s = make(eng, budget=8)
    a = s.add_request(list(range(1, 6)), 4)  # 5 tokens
    b = s.add_request(list(range(10, 30)), 3)  # 20 tokens
    s.step()
    assert eng.steps[-1] == [(0, 5, 1), (1, 3, 0)]  # a whole, b's first portion fills the budget
    s.step()
    assert eng.steps[-1] == [(0, 1, 1), (1, 7, 0)]  # a decodes first, b gets the rest of the budget
    s.run()
    assert s.result(a) == alone(range(1, 6), 4) and s.result(b) == alone(range(10, 30), 3)
    assert s.counters.finished == 2 and eng.cache.free_pages()[None] == 16


def test_matches_one_request_at_a_time(seed=0):
    rng = random.Random(seed)
    prompts = [[rng.randrange(VOCAB) for _ in range(rng.randint(1, 30))] for _ in range(12)]
    news = [rng.randint(1, 12) for _ in prompts]
    eng = FakeEngine(n_pages=24, page_size=4, max_slots=4)
    s = make(eng, budget=11)
    ids = [s.add_request(p, n) for p, n in zip(prompts, news)]
    s.run()
    for i, p, n in zip(ids, prompts, news):
        assert s.result(i) == alone(p, n)
    assert max(len(st) for st in eng.steps) <= 4
    assert all(sum(n for _, n, _ in st) <= 11 for st in eng.steps)


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 4: two requests of 8-token prompts that each grow to 20 cannot both stay
    eng = FakeEngine(n_pages=6, page_size=4, max_slots=2)
    s = make(eng, budget=32)
    a = s.add_request(list(range(8)), 12)
    b = s.add_request(list(range(20, 28)), 12)
    s.run()
    assert s.counters.preemptions >= 1
    assert s.requests[b].n_preempted >= 1 and s.requests[a].n_preempted == 0  # the older one is never the victim
    assert s.result(a) == alone(range(8), 12) and s.result(b) == alone(range(20, 28), 12)
    assert eng.cache.free_pages()[None] == 6


def test_admission_refuses_what_can_never_fit():
    eng = FakeEngine(n_pages=4, page_size=4, max_slots=2, max_positions=64)
    s = make(eng)
    with pytest.raises(AdmissionError, match="pages"):
        s.add_request(list(range(10)), 10)  # 19 positions > 16
    s.add_request(list(range(10)), 7)  # 16 positions fit exactly
    with pytest.raises(AdmissionError, match="context"):
        s.add_request(list(range(64)), 1)
    with pytest.raises(AdmissionError, match="empty"):
        s.add_request([], 1)
    s.run()


def test_eos_stops_without_being_appended_and_length_limits():
    eng = FakeEngine(n_pages=16)
    s = make(eng)
    want = alone([1, 2, 3], 6)
    eos = want[3]
    a = s.add_request([1, 2, 3], 6, eos_ids=(eos,))
    b = s.add_request([1, 2, 3], 6)
    c = s.add_request([1, 2, 3], -1)  # fill the context
    s.run()
    first = want.index(eos)
    assert s.result(a) == want[:first] and s.requests[a].finish_reason == "stop"
    assert s.result(b) == want and s.requests[b].finish_reason == "length"
    assert len(s.result(c)) == 64 - 3


def test_waiting_requests_enter_when_slots_free_up():
    eng = FakeEngine(n_pages=32, max_slots=2)
    s = make(eng)
    ids = [s.add_request([i + 1, i + 2], 3) for i in range(5)]
    s.step()
    assert len(s.running) == 2 and len(s.waiting) == 3
    s.run()
    assert [s.result(i) for i in ids] == [alone([i + 1, i + 2], 3) for i in range(5)]


@pytest.mark.parametrize("seed", range(6))
def test_random_load_with_window_group_and_tight_pool(seed):
    rng = random.Random(seed)
    eng = FakeEngine(n_pages=rng.choice([10, 13, 16]), page_size=rng.choice([2, 4]), max_slots=rng.choice([2, 3, 4]),
                     max_positions=40, window=rng.choice([3, 9]))
    s = make(eng, budget=rng.choice([3, 7, 20]))
    reqs = []
    for _ in range(15):
        p = [rng.randrange(VOCAB) for _ in range(rng.randint(1, 12))]
        n = rng.randint(1, 8)
        reqs.append((s.add_request(p, n), p, n))
    s.run()
    for i, p, n in reqs:
        assert s.result(i) == alone(p, n)
    assert all(v == eng.cache.groups[k].pool.n_pages for k, v in eng.cache.free_pages().items())
    assert eng.cache.n_free_slots == eng.cache.max_slots
