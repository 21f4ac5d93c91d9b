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
        specs = [CacheSpec(paged=KvCacheSpec(1, 2, None)), CacheSpec(paged=KvCacheSpec(1, 2, window))]
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


# ---- decoding issued one step ahead of the host ---------------------------------------------------
class FakeAheadRun:
    """What DecodeAhead does on the GPU, on the CPU: a step is 'issued' (pages mapped, lengths advanced,
    the token chosen by the 'device' kept there) and its tokens are handed out later, oldest first."""

    def __init__(self, eng, slots, tokens):
        self.eng, self.slots = eng, list(slots)
        self.device_tokens = list(tokens)
        self.queue = []
        self.issued = self.collected = 0

    def issue(self):
        from ferrox_b200.engine.step import OutOfPages

        cache = self.eng.cache
        wanted = {}
        for s in self.slots:
            for key, n in cache.pages_needed(s, cache.seq_len[s] + 1).items():
                wanted[key] = wanted.get(key, 0) + n
        if not cache.can_reserve(wanted):
            raise OutOfPages("no page")
        chosen = []
        for s, t in zip(self.slots, self.device_tokens):
            start = cache.seq_len[s]
            assert len(self.eng.history[s]) == start
            assert cache.reserve(s, start + 1)
            self.eng.history[s].append(t)
            chosen.append(next_token(self.eng.history[s]))
            cache.commit(s, start + 1)
        cache.check_invariants()
        self.device_tokens = chosen
        self.queue.append(chosen)
        self.issued += 1
        assert self.issued - self.collected <= 2, "more than one step ahead of the host"

    def collect(self):
        self.collected += 1
        return self.queue.pop(0)

    def close(self):
        assert not self.queue


class FakeAheadEngine(FakeEngine):
    def __init__(self, *a, ready_after=2, **kw):
        super().__init__(*a, **kw)
        self.sizes_seen = {}
        self.ready_after = ready_after
        self.ahead_runs = 0

    def step(self, entries):
        if all(len(e.tokens) == 1 for e in entries):
            self.sizes_seen[len(entries)] = self.sizes_seen.get(len(entries), 0) + 1
        return super().step(entries)

    def decode_ahead(self, slots, tokens, sampling=None):
        if self.sizes_seen.get(len(slots), 0) < self.ready_after:   # "no graph of this size yet"
            return None
        self.ahead_runs += 1
        self.sampling_seen = sampling
        return FakeAheadRun(self, slots, tokens)


def make_greedy(engine, budget=16):
    # the real sampler's plain path is an arg max too; the requests' parameters must say "greedy"
    return Scheduler(engine, max_batch_tokens=budget, sampler=ArgmaxSampler())


def test_steps_issued_ahead_give_the_same_tokens_and_respect_limits():
    eng = FakeAheadEngine(n_pages=32, page_size=4, max_slots=3)
    s = make_greedy(eng)
    prompts = [[3, 1, 4], [1, 5, 9, 2, 6], [5, 3]]
    limits = [20, 9, 14]
    ids = [s.add_request(p, n) for p, n in zip(prompts, limits)]
    s.run()
    assert [s.result(i) for i in ids] == [alone(p, n) for p, n in zip(prompts, limits)]
    assert eng.ahead_runs >= 2 and s.counters.ahead_steps >= 8
    assert s.cache.n_free_slots == 3
    eng.cache.check_invariants()


def test_end_of_sequence_shows_one_step_late_and_the_extra_step_is_dropped():
    prompts = [[3, 1, 4], [1, 5, 9, 2, 6]]
    free = [alone(p, 16) for p in prompts]
    eos = free[0][9]
    want = [f[:f.index(eos)] if eos in f else f for f in free]
    eng = FakeAheadEngine(n_pages=32, page_size=4, max_slots=2)
    s = make_greedy(eng)
    ids = [s.add_request(p, 16, eos_ids=(eos,)) for p in prompts]
    s.run()
    assert [s.result(i) for i in ids] == want
    assert s.requests[ids[0]].finish_reason == "stop"
    assert eng.ahead_runs >= 1 and s.cache.n_free_slots == 2
    eng.cache.check_invariants()


def test_pages_run_out_inside_a_run_issued_ahead():
    prompts = [[1, 2, 3], [4, 5, 6], [7, 8, 9]]
    want = [alone(p, 14) for p in prompts]
    eng = FakeAheadEngine(n_pages=9, page_size=4, max_slots=3)   # 3 x 16 positions do not fit 36
    s = make_greedy(eng)
    ids = [s.add_request(p, 14) for p in prompts]
    s.run()
    assert [s.result(i) for i in ids] == want
    assert s.counters.preemptions >= 1 and eng.ahead_runs >= 1
    eng.cache.check_invariants()


def test_requests_with_a_repetition_penalty_are_never_issued_ahead():
    eng = FakeAheadEngine(n_pages=32, page_size=4, max_slots=2, ready_after=0)
    s = make_greedy(eng)
    s.add_request([1, 2, 3], 8, SamplingParams(temperature=0.7, seed=1, repetition_penalty=1.3))
    s.add_request([4, 5], 8)
    s.run()
    assert eng.ahead_runs == 0


def test_sampled_requests_are_issued_ahead_with_their_own_generators():
    """Sampling without a repetition penalty needs nothing from the host but a uniform draw a step, which does not
    depend on the tokens: such requests decode ahead too, and the run gets each request's parameters and generator."""
    eng = FakeAheadEngine(n_pages=32, page_size=4, max_slots=2, ready_after=0)
    s = make_greedy(eng)
    a = s.add_request([1, 2, 3], 8, SamplingParams(temperature=0.7, top_k=5, seed=1))
    b = s.add_request([4, 5], 8)
    s.run()
    assert eng.ahead_runs >= 1
    (pa, ga), (pb, gb) = eng.sampling_seen
    assert pa.temperature == 0.7 and pa.top_k == 5 and pb.greedy
    assert ga is not gb and ga.state != gb.state      # one generator per request, seeded by the request
    assert len(s.result(a)) == 8 and len(s.result(b)) == 8
    eng.cache.check_invariants()