"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

Each call of :meth:`Scheduler.schedule` decides one step:

1. every running request that decodes brings its one token (decodes come first);
2. running requests still in their prompt bring a portion, in order of admission,
   while the step's token budget lasts;
3. waiting requests are admitted first come first served while a slot is free,
   budget is left and the pages for their first portion are free.

When pages run out: a prompt portion is shortened to what fits, or waits; if even
the decodes do not fit, the most recently admitted running request is preempted:
its pages and slot are given back and it returns to the head of the waiting queue
with prompt + generated tokens as its new prompt, to be recomputed.  A request
whose prompt plus ``max_new_tokens`` could never fit the pool, or the context, is
refused at admission, so one request alone can always run to its end and the
scheduler cannot stall.

Reference: the continuous batcher admits while slots are free, runs whole prompts
at admission and then one token per live slot and step
(crates/ferrox-server/src/batch_scheduler.rs:158-243, admit :271-298, finish
:195-211,235-237,317-335); pool exhaustion is an error at admission, never in
mid-decode (generate.rs:44-80,329-331); fixed-size prompt chunks generate.rs:169-186.
EOS ends a request without being appended (batch_scheduler.rs:201-205).
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

from ..sampling.sampler import SamplingParams, XorShift64
from .batch import StepEntry


def encode_prompt(p, vocab_size: int) -> List[int]:
    """Token ids as given; text is encoded byte by byte (the reference's fallback
    tokenizer, crates/ferrox-models/src/tokenizer.rs:40-56)."""
    if isinstance(p, str):
        if vocab_size < 256:
            raise ValueError("byte-level prompts need a vocabulary of at least 256")
        return list(p.encode("utf-8"))
    ids = [int(t) for t in p]
    for t in ids:
        if not 0 <= t < vocab_size:
            raise ValueError(f"prompt token {t} outside vocab_size {vocab_size}")
    return ids


class AdmissionError(ValueError):
    pass


@dataclass
class Request:
    rid: int
    prompt: List[int]
    max_new: int
    params: SamplingParams
    eos_ids: Sequence[int]
    generated: List[int] = field(default_factory=list)
    slot: Optional[int] = None
    fed: int = 0  # tokens whose keys and values are in the cache
    finish_reason: Optional[str] = None
    rng: XorShift64 = None
    admitted_at: int = -1
    n_preempted: int = 0

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.generated

    @property
    def pending(self) -> int:
        return len(self.prompt) + len(self.generated) - self.fed


@dataclass
class Counters:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    decode_steps: int = 0  # steps in which every entry was a single decoded token
    decode_step_tokens: int = 0
    decode_seconds: float = 0.0  # host wall time of those steps, sampling and read-back included
    decode_h2d_bytes: int = 0
    decode_d2h_bytes: int = 0
    ahead_steps: int = 0  # decode steps issued before the host had read the step before them


class Scheduler:
    def __init__(self, engine, max_batch_tokens: int = 2048, sampler=None):
        self.engine = engine
        self.cache = engine.cache
        self.max_batch_tokens = int(max_batch_tokens)
        if self.max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be at least 1")
        if sampler is None:
            from ..sampling.sampler import Sampler

            sampler = Sampler(engine.rt.device)
        self.sampler = sampler
        self.waiting: deque = deque()
        self.running: List[Request] = []
        self.requests: Dict[int, Request] = {}
        self.counters = Counters()
        self._next_id = 0
        self._clock = 0

    # ---- admission --------------------------------------------------------------
    def add_request(self, prompt: Sequence[int], max_new_tokens: int, params: SamplingParams = None,
                    eos_ids: Sequence[int] = ()) -> int:
        prompt = list(prompt)
        if not prompt:
            raise AdmissionError("empty prompt")
        ctx = self.cache.max_positions
        if len(prompt) >= ctx:
            raise AdmissionError(f"prompt length {len(prompt)} >= context size {ctx}")
        max_new = ctx - len(prompt) if max_new_tokens < 0 else min(int(max_new_tokens), ctx - len(prompt))
        # the last generated token is never fed back, so prompt + max_new - 1 positions are held at most
        worst = len(prompt) + max(0, max_new - 1)
        need = (worst + self.cache.page_size - 1) // self.cache.page_size
        for key, g in self.cache.groups.items():
            # a windowed group holds at most the window plus the pages of one portion
            floor = need if key is None else min(need, (key + self.cache.page_size - 1) // self.cache.page_size + 2)
            if floor > g.pool.n_pages:
                raise AdmissionError(
                    f"request of up to {worst} positions needs {floor} pages, the pool has {g.pool.n_pages}")
        params = params or SamplingParams()
        r = Request(self._next_id, prompt, max_new, params, tuple(eos_ids), rng=XorShift64(params.seed))
        self._next_id += 1
        self.requests[r.rid] = r
        if max_new == 0:
            r.finish_reason = "length"
            self.counters.finished += 1
        else:
            self.waiting.append(r)
        return r.rid

    def result(self, rid: int) -> List[int]:
        return list(self.requests[rid].generated)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- one step -----------------------------------------------------------------
    def schedule(self) -> List[tuple]:
        """Decide the next step: a list of (request, number of tokens).  Admits and
        preempts as a side effect; maps no pages (the step function does)."""
        preempted = False
        while True:
            plan = self._plan(admit=not preempted)
            if plan is None or (not plan and self.running):
                # a decode does not fit, or nothing at all does: the youngest gives way
                if len(self.running) <= 1:
                    raise RuntimeError("scheduler: a request alone does not fit the page pool")
                self._preempt(max(self.running, key=lambda q: q.admitted_at))
                preempted = True
                continue
            return plan

    def _plan(self, admit: bool) -> Optional[List[tuple]]:
        """None: a decoding request lacks a page."""
        budget = self.max_batch_tokens
        free = dict(self.cache.free_pages())
        plan: List[tuple] = []

        def fits(r: Request, n: int) -> bool:
            need = self.cache.pages_needed(r.slot, r.fed + n)
            return all(free[k] >= v for k, v in need.items())

        def take(r: Request, n: int) -> None:
            for k, v in self.cache.pages_needed(r.slot, r.fed + n).items():
                free[k] -= v
            plan.append((r, n))

        by_age = sorted(self.running, key=lambda q: q.admitted_at)
        # 1. decodes, oldest first
        for r in by_age:
            if r.pending != 1 or budget < 1:
                continue
            if not fits(r, 1):
                return None
            take(r, 1)
            budget -= 1
        # 2. prompts in progress, in order of admission
        for r in by_age:
            if r.pending <= 1 or budget < 1:
                continue
            n = self._largest_fitting(r, min(r.pending, budget), fits)
            if n >= 1:
                take(r, n)
                budget -= n
        # 3. admissions, first come first served
        while admit and self.waiting and budget >= 1 and self.cache.n_free_slots > 0:
            r = self.waiting[0]
            slot = self.cache.open_request()
            r.slot, r.fed = slot, 0
            n = self._largest_fitting(r, min(r.pending, budget), fits)
            if n < 1:
                self.cache.close_request(slot)
                r.slot = None
                break
            self.waiting.popleft()
            self._clock += 1
            r.admitted_at = self._clock
            self.running.append(r)
            take(r, n)
            budget -= n
        return plan

    def _largest_fitting(self, r: Request, n: int, fits) -> int:
        """The most tokens <= n of ``r`` whose pages are free (whole pages at a time)."""
        if n < 1 or fits(r, n):
            return max(n, 0)
        ps = self.cache.page_size
        # shrink to page boundaries: positions up to the end of an already mapped page cost nothing
        while n > 0:
            end = ((r.fed + n - 1) // ps) * ps  # last position of the previous page + 1
            n = end - r.fed
            if n >= 1 and fits(r, n):
                return n
        return 0

    def _preempt(self, r: Request) -> None:
        self.cache.close_request(r.slot)
        self.running.remove(r)
        r.slot, r.fed = None, 0
        r.n_preempted += 1
        self.counters.preemptions += 1
        self.waiting.appendleft(r)

    def step(self) -> List[Request]:
        """Run one step; returns the requests that finished in it."""
        plan = self.schedule()
        if not plan:
            if self.idle:
                return []
            raise RuntimeError("scheduler stalled: work is left but nothing fits (pool too small for one request)")
        entries, sampled_from = [], []
        t0 = time.perf_counter()
        all_decode = all(n == 1 and r.generated and r.pending == 1 for r, n in plan)
        for r, n in plan:
            toks = r.tokens[r.fed:r.fed + n]
            last = r.fed + n == len(r.prompt) + len(r.generated)
            entries.append(StepEntry(r.slot, toks, want=[n - 1] if last else []))
            if last:
                sampled_from.append(r)
            if n == 1 and r.generated and last:
                self.counters.decode_tokens += 1
            else:
                self.counters.prefill_tokens += n
        logits = self.engine.step(entries)
        for r, n in plan:
            r.fed += n
        self.counters.steps += 1
        finished = []
        if sampled_from:
            ids = self.sampler.sample(logits, [r.params for r in sampled_from], [r.rng for r in sampled_from],
                                      [r.generated for r in sampled_from])
            for r, tok in zip(sampled_from, ids):
                self._take_token(r, int(tok))
                if r.finish_reason:
                    finished.append(r)
        self._retire(finished)
        if all_decode:
            from . import step as _stepmod

            c = self.counters
            c.decode_steps += 1
            c.decode_step_tokens += len(plan)
            c.decode_seconds += time.perf_counter() - t0
            c.decode_h2d_bytes += _stepmod.last_h2d_bytes
            c.decode_d2h_bytes += 4 * len(sampled_from)
        return finished

    def run(self) -> None:
        while not self.idle:
            if not self._decode_ahead():
                self.step()

    # ---- decoding issued ahead of the host ----------------------------------------------
    def _decode_ahead(self) -> bool:
        """While nothing waits, every running request is decoding (greedily, or sampling without a repetition
        penalty) and a CUDA graph of this batch size exists, steps are issued one ahead: the host reads a step's tokens while the next step runs.  Only
        lengths decide how many steps may be issued (no request reaches its limit inside the run); an end-of-
        sequence token shows one step late, the step issued meanwhile for that request is thrown away.  Pages
        that run out end the run before the step that lacks them: the ordinary step then decides.
        Returns False when it did nothing."""
        issue = getattr(self.engine, "decode_ahead", None)
        if issue is None or self.waiting or not self.running or len(self.running) > self.max_batch_tokens:
            return False
        reqs = sorted(self.running, key=lambda q: q.admitted_at)
        for r in reqs:
            if r.pending != 1 or not r.generated or r.params.repetition_penalty != 1.0:
                return False
        ctx = self.cache.max_positions
        n_safe = min(min(r.max_new - len(r.generated), ctx - len(r.prompt) - len(r.generated)) for r in reqs)
        if n_safe < 2:
            return False
        if all(r.params.greedy for r in reqs):
            run = issue([r.slot for r in reqs], [r.generated[-1] for r in reqs])
        else:
            # (a generator's draws go with the steps as they are issued: a step issued for a request that then turns
            # out to have ended costs that request a draw it no longer needs)
            run = issue([r.slot for r in reqs], [r.generated[-1] for r in reqs], [(r.params, r.rng) for r in reqs])
        if run is None:
            return False
        from .step import OutOfPages

        t0 = time.perf_counter()
        stop = False
        h2d = 0
        while run.issued < n_safe and not stop:
            try:
                run.issue()
            except OutOfPages:
                break
            from . import step as _stepmod

            h2d += _stepmod.last_h2d_bytes
            for r in reqs:
                r.fed += 1
            if run.issued - run.collected == 2:
                stop = self._absorb(reqs, run.collect())
        if run.issued == 0:
            return False
        while run.collected < run.issued:
            self._absorb(reqs, run.collect())
        run.close()
        c = self.counters
        c.steps += run.issued
        c.decode_steps += run.issued
        c.ahead_steps += run.issued
        c.decode_seconds += time.perf_counter() - t0
        c.decode_h2d_bytes += h2d
        c.decode_d2h_bytes += 4 * len(reqs) * run.issued
        self._retire([r for r in reqs if r.finish_reason])
        return True

    def _absorb(self, reqs, tokens) -> bool:
        """Takes one step's chosen tokens; True when a request ended with them."""
        ended = False
        for r, tok in zip(reqs, tokens):
            if r.finish_reason:
                continue   # ended a step ago: this token came from the step issued meanwhile
            self.counters.decode_tokens += 1
            self.counters.decode_step_tokens += 1
            self._take_token(r, int(tok))
            ended = ended or bool(r.finish_reason)
        return ended

    def _take_token(self, r: Request, tok: int) -> None:
        if tok in r.eos_ids:
            r.finish_reason = "stop"
        else:
            r.generated.append(tok)
            if len(r.generated) >= r.max_new:
                r.finish_reason = "length"
            elif len(r.prompt) + len(r.generated) >= self.cache.max_positions:
                r.finish_reason = "context"

    def _retire(self, finished) -> None:
        for r in finished:
            self.cache.close_request(r.slot)
            self.running.remove(r)
            r.slot = None
            self.counters.finished += 1
