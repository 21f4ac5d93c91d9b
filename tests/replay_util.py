"""Helpers of the replay tests: drive the engine's step function with traces cut in
different ways and collect the logits of every position of every request."""
from __future__ import annotations

import random
from typing import Dict, List

import torch

import plain_qwen2moe as plain


def plain_logits(folder: str, prompts: Dict[str, List[int]], dtype=torch.float32) -> Dict[str, torch.Tensor]:
    cfg, w = plain.load_model(folder, dtype)
    return {rid: plain.forward(cfg, w, toks).to(torch.float32) for rid, toks in prompts.items()}


def drawn_model(cfg: dict, seed: int, std: float = 0.02, norm_init: str = "around_one", device="cuda:0"):
    """(cfg, tensors) for the plain implementation, without a folder: the values that the random-weights mode gives
    this configuration and seed (stored as bfloat16, as a folder written by it holds them), drawn on the device,
    where a model of the real widths takes a moment, and copied to the host in 32 bits.  The engine made by
    ``Engine.from_random(cfg, seed=..., on_device=True)`` with the same arguments holds the same values."""
    from ferrox_b200.config.registry import resolve
    from ferrox_b200.parts.build import build_model
    from ferrox_b200.weights.random_init import random_tensors

    decls = build_model(resolve(cfg)[1]).tensor_decls()
    w = {n: t.cpu().float() for n, t in random_tensors(decls, seed, torch.bfloat16, std, norm_init, device)}
    return cfg, w


class Expected:
    """Plain logits per request plus, per position, the router's smallest relative
    margin over the layers (see plain.router_margins)."""

    def __init__(self, model, prompts: Dict[str, List[int]], one_layer: bool = False):
        """``model``: a model folder, or (cfg, tensors) as :func:`drawn_model` gives them.
        ``one_layer``: keep what `close_to_a_choice` needs (a model of one layer only)."""
        self.cfg, self.w = plain.load_model(model, torch.float32) if isinstance(model, str) else model
        self.logits, self.margins, self.ffn_inputs = {}, {}, {}
        for rid, toks in prompts.items():
            if one_layer:
                lg, mg, self.ffn_inputs[rid] = plain.forward(self.cfg, self.w, toks, return_ffn_inputs=True)
            else:
                lg, mg = plain.forward(self.cfg, self.w, toks, return_margins=True)
            self.logits[rid], self.margins[rid] = lg, mg

    def close_to_a_choice(self, rid: str, t: int, got: torch.Tensor, rel: float = 0.05) -> float:
        """In a model of one layer the logits of a position hang on its own router's choice only.  The smallest
        distance (relative to the largest plain logit of the request) between ``got`` and the plain logits of
        position t under any choice of experts that differs from the plain one in one expert near the border
        (plain.close_choices): what an engine with rounded router logits may rightly have computed."""
        h, n = self.ffn_inputs[rid]
        router = n[t] @ self.w["model.layers.0.mlp.gate.weight"].T
        scale = float(self.logits[rid].abs().max())
        best = float("inf")
        for chosen in plain.close_choices(router, self.cfg["num_experts_per_tok"], rel):
            lg = plain.one_layer_position(self.cfg, self.w, h[t], n[t], chosen)
            best = min(best, float((got - lg).abs().max()) / scale)
        return best

    def __getitem__(self, rid):
        return self.logits[rid]

    def __iter__(self):
        return iter(self.logits)


class Collector:
    """Runs steps against an engine and stores logits by (request, position)."""

    def __init__(self, eng):
        from ferrox_b200 import StepEntry

        self.eng = eng
        self.StepEntry = StepEntry
        self.slots: Dict[str, int] = {}
        self.fed: Dict[str, int] = {}
        self.logits: Dict[str, Dict[int, torch.Tensor]] = {}

    def step(self, portions: Dict[str, List[int]], end=()):
        """``portions``: request id -> the tokens it brings; logits are wanted at every place."""
        entries, order = [], []
        for rid, toks in portions.items():
            if rid not in self.slots:
                slot = self.eng.open_request()
                assert slot is not None, "no free slot"
                self.slots[rid] = slot
                self.fed[rid] = 0
                self.logits[rid] = {}
            entries.append(self.StepEntry(self.slots[rid], list(toks), want=list(range(len(toks)))))
            order.append((rid, len(toks)))
        out = self.eng.step(entries).to("cpu")
        r = 0
        for rid, n in order:
            for i in range(n):
                self.logits[rid][self.fed[rid] + i] = out[r]
                r += 1
            self.fed[rid] += n
        for rid in end:
            self.eng.close_request(self.slots.pop(rid))
        self.eng.cache.check_invariants()

    def stacked(self, rid: str) -> torch.Tensor:
        d = self.logits[rid]
        return torch.stack([d[i] for i in range(len(d))])


def run_whole(eng, prompts):
    c = Collector(eng)
    for rid, toks in prompts.items():
        c.step({rid: toks}, end=[rid])
    return {rid: c.stacked(rid) for rid in prompts}


def run_tail_decode(eng, prompts, tail=32):
    """Most of each request in one step, the last ``tail`` tokens one by one."""
    c = Collector(eng)
    for rid, toks in prompts.items():
        head = max(1, len(toks) - tail)
        c.step({rid: toks[:head]})
        for i in range(head, len(toks)):
            c.step({rid: toks[i:i + 1]})
        eng.close_request(c.slots.pop(rid))
    return {rid: c.stacked(rid) for rid in prompts}


def run_decode_together(eng, prompts, tail=8):
    """Most of each request in a step of its own, then the last ``tail`` tokens of all requests one by one in
    common steps: a decode batch of requests of different lengths."""
    c = Collector(eng)
    rest = {}
    for rid, toks in prompts.items():
        head = max(1, len(toks) - tail)
        rest[rid] = list(toks[head:])
        c.step({rid: toks[:head]}, end=[] if rest[rid] else [rid])
    while any(rest.values()):
        portions = {rid: [r.pop(0)] for rid, r in rest.items() if r}
        c.step(portions, end=[rid for rid in portions if not rest[rid]])
    return {rid: c.stacked(rid) for rid in prompts}


def run_portions(eng, prompts, seed=0, sizes=(2, 3, 5, 2, 7, 11, 2, 16, 4, 33, 2)):
    """Portions of changing size, down to two tokens."""
    c = Collector(eng)
    for rid, toks in prompts.items():
        i, j = 0, 0
        while i < len(toks):
            n = min(sizes[j % len(sizes)], len(toks) - i)
            c.step({rid: toks[i:i + n]})
            i += n
            j += 1
        eng.close_request(c.slots.pop(rid))
    return {rid: c.stacked(rid) for rid in prompts}


def run_mixed(eng, prompts, seed=0, max_live=4, max_portion=9):
    """Up to ``max_live`` requests at a time; each step takes a random portion of
    some (prefill) beside single tokens of others (as decoding would); requests end
    and new ones take over their pages."""
    rng = random.Random(seed)
    c = Collector(eng)
    waiting = list(prompts.items())
    live: Dict[str, List[int]] = {}
    mode: Dict[str, str] = {}
    while waiting or live:
        while waiting and len(live) < max_live and (not live or rng.random() < 0.6):
            rid, toks = waiting.pop(0)
            live[rid] = list(toks)
            mode[rid] = "prefill"
        portions, ended = {}, []
        for rid in list(live):
            if rng.random() < 0.25 and len(portions) + 1 < len(live):
                continue  # this request sits the step out
            rest = live[rid]
            if mode[rid] == "prefill":
                n = min(len(rest), rng.choice([2, 2, 3, 5, max_portion, max_portion * 2]))
                if len(rest) - n <= min(8, len(rest) // 3):
                    mode[rid] = "decode"
            else:
                n = 1
            portions[rid] = rest[:n]
            live[rid] = rest[n:]
            if not live[rid]:
                ended.append(rid)
                del live[rid]
        if portions:
            c.step(portions, end=ended)
    return {rid: c.stacked(rid) for rid in prompts}


def max_rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    scale = want.abs().max().clamp_min(1e-30)
    return float((got - want).abs().max() / scale)
