"""Choice of the next token: greedy, or temperature with top-k / top-p and a
repetition penalty, as the reference samples
(crates/ferrox-models/src/sampling.rs:14-52 parameters, :93-189 procedure).

The logits stay on the device; the kernels of ``csrc/sampling.cu`` do the work.  The
uniform draws come from the reference's generator (:67-84: the xorshift step
``s ^= s<<13; s ^= s>>7; s ^= s<<17``, seed 0 replaced by 0x9E3779B97F4A7C15, a
draw being the top 24 bits / 2^24), one generator per request, so a request's
sample stream does not depend on what it is batched with.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence

import torch

_MASK = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.0  # <= 0: greedy
    top_k: int = 0  # 0: off
    top_p: float = 1.0  # 1: off
    repetition_penalty: float = 1.0  # 1: off; applied to the tokens generated so far
    seed: int = 0

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0


class XorShift64:
    def __init__(self, seed: int):
        seed &= _MASK
        self.state = seed if seed != 0 else 0x9E3779B97F4A7C15

    def next_u64(self) -> int:
        s = self.state
        s ^= (s << 13) & _MASK
        s ^= s >> 7
        s ^= (s << 17) & _MASK
        self.state = s
        return s

    def next_f32(self) -> float:
        return (self.next_u64() >> 40) / float(1 << 24)


class Sampler:
    """Samples one token per row of a [n, vocab] float32 logits tensor on the device."""

    def __init__(self, device):
        self.device = torch.device(device)

    def sample(self, logits: torch.Tensor, params: Sequence[SamplingParams], rngs: Sequence[XorShift64],
               histories: Sequence[Sequence[int]]) -> List[int]:
        from ..kernels import ops

        n = logits.shape[0]
        if n == 0:
            return []
        dev = self.device
        out = torch.empty(n, dtype=torch.int32, device=dev)
        plain = all(p.greedy and p.repetition_penalty == 1.0 for p in params)
        if plain:
            return ops.argmax(logits, out).tolist()
        work = logits.clone()
        if any(p.repetition_penalty != 1.0 and len(h) for p, h in zip(params, histories)):
            flat, offs = [], [0]
            for p, h in zip(params, histories):
                if p.repetition_penalty != 1.0:
                    flat.extend(h)
                offs.append(len(flat))
            hist = torch.tensor(flat or [0], dtype=torch.int32, device=dev)
            offsets = torch.tensor(offs, dtype=torch.int32, device=dev)
            pen = torch.tensor([p.repetition_penalty for p in params], dtype=torch.float32, device=dev)
            ops.repetition_penalty(work, hist, offsets, pen)
        greedy_ids = ops.argmax(work, out).tolist()
        if all(p.greedy for p in params):
            return greedy_ids
        temp = torch.tensor([p.temperature if not p.greedy else 1.0 for p in params], dtype=torch.float32, device=dev)
        top_k = torch.tensor([p.top_k for p in params], dtype=torch.int32, device=dev)
        top_p = torch.tensor([p.top_p for p in params], dtype=torch.float32, device=dev)
        # (the reference draws only once the filtered mass has turned out positive, sampling.rs:160-168: a request
        # whose candidates were all filtered away gets its generator's state back below)
        before = [r.state for r in rngs]
        draws = [r.next_f32() if not p.greedy else 0.0 for p, r in zip(params, rngs)]
        draw = torch.tensor(draws, dtype=torch.float32, device=dev)
        sampled = torch.empty(n, dtype=torch.int32, device=dev)
        ops.sample(work, temp, top_k, top_p, draw, sampled)  # turns ``work`` into probabilities
        sampled = sampled.tolist()
        fallback = None
        result = []
        for i, p in enumerate(params):
            if p.greedy:
                result.append(greedy_ids[i])
            elif sampled[i] >= 0:
                result.append(sampled[i])
            else:  # every candidate filtered away: greedy on the untouched logits (sampling.rs:160-165), no draw used
                rngs[i].state = before[i]
                if fallback is None:
                    fallback = ops.argmax(logits, torch.empty(n, dtype=torch.int32, device=dev)).tolist()
                result.append(fallback[i])
        return result
