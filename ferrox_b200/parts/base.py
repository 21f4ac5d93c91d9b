"""Interfaces of the parts and the registry that maps a spec's ``kind`` to its class.

Every part is built from its spec alone, declares the tensors it expects
(``tensor_decls``), takes them from a :class:`~ferrox_b200.weights.loader.WeightSource`
(``load``) and runs on the tokens of one step.  The residual stream ``h`` is a
32-bit [tokens, hidden] tensor in both engines; a part that adds to it does the
addition in 32 bits.

    Norm.forward(h, rows=None)            -> x  [tokens or len(rows), hidden], compute dtype
    Mixer.cache_spec()                    -> CacheSpec or None
    Mixer.forward_add(x, h, batch, cache) -> None      (h += mixer(x))
    FeedForward.forward_add(x, h, batch)  -> None      (h += ffn(x))
    Block.forward(h, batch, cache)        -> None

``batch`` is the step's :class:`~ferrox_b200.engine.batch.StepBatch` (token
positions, which request each token belongs to, the requests' slots); ``cache`` is
the :class:`~ferrox_b200.cache.manager.LayerCache` of the schedule entry that is
running.  No part knows which model it is in or which layer it is.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List

import torch

from ..weights.loader import TensorDecl


# A step of few tokens costs the host more than the device (a launch takes the GPU a few microseconds and Python as
# long again to prepare); a sixth of that is the caching allocator, asked some 15 times a layer for buffers of the
# same shapes as in the step before.  Steps of up to REUSE_MAX_TOKENS tokens that are not captured into a graph keep
# their buffers instead: the n-th request of a step gets the n-th buffer of the step before if shape and type agree.
# What a step hands to its caller (the logits) never comes from there.
REUSE_MAX_TOKENS = 512
REUSE_MAX_BYTES = 1 << 30


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype  # compute dtype: torch.float32 or torch.bfloat16

    def __post_init__(self):
        self._kept = []          # buffers of the last small step, in the order they were asked for
        self._next = -1          # index of the next request; -1: buffers are not kept
        self._kept_bytes = 0

    def begin_step(self, n_tokens: int) -> None:
        """An eager step begins (never inside a graph capture: a graph owns its memory)."""
        self._next = 0 if 0 < n_tokens <= REUSE_MAX_TOKENS and self.device.type == "cuda" else -1

    def end_step(self) -> None:
        self._next = -1

    def empty(self, *shape, dtype=None, fresh: bool = False) -> torch.Tensor:
        """``fresh``: a buffer of the caller's own, for what outlives the step."""
        dt = dtype or self.dtype
        i = self._next
        if i < 0 or fresh:
            return torch.empty(shape, dtype=dt, device=self.device)
        self._next = i + 1
        kept = self._kept
        if i < len(kept):
            t = kept[i]
            if t is not None and t.shape == shape and t.dtype == dt:
                return t
        t = torch.empty(shape, dtype=dt, device=self.device)
        n = t.numel() * t.element_size()
        if i < len(kept):
            old = kept[i]
            if old is not None:
                self._kept_bytes -= old.numel() * old.element_size()
            kept[i] = None
        if self._kept_bytes + n <= REUSE_MAX_BYTES:
            if i < len(kept):
                kept[i] = t
            else:
                kept.extend([None] * (i - len(kept)))
                kept.append(t)
            self._kept_bytes += n
        return t


class Part:
    # True when ``forward`` only enqueues kernels on the batch's stream at fixed
    # addresses (no host reads of device data, no Python state that changes per
    # step), so that a decode step can be captured in a CUDA graph.
    graph_safe = False

    def __init__(self, spec):
        self.spec = spec
        self.rt: Runtime | None = None

    def tensor_decls(self) -> List[TensorDecl]:
        return []

    def load(self, src, rt: Runtime) -> None:
        self.rt = rt

    def reset_after_fault(self) -> None:
        """Called after a step whose kernels raised the status word: put back any device-side scratch that an
        aborted kernel may have left half-used.  Parts that own parts pass the call on."""


class Norm(Part):
    def forward(self, h: torch.Tensor, rows=None) -> torch.Tensor:  # pragma: no cover - interface
        raise NotImplementedError

    def as_rms(self):
        """(weight, eps) if this norm is x / sqrt(mean(x^2) + eps) * weight over whole rows, which a kernel that
        has just produced the rows can apply itself; None otherwise."""
        return None


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward_add(self, x, h, batch, cache) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class FeedForward(Part):
    # A feed-forward whose last kernel can also apply the norm that follows it sets ``fuses_norm`` and takes
    # ``forward_add(x, h, batch, then_norm=norm)``: it returns that norm's output on the new ``h``, or None if it
    # left the norm to the caller.  Parts without the flag are never given the argument.
    fuses_norm = False

    def forward_add(self, x, h, batch) -> None:  # pragma: no cover - interface
        raise NotImplementedError


class Block(Part):
    mixer: Mixer
    # A block that can take its first norm's output from the block before it (``forward(..., x=...)``) and hand the
    # next block's to it (``then_norm=`` that block's first norm; returns its output or None) sets ``passes_norm``
    # and names its first norm ``norm1``.  Blocks without the flag are called with (h, batch, cache) only.
    passes_norm = False

    def forward(self, h, batch, cache) -> None:  # pragma: no cover - interface
        raise NotImplementedError


_PARTS: Dict[str, Callable] = {}


def register_part(kind: str, factory: Callable, *, replace: bool = False) -> None:
    """``factory(spec) -> Part``.  ``kind`` is the string a spec carries."""
    if kind in _PARTS and not replace:
        raise ValueError(f"part kind {kind!r} is already registered")
    _PARTS[kind] = factory


def build_part(spec) -> Part:
    kind = getattr(spec, "kind", None)
    if kind not in _PARTS:
        raise ValueError(f"no part registered for kind {kind!r}; known: {', '.join(sorted(_PARTS))}")
    return _PARTS[kind](spec)
