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


@dataclass
class Runtime:
    device: torch.device
    dtype: torch.dtype  # compute dtype: torch.float32 or torch.bfloat16

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)


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
