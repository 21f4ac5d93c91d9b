"""The step function: run exactly the tokens given, as one batch, from the cache.

    logits = step(model, cache, entries)

For every entry the cache manager maps pages for the new positions (all entries or
none: a step that does not fit raises :class:`OutOfPages` before anything is
changed), the model runs the flattened batch once, and the requests' lengths
advance.  The logits come back as one [wanted, vocab] float32 tensor in the order of
the entries and of their ``want`` lists.
"""
from __future__ import annotations

from typing import Sequence

import torch

from ..kernels import ops
from .batch import StepBatch, StepEntry, flatten


class OutOfPages(RuntimeError):
    """The step's tokens do not fit the free pages; nothing was changed."""


class StepFault(RuntimeError):
    """A kernel met a token id outside the vocabulary or a position without a page."""


last_h2d_bytes = 0  # host-to-device bytes of the most recent step (token ids, positions, slots)


def step(model, cache, entries: Sequence[StepEntry], *, check: bool = True) -> torch.Tensor:
    global last_h2d_bytes
    if not entries:
        return model.rt.empty(0, model.spec.vocab_size, dtype=torch.float32)
    seen = set()
    for e in entries:
        if e.slot in seen:
            raise ValueError(f"slot {e.slot} appears twice in one step")
        if len(e.tokens) == 0:
            raise ValueError("an entry must bring at least one token")
        seen.add(e.slot)
        e.start = cache.seq_len[e.slot]
        vocab = model.spec.vocab_size
        if min(e.tokens) < 0 or max(e.tokens) >= vocab:
            raise ValueError(f"token id outside the vocabulary of {vocab}")
    # all-or-nothing reservation across the entries
    wanted = {}
    for e in entries:
        for key, n in cache.pages_needed(e.slot, e.start + len(e.tokens)).items():
            wanted[key] = wanted.get(key, 0) + n
    if not cache.can_reserve(wanted):
        raise OutOfPages(f"step needs {wanted} pages, free: {cache.free_pages()}")
    for e in entries:
        ok = cache.reserve(e.slot, e.start + len(e.tokens))
        assert ok
    cache.sync_tables()

    status = _status(model.rt.device)
    batch = flatten(entries, model.rt.device, status, ops.stream_ptr())
    last_h2d_bytes = batch.h2d_bytes
    logits = model.forward(batch, lambda entry: cache.layer_cache(entry.cache, entry.writes_cache))
    for e in entries:
        cache.commit(e.slot, e.start + len(e.tokens))
    if check:
        code = int(status.item())
        if code:
            status.zero_()
            what = {1: "a token id outside the vocabulary", 2: "a position without a cache page"}.get(code, code)
            raise StepFault(f"step met {what}")
    return logits


_status_cache = {}


def _status(device) -> torch.Tensor:
    key = str(device)
    if key not in _status_cache:
        _status_cache[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_cache[key]
