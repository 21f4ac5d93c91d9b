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


def step(model, cache, entries: Sequence[StepEntry], *, check: bool = True, graphs=None) -> torch.Tensor:
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
    logits = None
    if graphs is not None and graphs.eligible(entries):
        logits = graphs.run(entries, status)
        last_h2d_bytes = 20 * len(entries)
    if logits is None:
        batch = flatten(entries, model.rt.device, status, ops.stream_ptr())
        last_h2d_bytes = batch.h2d_bytes
        logits = model.forward(batch, lambda entry: cache.layer_cache(entry.cache, entry.writes_cache))
    for e in entries:
        cache.commit(e.slot, e.start + len(e.tokens))
    if check:
        code = int(status.item())
        if code:
            status.zero_()
            what = {1: "a token id outside the vocabulary", 2: "a position without a cache page",
                    3: "a bounded wait that ran out inside a tensor-core kernel"}.get(code, code)
            raise StepFault(f"step met {what}")
    return logits


_status_cache = {}


def _status(device) -> torch.Tensor:
    key = str(device)
    if key not in _status_cache:
        _status_cache[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _status_cache[key]


class GraphedDecode:
    """Decode steps (every entry brings one token and wants its logits) replayed
    from CUDA graphs, one graph per batch size.

    The first decode step of a size runs eagerly; the second is captured; later ones
    copy the step's integers into the graph's static buffer and replay.  Everything
    a graph reads lives at fixed addresses: the static buffer, the cache pages, the
    block tables, the weights and the temporaries of the graph's own memory pool.
    The returned logits are the graph's output buffer: read them before the next
    step of the same size.
    """

    def __init__(self, model, cache, max_batch: int = 256):
        self.model, self.cache = model, cache
        self.max_batch = max_batch
        self.seen = set()
        self.graphs = {}
        self.kernels_per_replay = {}

    def eligible(self, entries) -> bool:
        return (len(entries) <= self.max_batch and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries))

    def run(self, entries, status):
        import numpy as np

        B = len(entries)
        if B not in self.graphs:
            if B not in self.seen:
                self.seen.add(B)
                return None  # first time: the caller runs it eagerly
            self._capture(B, entries, status)
        g = self.graphs[B]
        g["event"].synchronize()  # the previous copy out of the pinned buffer is done
        host = g["host"].numpy()
        for b, e in enumerate(entries):
            host[b] = e.tokens[0]
            host[B + b] = e.start
            host[3 * B + b] = e.slot
        g["dev"].copy_(g["host"], non_blocking=True)
        g["event"].record()
        g["graph"].replay()
        ops.count_launches(self.kernels_per_replay[B])
        return g["logits"]

    def _capture(self, B, entries, status):
        import numpy as np

        dev = self.model.rt.device
        n = 5 * B
        host = torch.empty(n, dtype=torch.int32).pin_memory()
        arr = host.numpy()
        arr[2 * B:3 * B] = np.arange(B)  # token_seq: token b belongs to entry b
        arr[4 * B:5 * B] = np.arange(B)  # want_rows: every row
        for b, e in enumerate(entries):
            arr[b], arr[B + b], arr[3 * B + b] = e.tokens[0], e.start, e.slot
        buf = torch.empty(n, dtype=torch.int32, device=dev)
        buf.copy_(host)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            batch = StepBatch(
                n_tokens=B, n_seqs=B, n_want=B, token_ids=buf[:B], positions=buf[B:2 * B], token_seq=buf[2 * B:3 * B],
                seq_slot=buf[3 * B:4 * B], want_rows=buf[4 * B:], status=status, stream=ops.stream_ptr(),
                entries=list(entries), max_len=self.cache.max_positions, max_new=1, h2d_bytes=4 * n,
            )
            logits = self.model.forward(batch, lambda entry: self.cache.layer_cache(entry.cache, entry.writes_cache))
        self.kernels_per_replay[B] = ops.launch_count() - before
        self.graphs[B] = {"graph": graph, "host": host, "dev": buf, "logits": logits, "event": torch.cuda.Event()}
