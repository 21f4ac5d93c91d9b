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
        vocab = model.spec.vocab_size
        if min(e.tokens) < 0 or max(e.tokens) >= vocab:
            raise ValueError(f"token id outside the vocabulary of {vocab}")
    # all-or-nothing reservation across the entries, in one call of the native book-keeping
    slots, counts = [e.slot for e in entries], [len(e.tokens) for e in entries]
    starts = cache.reserve_step(slots, counts)
    if starts is None:
        raise OutOfPages(f"step of {sum(counts)} tokens does not fit the free pages {cache.free_pages()}")
    for e, st in zip(entries, starts):
        e.start = st
    cache.sync_tables()

    status = _status(model.rt.device)
    logits = None
    if graphs is not None and graphs.eligible(entries):
        logits = graphs.run(entries, status)
        last_h2d_bytes = 20 * len(entries)
    if logits is None:
        batch = flatten(entries, model.rt.device, status, ops.stream_ptr())
        last_h2d_bytes = batch.h2d_bytes
        model.rt.begin_step(batch.n_tokens)      # small eager steps keep their buffers from step to step
        try:
            with ops.stream_scope(batch.stream):
                logits = model.forward(batch, lambda entry: cache.layer_cache(entry.cache, entry.writes_cache))
        finally:
            model.rt.end_step()
    if check:
        code = int(status.item())
        if code:
            # The requests' lengths have not advanced: the step counts as not run (its pages stay mapped, which a
            # later step of the same requests finds done).  Parts put back what an aborted kernel may have left.
            status.zero_()
            model.reset_after_fault()
            what = {1: "a token id outside the vocabulary", 2: "a position without a cache page",
                    3: "a bounded wait that ran out inside a tensor-core kernel"}.get(code, code)
            raise StepFault(f"step met {what}")
    cache.commit_step(slots, counts)
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
        self.sampled = {}   # graphs that end with the choice of the next tokens by sampling, for steps issued ahead
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

    def _capture(self, B, entries, status, sampled: bool = False):
        """``sampled``: the graph ends with temperature / top-k / top-p sampling instead of the arg max alone; its
        static buffer holds five more runs of B values (top_k, sample or not, temperature, top_p, draw)."""
        import numpy as np

        dev = self.model.rt.device
        n = 10 * B if sampled else 5 * B
        host = torch.zeros(n, dtype=torch.int32).pin_memory()
        arr = host.numpy()
        arr[2 * B:3 * B] = np.arange(B)  # token_seq: token b belongs to entry b
        arr[4 * B:5 * B] = np.arange(B)  # want_rows: every row
        for b, e in enumerate(entries):
            arr[b], arr[B + b], arr[3 * B + b] = e.tokens[0], e.start, e.slot
        buf = torch.empty(n, dtype=torch.int32, device=dev)
        buf.copy_(host)
        chosen = torch.zeros(B, dtype=torch.int32, device=dev)   # arg max of each row of the logits, for steps issued ahead
        if sampled:
            best = torch.zeros(B, dtype=torch.int32, device=dev)
            work = torch.empty(B, self.model.spec.vocab_size, dtype=torch.float32, device=dev)
            fl = buf.view(torch.float32)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops.launch_count()
        with torch.cuda.graph(graph):
            batch = StepBatch(
                n_tokens=B, n_seqs=B, n_want=B, token_ids=buf[:B], positions=buf[B:2 * B], token_seq=buf[2 * B:3 * B],
                seq_slot=buf[3 * B:4 * B], want_rows=buf[4 * B:5 * B], status=status, stream=ops.stream_ptr(),
                entries=list(entries), max_len=self.cache.max_positions, max_new=1, h2d_bytes=20 * B,
            )
            with ops.stream_scope(batch.stream):
                logits = self.model.forward(batch, lambda entry: self.cache.layer_cache(entry.cache, entry.writes_cache))
                if sampled:
                    ops.argmax(logits, best)
                    ops.sample_or(logits, work, fl[7 * B:8 * B], buf[5 * B:6 * B], fl[8 * B:9 * B], fl[9 * B:10 * B],
                                  buf[6 * B:7 * B], best, chosen)
                else:
                    ops.argmax(logits, chosen)
        self.kernels_per_replay[(B, sampled)] = ops.launch_count() - before
        if not sampled:
            self.kernels_per_replay[B] = self.kernels_per_replay[(B, False)]
        (self.sampled if sampled else self.graphs)[B] = {
            "graph": graph, "host": host, "dev": buf, "logits": logits, "event": torch.cuda.Event(), "chosen": chosen,
            # steps issued ahead: two pinned buffers each way, used in turn
            "ahead_in": [torch.empty(n, dtype=torch.int32).pin_memory() for _ in range(2)],
            "ahead_in_done": [torch.cuda.Event() for _ in range(2)],
            "ahead_out": [torch.empty(B, dtype=torch.int32).pin_memory() for _ in range(2)],
            "ahead_out_done": [torch.cuda.Event() for _ in range(2)],
        }
        for h in (self.sampled if sampled else self.graphs)[B]["ahead_in"]:
            h.copy_(host)

    def capture_sampled(self, B, slots, status) -> None:
        """The sampling graph of batch size B, captured when decoding ahead first asks for it (the plain graph of
        this size exists by then, so every kernel of the model has run before)."""
        if B in self.sampled:
            return
        entries = []
        for s in slots:
            e = StepEntry(s, [0], want=[0])
            e.start = self.cache.seq_len[s]
            entries.append(e)
        dev = self.model.rt.device
        # the sampling kernel once outside a capture
        z = torch.zeros(1, 4, device=dev)
        one_i, one_f = torch.ones(1, dtype=torch.int32, device=dev), torch.ones(1, device=dev)
        ops.sample_or(z, z.clone(), one_f, one_i, one_f, one_f * 0.5, one_i, one_i, one_i.clone())
        self._capture(B, entries, status, sampled=True)

    # ---- steps issued ahead of the host ------------------------------------------------
    def replay_ahead(self, B, starts, slots, tokens, turn: int, sampling=None) -> None:
        """Replay the graph of size B without waiting for anything.  ``tokens`` None: the step's tokens are the
        ones the previous replay of this size chose, which never left the device.  The chosen tokens of this
        replay travel to pinned memory behind it; :meth:`chosen_tokens` waits for them.  ``sampling``: the
        step's (top_k, sample or not, temperature, top_p, draw), each a list of B; the sampling graph then."""
        g = self.graphs[B] if sampling is None else self.sampled[B]
        g["ahead_in_done"][turn].synchronize()
        host = g["ahead_in"][turn]
        arr = host.numpy()
        arr[B:2 * B] = starts
        arr[3 * B:4 * B] = slots
        if sampling is not None:
            import numpy as np

            top_k, use, temp, top_p, draw = sampling
            arr[5 * B:6 * B] = top_k
            arr[6 * B:7 * B] = use
            arr[7 * B:10 * B].view(np.float32)[:] = list(temp) + list(top_p) + list(draw)
        if tokens is not None:
            arr[:B] = tokens
            g["dev"].copy_(host, non_blocking=True)
        else:
            g["dev"][B:].copy_(host[B:], non_blocking=True)
            g["dev"][:B].copy_(g["chosen"], non_blocking=True)
        g["ahead_in_done"][turn].record()
        g["graph"].replay()
        ops.count_launches(self.kernels_per_replay[(B, sampling is not None)])
        g["ahead_out"][turn].copy_(g["chosen"], non_blocking=True)
        g["ahead_out_done"][turn].record()

    def chosen_tokens(self, B, turn: int, sampled: bool = False):
        g = self.sampled[B] if sampled else self.graphs[B]
        g["ahead_out_done"][turn].synchronize()
        return g["ahead_out"][turn].tolist()


class DecodeAhead:
    """Decode steps of a fixed set of requests, issued one step ahead of the host: step k+1 is on the stream
    before the host has read what step k chose.  The chosen token of a request is fed to its next step on the
    device; the host reads it one step later, from pinned memory.  A step maps its pages and advances the
    requests' lengths when it is issued (both depend on counts only, not on the tokens).

    Greedy by default.  ``sampling``: per request its (SamplingParams, generator); the choice is then made inside
    the graph by the sampling kernel (no repetition penalty: that needs the tokens on the host).  A request's
    uniform draws come from its own generator, one per step in which it samples, as without the graph: they do
    not depend on the tokens, so the host can send them with the step."""

    def __init__(self, model, cache, graphs, slots, tokens, sampling=None):
        self.model, self.cache, self.graphs = model, cache, graphs
        self.slots, self.first_tokens = list(slots), list(tokens)
        self.B = len(self.slots)
        self._ones = [1] * self.B
        self.issued = self.collected = 0
        self.sampling = None
        if sampling is not None and any(not p.greedy for p, _ in sampling):
            if any(p.repetition_penalty != 1.0 for p, _ in sampling):
                raise ValueError("steps issued ahead cannot apply a repetition penalty")
            self.sampling = list(sampling)
            graphs.capture_sampled(self.B, self.slots, _status(model.rt.device))

    @staticmethod
    def ready(graphs, n: int) -> bool:
        return graphs is not None and n in graphs.graphs

    def issue(self) -> None:
        """Maps a page where a request needs one (all requests or none: OutOfPages before any change), then
        replays the step."""
        global last_h2d_bytes
        cache = self.cache
        starts = cache.reserve_step(self.slots, self._ones)
        if starts is None:
            raise OutOfPages(f"a decode step of {self.B} requests does not fit the free pages {cache.free_pages()}")
        cache.sync_tables()
        first = self.issued == 0
        step_sampling = None
        if self.sampling is not None:
            ps = [p for p, _ in self.sampling]
            step_sampling = ([p.top_k for p in ps], [0 if p.greedy else 1 for p in ps],
                             [1.0 if p.greedy else p.temperature for p in ps], [p.top_p for p in ps],
                             [0.0 if p.greedy else g.next_f32() for p, g in self.sampling])
        self.graphs.replay_ahead(self.B, starts, self.slots, self.first_tokens if first else None, self.issued & 1,
                                 step_sampling)
        last_h2d_bytes = ((20 if first else 16) + (20 if step_sampling else 0)) * self.B
        cache.commit_step(self.slots, self._ones)
        self.issued += 1

    def collect(self):
        """The tokens chosen by the oldest step not read yet (waits for it)."""
        toks = self.graphs.chosen_tokens(self.B, self.collected & 1, self.sampling is not None)
        self.collected += 1
        return toks

    def close(self) -> None:
        status = _status(self.model.rt.device)
        code = int(status.item())
        if code:
            status.zero_()
            self.model.reset_after_fault()
            raise StepFault(f"a step issued ahead met fault code {code}")
