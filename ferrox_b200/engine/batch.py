"""One step's batch, flattened for the kernels.

A step is a list of entries (request slot, its next tokens, the places among them
whose logits are wanted).  Portions of prompts and single decoded tokens are
treated alike: every token gets its absolute position and the index of its entry,
every entry the slot of its request.  The integer arrays travel to the device in
one copy.

The reference has three entry points that are never mixed in one call
(crates/ferrox-models/src/decoder.rs:1237 one token, :2952 a run of one request's
tokens from ``start_pos``, :3701 one token of each of N requests); per token they
do what this batch describes: rotary angle from the absolute position, K/V stored
at that position, attention over the request's own keys.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    slot: int
    tokens: Sequence[int]
    want: Sequence[int] = ()  # indices into ``tokens``
    start: int = -1  # absolute position of tokens[0]; filled in by the step function


@dataclass
class StepBatch:
    n_tokens: int
    n_seqs: int
    n_want: int
    token_ids: torch.Tensor  # [T] int32
    positions: torch.Tensor  # [T] int32, absolute
    token_seq: torch.Tensor  # [T] int32, index of the token's entry
    seq_slot: torch.Tensor  # [B] int32, slot of each entry's request
    want_rows: torch.Tensor  # [n_want] int32, flat token indices
    status: torch.Tensor  # [1] int32, raised by kernels that meet a bad id or a missing page
    stream: int
    entries: List[StepEntry] = field(default_factory=list)  # host view, for parts written in Python
    max_len: int = 0  # longest request length after this step
    max_new: int = 0  # most tokens any entry brings
    h2d_bytes: int = 0  # size of the step's host-to-device copy
    # per-step values that a part makes once and the layers like it share (rotary tables, the work lists of a
    # mixer's kernels), under keys of the part's own choosing
    shared: dict = field(default_factory=dict)


def flatten(entries: Sequence[StepEntry], device, status: torch.Tensor, stream: int) -> StepBatch:
    T = sum(len(e.tokens) for e in entries)
    B = len(entries)
    W = sum(len(e.want) for e in entries)
    buf = np.empty(3 * T + B + W, dtype=np.int32)
    tok, pos, seq = buf[:T], buf[T:2 * T], buf[2 * T:3 * T]
    slots, want = buf[3 * T:3 * T + B], buf[3 * T + B:3 * T + B + W]
    t = w = 0
    max_len = max_new = 0
    for b, e in enumerate(entries):
        n = len(e.tokens)
        tok[t:t + n] = e.tokens
        pos[t:t + n] = np.arange(e.start, e.start + n, dtype=np.int32)
        seq[t:t + n] = b
        slots[b] = e.slot
        for i in e.want:
            if not 0 <= i < n:
                raise ValueError(f"want index {i} outside the entry's {n} tokens")
            want[w] = t + i
            w += 1
        t += n
        max_len = max(max_len, e.start + n)
        max_new = max(max_new, n)
    dev = torch.from_numpy(buf).to(device, non_blocking=False)
    return StepBatch(
        n_tokens=T, n_seqs=B, n_want=W,
        token_ids=dev[:T], positions=dev[T:2 * T], token_seq=dev[2 * T:3 * T],
        seq_slot=dev[3 * T:3 * T + B], want_rows=dev[3 * T + B:3 * T + B + W],
        status=status, stream=stream, entries=list(entries), max_len=max_len, max_new=max_new,
        h2d_bytes=buf.nbytes,
    )
