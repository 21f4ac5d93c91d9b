"""What a mixer asks of the cache manager, as plain data.

A mixer may need keys and values in pages (:class:`KvCacheSpec`; ``window`` tells
how far back it reads, which decides when pages can be given back), a block of
fixed size per request (:class:`StateSpec`; recurrent mixers), both, or nothing.
The reference's counterpart is the ``Engine::State`` associated type
(crates/ferrox-models/src/engine.rs:44-53): ``Vec<KvCache>`` for its decoder, a
fixed recurrent state for its linear-attention model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class KvCacheSpec:
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # None: every earlier position stays readable


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheSpec:
    kv: Optional[KvCacheSpec] = None
    state: Optional[StateSpec] = None
