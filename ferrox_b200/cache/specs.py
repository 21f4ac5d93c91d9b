"""What a mixer asks of the cache manager, as plain data.

A mixer may need something stored per position, in pages (:class:`PagedSpec`: one or
more named tensors, each with the shape of one position's entry; ``window`` tells
how far back the mixer reads, which decides when pages can be given back), a block
of fixed size per request (:class:`StateSpec`; recurrent mixers), both, or nothing.
Keys and values of an attention layer are the built-in case (:func:`KvCacheSpec`);
a mixer that keeps one vector per position, or three tensors, names them itself.

The reference's counterpart is the ``Engine::State`` associated type
(crates/ferrox-models/src/engine.rs:44-53): ``Vec<KvCache>`` for its decoder, a
fixed recurrent state for its linear-attention model.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch


@dataclass(frozen=True)
class PagedTensorSpec:
    """One tensor of a paged payload.  ``token_shape`` is what one position stores.

    ``lead_dims`` of the entry's leading dimensions come before the position inside a page: the tensor is
    ``[n_pages, *token_shape[:lead_dims], page_size, *token_shape[lead_dims:]]``.  Keys and values use
    ``token_shape=(n_kv_heads, head_dim)`` with ``lead_dims=1``, so that one head's positions of a page lie together;
    ``lead_dims=0`` gives ``[n_pages, page_size, *token_shape]``.  ``dtype`` None: the engine's cache dtype."""

    name: str
    token_shape: Tuple[int, ...]
    lead_dims: int = 0
    dtype: Optional[torch.dtype] = None

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        if not 0 <= self.lead_dims <= len(self.token_shape):
            raise ValueError(f"paged tensor {self.name!r}: lead_dims outside its token shape")
        return (*self.token_shape[:self.lead_dims], page_size, *self.token_shape[self.lead_dims:])


@dataclass(frozen=True)
class PagedSpec:
    tensors: Tuple[PagedTensorSpec, ...]
    window: Optional[int] = None  # None: every earlier position stays readable


def KvCacheSpec(n_kv_heads: int, head_dim: int, window: Optional[int] = None) -> PagedSpec:
    """Keys and values of an attention layer: ``k`` and ``v``, each [n_pages, n_kv_heads, page_size, head_dim]."""
    shape = (int(n_kv_heads), int(head_dim))
    return PagedSpec((PagedTensorSpec("k", shape, lead_dims=1), PagedTensorSpec("v", shape, lead_dims=1)), window)


@dataclass(frozen=True)
class StateSpec:
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass(frozen=True)
class CacheSpec:
    paged: Optional[PagedSpec] = None
    state: Optional[StateSpec] = None
