"""Position encodings: parts that the attention mixer builds from its spec and asks to apply themselves.

    PositionEncoding.rotate_and_store(qkv, batch, cache, n_heads, n_kv_heads, head_dim)

encodes each token's absolute position into the query and key heads of the fused [q|k|v] rows, in place, and stores
the keys (as encoded) and the values in the layer's cache pages.  The mixer knows nothing of how: another pairing of
the elements, other frequencies per band or no rotation at all is another part with this one method.

``rope_neox``: pairs (i, i + r/2) of the first r = ``rotary_dim`` elements of every query and key head are rotated by
pos * theta^(-2i/r) (reference: crates/ferrox-core/src/attention.rs:20-32).  The table of inverse frequencies is made
in 32 bits with the reference's expression, 1 / theta^(2i/r); the angle, sine and cosine are computed in 32 bits on
the device.  The kernel behind it takes the pairing rule and the frequency table as arguments, as the reference
carries split-half and adjacent pairing and per-band frequency factors side by side (attention.rs:319-370).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Part, register_part


class PositionEncoding(Part):
    def rotate_and_store(self, qkv, batch, cache, n_heads: int, n_kv_heads: int, head_dim: int) -> None:
        raise NotImplementedError  # pragma: no cover - interface

    def in_decode_kernel(self, batch, head_dim: int):
        """Optional.  A decode step of one token a request can leave this part's work to the attention kernel
        (``ops.decode_attention(store_new=True)``: split-half rotation over the whole head from a table of cos and
        sin, or none).  A part whose encoding is of that form returns the one-element tuple (table or None); any
        other returns None (the default) and is asked to :meth:`rotate_and_store` as always."""
        return None


class RotaryEncoding(PositionEncoding):
    """Rotation of element pairs by pos * inv_freq[i]: a frequency table, a pairing rule and a rotary width.
    Subclasses set them in ``load`` (or override :meth:`frequencies`)."""

    graph_safe = True
    pairing = ops.PAIR_HALVES

    def frequencies(self) -> torch.Tensor:
        """[rotary_dim / 2] float32 on the CPU: 1 / theta^(2i/r), the reference's expression in 32 bits."""
        r = self.spec.rotary_dim
        i = torch.arange(0, r // 2, dtype=torch.float32)
        theta = torch.tensor(float(self.spec.theta), dtype=torch.float32)
        return (1.0 / torch.pow(theta, (2.0 * i) / float(r))).to(torch.float32)

    def load(self, src, rt):
        super().load(src, rt)
        self.rotary_dim = int(self.spec.rotary_dim)
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim={self.rotary_dim}: pairs need an even width")
        self.inv_freq = self.frequencies().to(rt.device)
        # what makes two parts' tables of a step the same table
        self._table_key = ("rotary table", self.rotary_dim, self.inv_freq.cpu().numpy().tobytes())

    def table(self, batch):
        """cos and sin of this step's angles, made once and shared by every layer with the same frequencies."""
        t = batch.shared.get(self._table_key)
        if t is None:
            t = self.rt.empty(batch.n_tokens, self.rotary_dim // 2, 2, dtype=torch.float32)
            ops.rope_table(batch.positions, self.inv_freq, t, stream=batch.stream)
            batch.shared[self._table_key] = t
        return t

    def in_decode_kernel(self, batch, head_dim):
        if self.pairing != ops.PAIR_HALVES or self.rotary_dim != head_dim:
            return None
        return (self.table(batch),)

    def rotate_and_store(self, qkv, batch, cache, n_heads, n_kv_heads, head_dim):
        if self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} exceeds head_dim={head_dim}")
        ops.rope_kv_write(
            qkv, batch.positions, batch.token_seq, batch.seq_slot, self.inv_freq, self.rotary_dim, cache.k, cache.v,
            cache.block_table, cache.page_size, n_heads, n_kv_heads, head_dim, write_cache=cache.writes,
            status=batch.status, stream=batch.stream, cos_sin=self.table(batch), pairing=self.pairing,
        )


class RopeNeox(RotaryEncoding):
    pairing = ops.PAIR_HALVES


class NoPosition(PositionEncoding):
    """No position encoding: keys and queries are stored as projected."""

    graph_safe = True

    def in_decode_kernel(self, batch, head_dim):
        return (None,)

    def rotate_and_store(self, qkv, batch, cache, n_heads, n_kv_heads, head_dim):
        ops.rope_kv_write(
            qkv, batch.positions, batch.token_seq, batch.seq_slot, None, 0, cache.k, cache.v, cache.block_table,
            cache.page_size, n_heads, n_kv_heads, head_dim, write_cache=cache.writes, status=batch.status,
            stream=batch.stream,
        )


register_part("rope_neox", RopeNeox, replace=True)
register_part("no_position", NoPosition, replace=True)
