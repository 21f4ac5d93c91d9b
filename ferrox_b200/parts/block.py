"""Arrangement of a layer's parts: pre-norm with two residual additions,

    h += mixer(norm1(h));  h += ffn(norm2(h))

(reference: crates/ferrox-models/src/decoder.rs:2054-2173).  The block asks its
mixer what cache it needs and passes the step's batch through; it is built from
whatever norm, mixer and feed-forward its spec names.
"""
from __future__ import annotations

from ..kernels import ops
from .base import Block, build_part, register_part


class PreNormBlock(Block):
    def __init__(self, spec):
        super().__init__(spec)
        self.norm1 = build_part(spec.norm1)
        self.mixer = build_part(spec.mixer)
        self.norm2 = build_part(spec.norm2)
        self.ffn = build_part(spec.ffn)

    def tensor_decls(self):
        return (
            self.norm1.tensor_decls() + self.mixer.tensor_decls() + self.norm2.tensor_decls() + self.ffn.tensor_decls()
        )

    def load(self, src, rt):
        super().load(src, rt)
        for part in (self.norm1, self.mixer, self.norm2, self.ffn):
            part.load(src, rt)

    def reset_after_fault(self):
        for part in (self.norm1, self.mixer, self.norm2, self.ffn):
            part.reset_after_fault()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in (self.norm1, self.mixer, self.norm2, self.ffn))

    passes_norm = True

    def forward(self, h, batch, cache, x=None, then_norm=None):
        """``x``: norm1(h) if the block before has computed it.  ``then_norm``: the first norm of the block that runs
        next; its output on the new h is returned if the feed-forward's last kernel applied it, else None."""
        if x is None:
            with ops.trace_scope("norm"):
                x = self.norm1.forward(h)
        with ops.trace_scope("mixer"):
            self.mixer.forward_add(x, h, batch, cache)
        with ops.trace_scope("norm"):
            x2 = self.norm2.forward(h)
        with ops.trace_scope("feed-forward"):
            if then_norm is not None and self.ffn.fuses_norm:
                return self.ffn.forward_add(x2, h, batch, then_norm=then_norm)
            self.ffn.forward_add(x2, h, batch)
        return None


register_part("pre_norm", PreNormBlock, replace=True)
