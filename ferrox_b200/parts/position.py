"""Position encodings as parameters of the attention mixer.

``rope_neox``: pairs (i, i + r/2) of the first r = ``rotary_dim`` elements of every
query and key head are rotated by pos * theta^(-2i/r) (reference:
crates/ferrox-core/src/attention.rs:20-32).  The table of inverse frequencies is
made in 32 bits with the reference's expression, 1 / theta^(2i/r); the angle, sine
and cosine are computed in 32 bits inside the kernel.
"""
from __future__ import annotations

import torch

from .base import Part, register_part


class RopeNeox(Part):
    graph_safe = True
    def load(self, src, rt):
        super().load(src, rt)
        r = self.spec.rotary_dim
        i = torch.arange(0, r // 2, dtype=torch.float32)
        expo = (2.0 * i) / float(r)
        theta = torch.tensor(float(self.spec.theta), dtype=torch.float32)
        self.inv_freq = (1.0 / torch.pow(theta, expo)).to(torch.float32).to(rt.device)
        self.rotary_dim = r

    def table(self, batch):
        """cos and sin of this step's angles, made once and shared by every layer with
        the same base and width."""
        from ..kernels import ops

        key = ("rope_neox", float(self.spec.theta), self.rotary_dim)
        t = batch.shared.get(key)
        if t is None:
            t = self.rt.empty(batch.n_tokens, self.rotary_dim // 2, 2, dtype=torch.float32)
            ops.rope_table(batch.positions, self.inv_freq, t, stream=batch.stream)
            batch.shared[key] = t
        return t


class NoPosition(Part):
    graph_safe = True
    """No position encoding: keys and queries are stored as projected."""

    def load(self, src, rt):
        super().load(src, rt)
        self.inv_freq = None
        self.rotary_dim = 0

    def table(self, batch):
        return None


register_part("rope_neox", RopeNeox, replace=True)
register_part("no_position", NoPosition, replace=True)
