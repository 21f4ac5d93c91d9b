"""RMSNorm: x * (1 / sqrt(mean(x^2) + eps)) * w, statistics in 32 bits
(reference: crates/ferrox-core/src/matmul.rs:62-69,121-123)."""
from __future__ import annotations

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Norm, register_part


class RmsNorm(Norm):
    graph_safe = True
    def tensor_decls(self):
        return [TensorDecl(self.spec.prefix + "weight", (self.spec.size,), init="ones")]

    def load(self, src, rt):
        super().load(src, rt)
        self.weight = src.get(self.spec.prefix + "weight")

    def forward(self, h, rows=None):
        n = h.shape[0] if rows is None else rows.numel()
        out = self.rt.empty(n, self.spec.size)
        return ops.rmsnorm(h, self.weight, self.spec.eps, out, rows=rows)


    def as_rms(self):
        return self.weight, self.spec.eps


register_part("rms_norm", RmsNorm, replace=True)
