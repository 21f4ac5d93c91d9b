"""Dense SwiGLU feed-forward: down( silu(gate x) * (up x) ), no bias
(reference: crates/ferrox-moe/src/lib.rs:655-658; decoder.rs:2902-2913)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, register_part


def pack_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[gate rows ; up rows]: one product yields [gate | up] per token."""
    dt = torch.float32 if torch.float32 in (gate.dtype, up.dtype) else gate.dtype
    return torch.cat([gate.to(dt), up.to(dt)], dim=0).contiguous()


class SwigluMlp(FeedForward):
    graph_safe = True
    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        return [
            TensorDecl(p + "gate_proj.weight", (s.intermediate, s.hidden)),
            TensorDecl(p + "up_proj.weight", (s.intermediate, s.hidden)),
            TensorDecl(p + "down_proj.weight", (s.hidden, s.intermediate)),
        ]

    def load(self, src, rt):
        super().load(src, rt)
        p = self.spec.prefix
        self.w_gu = pack_gate_up(src.get(p + "gate_proj.weight"), src.get(p + "up_proj.weight"))
        self.w_down = src.get(p + "down_proj.weight")

    def forward_add(self, x, h, batch):
        T, I = x.shape[0], self.spec.intermediate
        act = self.rt.empty(T, I)
        ops.gated_linear(x, self.w_gu, act, status=batch.status, stream=batch.stream)  # silu(gate) * up in the epilogue
        ops.linear(act, self.w_down, h, accumulate=True, status=batch.status, stream=batch.stream)


register_part("swiglu_mlp", SwigluMlp, replace=True)
