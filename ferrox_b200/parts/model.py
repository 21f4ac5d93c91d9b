"""The decoder as data: an embedding, a list of blocks, the order in which they run
(the schedule), a final norm and the output head.

``forward`` runs exactly the tokens of one step: embedding rows, every schedule
entry against its cache, then the final norm and the head at the rows whose logits
are wanted (reference: final norm and head crates/ferrox-models/src/decoder.rs:
2193-2198; head on the last row only :2994-3009; tied head loader.rs:1428-1436).
"""
from __future__ import annotations

from typing import List

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import Part, Runtime, build_part


class DecoderModel(Part):
    def __init__(self, spec):
        super().__init__(spec)
        self.layers = [build_part(b) for b in spec.layers]
        self.final_norm = build_part(spec.final_norm)
        for e in spec.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, the model has {len(self.layers)}")
        self._check_cache_sharing()

    def _check_cache_sharing(self):
        seen = {}
        for e in self.spec.schedule:
            cs = self.layers[e.layer].mixer.cache_spec()
            if e.cache in seen and seen[e.cache] != cs:
                raise ValueError(f"cache {e.cache} is shared by layers whose cache needs differ")
            seen[e.cache] = cs

    def cache_specs(self) -> list:
        """One entry per cache index: what the layers bound to it need."""
        out = [None] * self.spec.n_caches
        for e in self.spec.schedule:
            out[e.cache] = self.layers[e.layer].mixer.cache_spec()
        return out

    def tensor_decls(self) -> List[TensorDecl]:
        s = self.spec
        d = [TensorDecl(s.embedding_name, (s.vocab_size, s.hidden))]
        for layer in self.layers:
            d += layer.tensor_decls()
        d += self.final_norm.tensor_decls()
        if s.head_name is not None:
            d.append(TensorDecl(s.head_name, (s.vocab_size, s.hidden)))
        return d

    def load(self, src, rt: Runtime) -> None:
        super().load(src, rt)
        s = self.spec
        self.embedding = src.get(s.embedding_name)
        for layer in self.layers:
            layer.load(src, rt)
        self.final_norm.load(src, rt)
        self.head = self.embedding if s.head_name is None else src.get(s.head_name)

    def reset_after_fault(self) -> None:
        for layer in self.layers:
            layer.reset_after_fault()
        self.final_norm.reset_after_fault()

    def graph_safe(self) -> bool:
        return all(l.graph_safe for l in self.layers) and self.final_norm.graph_safe

    def weight_bytes(self) -> int:
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for v in vars(obj).values():
                if isinstance(v, torch.Tensor) and v.is_cuda and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
                elif isinstance(v, Part):
                    visit(v)
                elif isinstance(v, list):
                    for x in v:
                        if isinstance(x, Part):
                            visit(x)

        visit(self)
        return total

    def forward(self, batch, caches) -> torch.Tensor:
        """``caches(entry) -> LayerCache``.  Returns [len(want_rows), vocab] float32."""
        s, rt = self.spec, self.rt
        h = rt.empty(batch.n_tokens, s.hidden, dtype=torch.float32)
        with ops.trace_scope("embedding"):
            ops.embed(self.embedding, batch.token_ids, h, status=batch.status, stream=batch.stream)
        x = None    # the next block's first norm of h, when the block before it has computed it
        for i, entry in enumerate(s.schedule):
            block = self.layers[entry.layer]
            if not block.passes_norm:
                block.forward(h, batch, caches(entry))
                x = None
                continue
            nxt = self.layers[s.schedule[i + 1].layer] if i + 1 < len(s.schedule) else None
            then = nxt.norm1 if nxt is not None and nxt.passes_norm else None
            x = block.forward(h, batch, caches(entry), x=x, then_norm=then)
        if batch.n_want == 0:
            return rt.empty(0, s.vocab_size, dtype=torch.float32, fresh=True)
        with ops.trace_scope("head"):
            x = self.final_norm.forward(h, rows=batch.want_rows)
            logits = rt.empty(batch.n_want, s.vocab_size, dtype=torch.float32, fresh=True)   # the caller's
            ops.linear(x, self.head, logits, status=batch.status, stream=batch.stream)
        return logits
