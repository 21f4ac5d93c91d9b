"""Plain-data descriptions of the parts a decoder is put together from.

A *spec* carries every size and constant of one part and the name prefix of its
tensors in the checkpoint; it holds no tensors and knows nothing of the model it
ends up in.  An architecture turns its ``config.json`` into a :class:`ModelSpec`
(one :class:`BlockSpec` per layer, chosen layer by layer, plus the order in which
the layers run); ``parts.build`` turns specs into parts that own weights and run
kernels.  New kinds of part register a spec class of their own with the same
``kind`` string as their implementation (``parts.registry``).

The reference keeps the same facts in ``ModelConfig`` and asks them per layer
(``layer_is_dense``, ``layer_sliding_window``, ``layer_rope_theta``;
crates/ferrox-models/src/config.rs:247-277).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    size: int
    eps: float
    prefix: str  # tensor: <prefix>weight
    kind: str = "rms_norm"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding, split-half pairing (i, i + rotary_dim/2)."""

    rotary_dim: int
    theta: float
    kind: str = "rope_neox"


@dataclass(frozen=True)
class NoPositionSpec:
    """Queries and keys are used as projected."""

    kind: str = "no_position"


@dataclass(frozen=True)
class AttentionSpec:
    hidden: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    qkv_bias: bool
    position: Optional[object]  # the spec of a position-encoding part (None: no encoding)
    window: Optional[int]  # None = all earlier keys; W = the last W positions, the query's own included
    prefix: str  # tensors: <prefix>{q,k,v}_proj.{weight,bias}, <prefix>o_proj.weight
    softmax_scale: Optional[float] = None  # None = 1/sqrt(head_dim)
    kind: str = "gqa_attention"


@dataclass(frozen=True)
class DenseMlpSpec:
    hidden: int
    intermediate: int
    prefix: str  # tensors: <prefix>{gate,up,down}_proj.weight
    kind: str = "swiglu_mlp"


@dataclass(frozen=True)
class MoeSpec:
    hidden: int
    n_experts: int
    top_k: int
    expert_intermediate: int
    shared_intermediate: int  # 0 = no shared expert
    norm_topk_prob: bool
    shared_gate: bool  # sigmoid(w . x) scales the shared expert's output
    prefix: str  # tensors: <prefix>gate.weight, <prefix>experts.<e>.{gate,up,down}_proj.weight,
    #                       <prefix>shared_expert.{gate,up,down}_proj.weight, <prefix>shared_expert_gate.weight
    kind: str = "softmax_topk_moe"


@dataclass(frozen=True)
class BlockSpec:
    """h += mixer(norm1(h)); h += ffn(norm2(h))."""

    norm1: object
    mixer: object
    norm2: object
    ffn: object
    kind: str = "pre_norm"


@dataclass(frozen=True)
class ScheduleEntry:
    """One call in the order of execution: run ``layer`` against cache ``cache``.

    ``layer`` may appear in several entries (the same weights run twice) and two
    entries may name the same ``cache`` (the later one reads what the earlier one
    wrote, with ``writes_cache=False``)."""

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: object
    embedding_name: str = "model.embed_tokens.weight"
    head_name: Optional[str] = "lm_head.weight"  # None = tied to the embedding
    eos_token_ids: Tuple[int, ...] = field(default_factory=tuple)

    @property
    def n_caches(self) -> int:
        return 1 + max((e.cache for e in self.schedule), default=-1)
