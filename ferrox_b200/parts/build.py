"""From a :class:`~ferrox_b200.parts.specs.ModelSpec` to a model made of parts."""
from __future__ import annotations

# importing the modules registers the parts that ship with the framework
from . import attention, block, mlp, moe, norm, position  # noqa: F401
from .model import DecoderModel


def build_model(spec) -> DecoderModel:
    return DecoderModel(spec)
