"""Weights by tensor name.

Every part declares the tensors it expects (:class:`TensorDecl`: name, shape, role).
:func:`check_declared` compares the declarations of a whole model with what a model
folder holds and raises ONE :class:`WeightsError` that lists every missing tensor,
every unexpected one and every wrong shape, each by name (the reference fails on
the first: ``TensorNotFound`` / ``ExpertCountMismatch``,
crates/ferrox-models/src/loader.rs:38-65,751-759,806-813).

Precision rule (:func:`resident_dtype`): in the bfloat16 engine a tensor stored in
16 bits is kept in bfloat16 and a tensor stored in 32 bits stays in 32 bits; integer
tables become int32; the 32-bit engine widens everything to float32 (exact for
bfloat16 and float16 inputs; the reference widens BF16 once at load,
loader.rs:762-770).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Sequence, Tuple

import torch

from .safetensors_io import ModelFiles


class WeightsError(ValueError):
    """The tensors of a model folder do not fit the model built from its config."""


@dataclass(frozen=True)
class TensorDecl:
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"  # how the random-weights mode fills it: normal | ones | zeros
    optional: bool = False  # present or absent by the file's choice (e.g. a gate vector)
    integer: bool = False  # an integer table (kept as int32)


def resident_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor has on the device for an engine of ``compute`` dtype."""
    if not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def check_declared(available: Dict[str, Tuple[int, ...]], decls: Sequence[TensorDecl], where: str) -> None:
    """``available``: name -> shape of what the folder holds."""
    missing: List[str] = []
    wrong: List[str] = []
    declared = set()
    for d in decls:
        declared.add(d.name)
        if d.name not in available:
            if not d.optional:
                missing.append(f"{d.name} {list(d.shape)}")
            continue
        found = tuple(available[d.name])
        if found != tuple(d.shape):
            wrong.append(f"{d.name}: expected {list(d.shape)}, found {list(found)}")
    unexpected = sorted(n for n in available if n not in declared)
    if missing or wrong or unexpected:
        parts = [f"{where}: the tensors do not fit the model that config.json describes."]
        if missing:
            parts.append(f"missing ({len(missing)}): " + "; ".join(missing))
        if unexpected:
            parts.append(f"unexpected ({len(unexpected)}): " + "; ".join(unexpected))
        if wrong:
            parts.append(f"wrong shape ({len(wrong)}): " + "; ".join(wrong))
        raise WeightsError("\n  ".join(parts))


class WeightSource:
    """What a part's ``load`` reads from: ``has(name)`` and ``get(name)``, the latter
    returning the tensor on the engine's device in its resident dtype."""

    def __init__(self, get_cpu: Callable[[str], torch.Tensor], names: Iterable[str], device, compute_dtype,
                 stored_dtype: Callable[[str], torch.dtype] | None = None):
        self._get_cpu = get_cpu
        self._stored_dtype = stored_dtype or (lambda n: get_cpu(n).dtype)
        self._names = set(names)
        self.device = torch.device(device)
        self.compute_dtype = compute_dtype

    def has(self, name: str) -> bool:
        return name in self._names

    def dtype_of(self, name: str) -> torch.dtype:
        """The dtype ``get(name)`` will return, without reading the data."""
        return resident_dtype(self._stored_dtype(name), self.compute_dtype)

    def get(self, name: str) -> torch.Tensor:
        t = self._get_cpu(name)
        want = resident_dtype(t.dtype, self.compute_dtype)
        # Move first, convert on the device: the host copy of a large matrix stays a
        # view of the mapped file.
        return t.to(self.device).to(want).contiguous()


def open_folder(folder: str, decls: Sequence[TensorDecl], device, compute_dtype) -> Tuple[WeightSource, ModelFiles]:
    files = ModelFiles(folder)
    check_declared({n: files.info(n)[1] for n in files.names()}, decls, folder)
    return WeightSource(files.tensor, files.names(), device, compute_dtype, lambda n: files.info(n)[0]), files


def from_dict(tensors: Dict[str, torch.Tensor], decls: Sequence[TensorDecl], device, compute_dtype) -> WeightSource:
    check_declared({n: tuple(t.shape) for n, t in tensors.items()}, decls, "<tensors in memory>")
    return WeightSource(tensors.__getitem__, tensors.keys(), device, compute_dtype)
