"""Random-weights mode: a model folder from a configuration and a seed.

Each tensor is drawn from a generator seeded by (seed, tensor name), so a tensor's
values do not depend on which other tensors exist or in which order they are made.
Matrices, biases and gate vectors are N(0, std); norm weights are 1 (``norm_init=
"ones"``), 1 + N(0, std) (``"around_one"``) or N(0, std) like everything else
(``"normal"``).  The reference's counterpart is ``Decoder::new_random_small``
(crates/ferrox-models/src/decoder.rs:373-388,397-514: xorshift64*, uniform +-0.05,
norm weights 1, no bias, no shared gate); unlike it, this mode fills biases and the
shared expert's gate as well, so that they are exercised.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterator, Sequence, Tuple

import torch

from .loader import TensorDecl
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.blake2b(f"{seed}:{name}".encode("utf-8"), digest_size=8).digest()
    return int.from_bytes(h, "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(decl: TensorDecl, seed: int, dtype, std: float, norm_init: str, device="cpu") -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_tensor_seed(seed, decl.name))
    if decl.integer:
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=dtype, device=device)
    if decl.init == "ones" and norm_init == "ones":
        return torch.ones(decl.shape, dtype=dtype, device=device)
    t = torch.empty(decl.shape, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
    if decl.init == "ones" and norm_init == "around_one":
        t += 1.0
    elif decl.init == "ones" and norm_init != "normal":
        raise ValueError(f"norm_init={norm_init!r}: expected ones, around_one or normal")
    return t.to(dtype)


def random_tensors(
    decls: Sequence[TensorDecl], seed: int, dtype=torch.bfloat16, std: float = 0.02, norm_init: str = "ones", device="cpu"
) -> Iterator[Tuple[str, torch.Tensor]]:
    for d in decls:
        yield d.name, random_tensor(d, seed, dtype, std, norm_init, device)


def write_random_model(
    folder: str,
    config: dict,
    seed: int,
    dtype: str = "bfloat16",
    std: float = 0.02,
    norm_init: str = "ones",
    optional_tensors: bool = True,
) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (the parsed
    JSON of any registered architecture).  Returns ``folder``."""
    from ..config.registry import resolve
    from ..parts.build import build_model

    _, spec = resolve(config)
    model = build_model(spec)
    decls = [d for d in model.tensor_decls() if optional_tensors or not d.optional]
    tensors: Dict[str, torch.Tensor] = dict(random_tensors(decls, seed, _DTYPES[dtype], std, norm_init))
    os.makedirs(folder, exist_ok=True)
    out = dict(config)
    out.setdefault("torch_dtype", dtype)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=2)
    write_safetensors(
        os.path.join(folder, "model.safetensors"),
        tensors,
        metadata={"format": "pt", "seed": seed, "std": std, "norm_init": norm_init},
    )
    return folder
