"""Random-weights mode: a model from a configuration and a seed, as a folder or straight into an engine.

One rule, the same on the device and on the CPU, bit for bit: a tensor's key is a hash of (seed, tensor name); its
element pair j takes two 64-bit values of a counter-based generator, ``mix(key + (2j+1) G)`` and ``mix(key + (2j+2) G)``,
turns them into uniforms in (0, 1) and those into two standard normals by the Box-Muller transform; the value is
``mean + std * z`` rounded once to 32 bits (and once more, to nearest even, for 16-bit storage).  The logarithm, cosine
and sine are series of additions, multiplications and divisions in 64-bit floating point, each rounded by itself, so
that :func:`normal_cpu` here and ``fx_random_normal`` (csrc/random_init.cu) give the same bits; a tensor does not depend
on which other tensors exist, on the order in which they are made or on where they are drawn.  A model of any size can
therefore be drawn on the device for the engine and handed, copied to the host, to a plain implementation.

Matrices, biases and gate vectors are N(0, std); norm weights are 1 (``norm_init="ones"``), 1 + N(0, std)
(``"around_one"``) or N(0, std) like everything else (``"normal"``).  The reference's counterpart is
``Decoder::new_random_small`` (crates/ferrox-models/src/decoder.rs:373-388,397-514: one xorshift64* stream from seed
42 for every tensor, uniform +-0.05, norm weights 1, no bias, no shared gate); unlike it, this mode fills biases and
the shared expert's gate as well, so that they are exercised.
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

_GOLDEN = 0x9E3779B97F4A7C15
_M1, _M2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_CHUNK = 1 << 20  # element pairs per pass of the CPU draw (temporaries stay in cache)


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's stream."""
    h = hashlib.blake2b(f"{seed}:{name}".encode("utf-8"), digest_size=8).digest()
    return int.from_bytes(h, "little")


def _i64(v: int) -> int:
    """A 64-bit pattern as the signed integer torch holds it in."""
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def _shr(x: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of 64-bit patterns held as int64."""
    return (x >> n) & ((1 << (64 - n)) - 1)


def _mix64(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _shr(z, 30)) * _i64(_M1)
    z = (z ^ _shr(z, 27)) * _i64(_M2)
    return z ^ _shr(z, 31)


def _unit_open(x: torch.Tensor) -> torch.Tensor:
    return (_shr(x, 12).to(torch.float64) + 0.5) * 2.220446049250313e-16


def _ln(u: torch.Tensor) -> torch.Tensor:
    m, e = torch.frexp(u)
    low = m < 0.7071067811865476
    m = torch.where(low, m * 2.0, m)
    e = torch.where(low, e - 1, e)
    s = (m + -1.0) / (m + 1.0)
    s2 = s * s
    p = torch.full_like(s, 1.0 / 21.0)
    for k in range(9, -1, -1):
        p = p * s2 + (1.0 / float(2 * k + 1))
    return (2.0 * s) * p + e.to(torch.float64) * 0.6931471805599453


def _cos_sin_turn(u: torch.Tensor):
    t = u * 4.0
    kf = torch.floor(t)
    k = kf.to(torch.int64) & 3
    f = t + -kf
    fold = f > 0.5
    f = torch.where(fold, 1.0 + -f, f)
    a = f * 1.5707963267948966
    a2 = a * a
    pc = torch.zeros_like(a)
    ps = torch.zeros_like(a)
    for n in range(10, 0, -1):
        pc = (1.0 + -pc) * (a2 / float((2 * n - 1) * (2 * n)))
        ps = (1.0 + -ps) * (a2 / float((2 * n) * (2 * n + 1)))
    c = 1.0 + -pc
    s = a * (1.0 + -ps)
    c, s = torch.where(fold, s, c), torch.where(fold, c, s)
    c_out = torch.where(k == 0, c, torch.where(k == 1, -s, torch.where(k == 2, -c, s)))
    s_out = torch.where(k == 0, s, torch.where(k == 1, c, torch.where(k == 2, -s, -c)))
    return c_out, s_out


def normal_cpu(key: int, n: int, mean: float = 0.0, std: float = 1.0) -> torch.Tensor:
    """The first ``n`` values of the stream of ``key`` as float32 on the CPU: the host's statement of the rule."""
    out = torch.empty(2 * ((n + 1) // 2), dtype=torch.float32)
    n_pairs = (n + 1) // 2
    for a in range(0, n_pairs, _CHUNK):
        b = min(n_pairs, a + _CHUNK)
        j = torch.arange(a, b, dtype=torch.int64)
        x1 = _mix64((2 * j + 1) * _i64(_GOLDEN) + _i64(key))
        x2 = _mix64((2 * j + 2) * _i64(_GOLDEN) + _i64(key))
        r = torch.sqrt(-2.0 * _ln(_unit_open(x1)))
        c, s = _cos_sin_turn(_unit_open(x2))
        pair = out[2 * a:2 * b].view(-1, 2)
        pair[:, 0] = (mean + std * (r * c)).to(torch.float32)
        pair[:, 1] = (mean + std * (r * s)).to(torch.float32)
    return out[:n]


def normal(key: int, shape, dtype, mean: float, std: float, device="cpu") -> torch.Tensor:
    """N(mean, std) of the stream of ``key`` in ``dtype`` (float32 or bfloat16), drawn where ``device`` says."""
    device = torch.device(device)
    n = 1
    for s in shape:
        n *= int(s)
    if device.type == "cuda":
        from ..kernels import ops

        kdt = dtype if dtype in (torch.float32, torch.bfloat16) else torch.float32
        t = torch.empty(tuple(shape), dtype=kdt, device=device)
        ops.random_normal(t, key, mean, std)
        return t.to(dtype)
    return normal_cpu(key, n, mean, std).reshape(tuple(shape)).to(dtype)


def random_tensor(decl: TensorDecl, seed: int, dtype, std: float, norm_init: str, device="cpu") -> torch.Tensor:
    if decl.integer:
        return torch.zeros(decl.shape, dtype=torch.int32, device=device)
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=dtype, device=device)
    if decl.init == "ones" and norm_init == "ones":
        return torch.ones(decl.shape, dtype=dtype, device=device)
    mean = 0.0
    if decl.init == "ones" and norm_init == "around_one":
        mean = 1.0
    elif decl.init == "ones" and norm_init != "normal":
        raise ValueError(f"norm_init={norm_init!r}: expected ones, around_one or normal")
    return normal(tensor_key(seed, decl.name), decl.shape, dtype, mean, std, device)


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
    device="cpu",
) -> str:
    """Write ``config.json`` and ``model.safetensors`` for ``config`` (the parsed
    JSON of any registered architecture).  ``device``: where the values are drawn
    (the same values either way).  Returns ``folder``."""
    from ..config.registry import resolve
    from ..parts.build import build_model

    _, spec = resolve(config)
    model = build_model(spec)
    decls = [d for d in model.tensor_decls() if optional_tensors or not d.optional]
    tensors: Dict[str, torch.Tensor] = {
        n: t.cpu() for n, t in random_tensors(decls, seed, _DTYPES[dtype], std, norm_init, device)}
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
