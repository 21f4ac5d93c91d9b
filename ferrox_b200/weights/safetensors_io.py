"""Reader and writer for the safetensors container, by tensor name.

Layout: 8 bytes little-endian header length N, N bytes of JSON
({name: {"dtype", "shape", "data_offsets": [begin, end]}}, optional
``__metadata__``), then the data.  The checks are those of the reference's parser
(crates/ferrox-safetensors/src/lib.rs:168-243): the header must fit the file and
stay under 100 MB, be UTF-8 JSON, every tensor's byte count must equal
product(shape) * sizeof(dtype), and the tensors, sorted by offset, must tile the
data section exactly, without gap or overlap.  A folder may hold one
``model.safetensors`` or shards listed in ``model.safetensors.index.json``
(``weight_map``; reference lib.rs:290-379).

Tensors come back as torch tensors that view a memory map of the file (bfloat16
through a 16-bit integer view, since numpy has no such type).
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterable, Tuple

import numpy as np
import torch

MAX_HEADER_BYTES = 100 * 1024 * 1024

_DTYPES = {
    "F32": (torch.float32, 4),
    "BF16": (torch.bfloat16, 2),
    "F16": (torch.float16, 2),
    "F64": (torch.float64, 8),
    "I64": (torch.int64, 8),
    "I32": (torch.int32, 4),
    "I16": (torch.int16, 2),
    "I8": (torch.int8, 1),
    "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    """The file is not a well-formed safetensors container."""


class SafetensorsFile:
    """One memory-mapped safetensors file."""

    def __init__(self, path: str):
        self.path = path
        try:
            self._fh = open(path, "rb")
        except OSError as e:
            raise SafetensorsError(f"{path}: cannot open ({e.strerror})") from None
        size = os.fstat(self._fh.fileno()).st_size
        if size < 8:
            raise SafetensorsError(f"{path}: {size} bytes is too short for a header length")
        (n,) = struct.unpack("<Q", self._fh.read(8))
        if n > MAX_HEADER_BYTES:
            raise SafetensorsError(f"{path}: header of {n} bytes exceeds the limit of {MAX_HEADER_BYTES}")
        if 8 + n > size:
            raise SafetensorsError(f"{path}: header of {n} bytes does not fit a file of {size} bytes")
        raw = self._fh.read(n)
        try:
            header = json.loads(raw.decode("utf-8"))
        except UnicodeDecodeError:
            raise SafetensorsError(f"{path}: header is not UTF-8") from None
        except json.JSONDecodeError as e:
            raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header must be a JSON object")
        self.metadata = header.pop("__metadata__", None) or {}
        self._data_start = 8 + n
        data_len = size - self._data_start
        self.entries: Dict[str, Tuple[torch.dtype, Tuple[int, ...], int, int]] = {}
        spans = []
        for name, info in header.items():
            try:
                dt, shape, (begin, end) = info["dtype"], tuple(int(s) for s in info["shape"]), info["data_offsets"]
            except (KeyError, TypeError, ValueError):
                raise SafetensorsError(f"{path}: malformed entry for tensor {name!r}") from None
            if dt not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name!r} has unsupported dtype {dt!r}")
            tdt, esz = _DTYPES[dt]
            count = 1
            for s in shape:
                if s < 0:
                    raise SafetensorsError(f"{path}: tensor {name!r} has a negative extent")
                count *= s
            if end - begin != count * esz or begin < 0:
                raise SafetensorsError(
                    f"{path}: tensor {name!r} spans {end - begin} bytes but {dt}{list(shape)} needs {count * esz}"
                )
            self.entries[name] = (tdt, shape, begin, end)
            spans.append((begin, end, name))
        spans.sort()
        cursor = 0
        for begin, end, name in spans:
            if begin != cursor:
                what = "overlaps the one before it" if begin < cursor else "leaves a gap before it"
                raise SafetensorsError(f"{path}: tensor {name!r} at offset {begin} {what}")
            cursor = end
        if cursor != data_len:
            raise SafetensorsError(f"{path}: tensors cover {cursor} bytes, the data section has {data_len}")
        self._mm = mmap.mmap(self._fh.fileno(), 0, access=mmap.ACCESS_READ) if size else None

    def names(self) -> Iterable[str]:
        return self.entries.keys()

    def info(self, name: str) -> Tuple[torch.dtype, Tuple[int, ...]]:
        dt, shape, _, _ = self.entries[name]
        return dt, shape

    def tensor(self, name: str) -> torch.Tensor:
        """A read-only view of the mapped file; copy (``.to(device)``, ``.clone()``)
        before the file object goes away."""
        tdt, shape, begin, end = self.entries[name]
        if end == begin:
            return torch.empty(shape, dtype=tdt)
        buf = np.frombuffer(self._mm, dtype=np.uint8, count=end - begin, offset=self._data_start + begin)
        import warnings

        with warnings.catch_warnings():
            warnings.simplefilter("ignore")  # torch warns that the array is read-only
            t = torch.from_numpy(buf)
        return t.view(tdt).reshape(shape)

    def close(self) -> None:
        # numpy views keep the map alive; dropping our handles is enough.
        self._mm = None
        self._fh.close()


class ModelFiles:
    """All safetensors of a model folder behind one name -> tensor lookup."""

    def __init__(self, folder: str):
        self.folder = folder
        index = os.path.join(folder, "model.safetensors.index.json")
        single = os.path.join(folder, "model.safetensors")
        self._files: Dict[str, SafetensorsFile] = {}
        self._where: Dict[str, str] = {}
        if os.path.exists(index):
            with open(index, "r", encoding="utf-8") as f:
                try:
                    weight_map = json.load(f)["weight_map"]
                except (json.JSONDecodeError, KeyError, TypeError):
                    raise SafetensorsError(f"{index}: no usable 'weight_map'") from None
            for name, shard in weight_map.items():
                if shard not in self._files:
                    self._files[shard] = SafetensorsFile(os.path.join(folder, shard))
                if name not in self._files[shard].entries:
                    raise SafetensorsError(f"{index}: maps {name!r} to {shard}, which does not hold it")
                self._where[name] = shard
        elif os.path.exists(single):
            self._files["model.safetensors"] = SafetensorsFile(single)
            for name in self._files["model.safetensors"].names():
                self._where[name] = "model.safetensors"
        else:
            raise SafetensorsError(f"{folder}: neither model.safetensors nor model.safetensors.index.json found")

    def names(self):
        return self._where.keys()

    def info(self, name):
        return self._files[self._where[name]].info(name)

    def tensor(self, name) -> torch.Tensor:
        return self._files[self._where[name]].tensor(name)

    def close(self):
        for f in self._files.values():
            f.close()


def write_safetensors(path: str, tensors: Dict[str, torch.Tensor], metadata: Dict[str, str] | None = None) -> None:
    """Write ``tensors`` (CPU, any supported dtype) in the order given."""
    header = {}
    if metadata:
        header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    offset = 0
    blobs = []
    for name, t in tensors.items():
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name!r}: dtype {t.dtype} cannot be stored")
        t = t.detach().contiguous().cpu()
        nbytes = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + nbytes]}
        offset += nbytes
        blobs.append(t)
    raw = json.dumps(header, separators=(",", ":")).encode("utf-8")
    raw += b" " * (-len(raw) % 8)  # keep the data section 8-byte aligned
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(raw)))
        f.write(raw)
        for t in blobs:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes())
