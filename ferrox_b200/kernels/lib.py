"""Builds and loads the kernel library (``libferrox_b200.so``).

The library is plain CUDA behind a C ABI (``csrc/api.h``): no Python or torch
headers, so a source file compiles in seconds with ``nvcc -gencode
arch=compute_100a,code=sm_100a``.  It is built in-tree under ``ferrox_b200/_build``
at first use (or by ``__graft_entry__.build()``), object by object, and rebuilt
when a source changes; while compiling, a line is printed to stderr every few
seconds.  If that folder cannot be written, a per-user folder under the system's
temporary directory is used.  There is no fallback: when the library cannot be
built or loaded, importing the kernels fails with the compiler's message.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.normpath(os.path.join(_HERE, "..", "csrc"))
LIB_NAME = "libferrox_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[ferrox_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("FERROX_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $FERROX_NVCC, $PATH and /usr/local/cuda/bin/nvcc)")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".h", ".cuh")))


def _digest(paths: List[str], extra: str = "") -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.encode())
        with open(os.path.join(CSRC, p), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def build_dir() -> str:
    d = os.path.normpath(os.path.join(_HERE, "..", "_build"))
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"ferrox_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def build(verbose: bool = True) -> str:
    """Compile what is out of date and link; returns the library's path."""
    out = build_dir()
    nvcc = find_nvcc()
    hdr = _digest(_headers(), " ".join(NVCC_FLAGS))
    jobs = []
    objects = []
    for src in sources():
        tag = _digest([src], hdr)
        obj = os.path.join(out, f"{src[:-3]}.{tag}.o")
        objects.append(obj)
        if not os.path.exists(obj):
            jobs.append((src, obj))
    lib_tag = hashlib.sha256(" ".join(os.path.basename(o) for o in objects).encode()).hexdigest()[:16]
    lib = os.path.join(out, LIB_NAME)
    stamp = os.path.join(out, LIB_NAME + ".tag")
    current = None
    if os.path.exists(lib) and os.path.exists(stamp):
        with open(stamp) as f:
            current = f.read().strip()
    if not jobs and current == lib_tag:
        return lib

    if verbose:
        _log(f"compiling {len(jobs)} of {len(objects)} CUDA sources for sm_100a into {out}")
    t0 = time.time()

    def compile_one(job):
        src, obj = job
        tmp = f"{obj}.{os.getpid()}.tmp"
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, src), "-o", tmp]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, obj)
        return src

    done = threading.Event()

    def ticker():
        while not done.wait(5.0):
            _log(f"still compiling ... {time.time() - t0:.0f} s")

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
            for src in pool.map(compile_one, jobs):
                if verbose:
                    _log(f"compiled {src} ({time.time() - t0:.0f} s)")
        # stale objects of earlier source versions
        keep = {os.path.basename(o) for o in objects}
        for f in os.listdir(out):
            if f.endswith(".o") and f not in keep:
                try:
                    os.remove(os.path.join(out, f))
                except OSError:
                    pass
        tmp = f"{lib}.{os.getpid()}.tmp"
        r = subprocess.run([nvcc, "-shared", "-o", tmp, *objects], capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(lib_tag)
    finally:
        done.set()
    if verbose:
        _log(f"built {lib} in {time.time() - t0:.0f} s")
    return lib


def load() -> ctypes.CDLL:
    """The loaded library (built first if need be)."""
    global _lib
    with _lock:
        if _lib is None:
            # torch brings the CUDA runtime the library links against
            import torch  # noqa: F401

            path = build()
            try:
                _lib = ctypes.CDLL(path, mode=ctypes.RTLD_GLOBAL)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
        return _lib
