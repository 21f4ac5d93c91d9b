"""Builds and loads the host-side native library (``libferrox_b200_host.so``): the
bookkeeping of the cache manager, plain C++ without CUDA (``csrc/host/*.cpp``).  It is
compiled with the host compiler into ``ferrox_b200/_build`` at first use, in a second
or two, and needs no GPU, so the parts of the framework that run on the CPU (cache
manager, scheduler and their tests) work wherever a C++ compiler is.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import threading
from typing import Optional

from .lib import KernelBuildError, _log, build_dir

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_SRC = os.path.normpath(os.path.join(_HERE, "..", "csrc", "host"))
LIB_NAME = "libferrox_b200_host.so"
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None


def _compiler() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and (os.path.exists(cand) or shutil.which(cand)):
            return cand
    raise KernelBuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++)")


def build() -> str:
    out = build_dir()
    srcs = sorted(os.path.join(HOST_SRC, f) for f in os.listdir(HOST_SRC) if f.endswith(".cpp"))
    h = hashlib.sha256(" ".join(CXX_FLAGS).encode())
    for s in srcs:
        with open(s, "rb") as f:
            h.update(f.read())
    tag = h.hexdigest()[:16]
    lib = os.path.join(out, LIB_NAME)
    stamp = lib + ".tag"
    if os.path.exists(lib) and os.path.exists(stamp) and open(stamp).read().strip() == tag:
        return lib
    tmp = f"{lib}.{os.getpid()}.tmp"
    r = subprocess.run([_compiler(), *CXX_FLAGS, "-o", tmp, *srcs], capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"host library failed to compile:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(tag)
    _log(f"built {lib}")
    return lib


def load() -> ctypes.CDLL:
    global _lib
    with _lock:
        if _lib is None:
            L = ctypes.CDLL(build())
            I, P = ctypes.c_int, ctypes.c_void_p
            IP = ctypes.POINTER(ctypes.c_int)
            sig = {
                "fxh_cache_create": ([I, IP, IP, I, I, I, I], P),
                "fxh_cache_destroy": ([P], None),
                "fxh_open": ([P], I), "fxh_close": ([P, I], I),
                "fxh_pages_needed": ([P, I, I, IP], I),
                "fxh_reserve": ([P, I, I], I), "fxh_commit": ([P, I, I], I),
                "fxh_reserve_step": ([P, I, IP, IP, IP], I), "fxh_commit_step": ([P, I, IP, IP], I),
                "fxh_table": ([P, I], ctypes.POINTER(ctypes.c_int32)),
                "fxh_free_pages": ([P, I], I), "fxh_peak_pages": ([P, I], I), "fxh_free_slots": ([P], I),
                "fxh_seq_len": ([P, I], I), "fxh_first_page": ([P, I, I], I), "fxh_n_logical": ([P, I, I], I),
                "fxh_is_live": ([P, I], I), "fxh_take_dirty": ([P, I, IP, I], I), "fxh_check": ([P], I),
            }
            for name, (args, res) in sig.items():
                fn = getattr(L, name)
                fn.argtypes, fn.restype = args, res
            _lib = L
        return _lib
