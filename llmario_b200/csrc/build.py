"""Compile the CUDA sources of this folder for sm_100a and load the result.

Every ``.cu`` file is compiled by ``nvcc`` to an object, the objects are linked into one shared
library, and the library is opened with ``ctypes`` (the kernels have a plain C interface: raw
device pointers, sizes and a stream).  The library is kept beside the sources under ``_build/``
when that folder can be written, else under the system's temporary folder; it is rebuilt when a
source, a header or a flag changes.  Nothing here needs a GPU: nvcc cross-compiles.
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
from typing import Dict, List, Optional, Sequence

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=177"]

HOST_DIR = os.path.join(HERE, "host")
HOST_PREFIX = "libllmario_host_"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-Wall"]

_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of llmario_b200 cannot be compiled "
                     "(looked at $NVCC, PATH and /usr/local/cuda/bin/nvcc)")


def _sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest(files: Sequence[str], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(f.encode())
        with open(os.path.join(HERE, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    local = os.path.join(HERE, "_build")
    try:
        os.makedirs(local, exist_ok=True)
        probe = os.path.join(local, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return local
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llmario_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[llmario_b200 build] {msg}", file=sys.stderr, flush=True)


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{p.stdout}")


def build_library(verbose: bool = True, extra_flags: Sequence[str] = ()) -> str:
    """Compile what is out of date and return the path of the shared library."""
    flags = ARCH_FLAGS + BASE_FLAGS + list(extra_flags)
    srcs, hdrs = _sources(), _headers()
    if not srcs:
        raise BuildError(f"no .cu sources in {HERE}")
    out_dir = _build_dir()
    tag = _digest(srcs + hdrs, flags)
    lib = os.path.join(out_dir, f"libllmario_b200_{tag}.so")
    if os.path.isfile(lib):
        return lib
    nvcc = _nvcc()
    t0 = time.time()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {out_dir} "
             "(first call only)")
    hdr_tag = _digest(hdrs, flags)
    objs: List[str] = []
    jobs = []
    for s in srcs:
        otag = hashlib.sha256((hdr_tag + _digest([s], flags)).encode()).hexdigest()[:16]
        obj = os.path.join(out_dir, f"{s[:-3]}_{otag}.o")
        objs.append(obj)
        if not os.path.isfile(obj):
            jobs.append((s, obj))
    done = [0]

    def compile_one(job):
        s, obj = job
        tmp = obj + f".{os.getpid()}.tmp"
        _run([nvcc, *flags, "-I", HERE, "-c", os.path.join(HERE, s), "-o", tmp], f"compiling {s}")
        os.replace(tmp, obj)
        done[0] += 1
        if verbose:
            _say(f"  [{done[0]}/{len(jobs)}] {s}  ({time.time() - t0:.0f} s)")

    if jobs:
        workers = max(1, min(len(jobs), os.cpu_count() or 1))
        with ThreadPoolExecutor(workers) as pool:
            list(pool.map(compile_one, jobs))
    tmp = lib + f".{os.getpid()}.tmp"
    _run([nvcc, "-shared", *ARCH_FLAGS, "-o", tmp, *objs, "-lcudart_static", "-ldl", "-lrt",
          "-lpthread"], "linking")
    os.replace(tmp, lib)
    keep = {os.path.basename(lib)} | {os.path.basename(o) for o in objs}
    for f in os.listdir(out_dir):           # objects and libraries of older sources
        if f.endswith((".so", ".o")) and f not in keep and not f.startswith(HOST_PREFIX):
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass
    if verbose:
        _say(f"built {os.path.basename(lib)} in {time.time() - t0:.0f} s")
    return lib


def load_library(verbose: bool = True) -> ctypes.CDLL:
    """The shared library of kernels, compiled on first use.  Raises :class:`BuildError` when
    it cannot be built or opened: there is no other implementation to fall back to."""
    with _lock:
        if "lib" in _loaded:
            return _loaded["lib"]
        path = build_library(verbose)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot open {path}: {e}") from None
        _loaded["lib"] = lib
        _loaded["path"] = path  # type: ignore[assignment]
        return lib


def library_path() -> Optional[str]:
    return _loaded.get("path")  # type: ignore[return-value]


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"),
                 shutil.which("clang++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return cand
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++): the host "
                     "library of llmario_b200 cannot be compiled")


def build_host_library(verbose: bool = True) -> str:
    """Compile the host-side C++ sources (``host/*.cpp``: cache bookkeeping) into one shared
    library with the system's C++ compiler and return its path.  No CUDA toolkit is needed."""
    srcs = sorted(f for f in os.listdir(HOST_DIR) if f.endswith(".cpp"))
    if not srcs:
        raise BuildError(f"no .cpp sources in {HOST_DIR}")
    h = hashlib.sha256()
    for f in srcs + sorted(f for f in os.listdir(HOST_DIR) if f.endswith((".h", ".hpp"))):
        h.update(f.encode())
        with open(os.path.join(HOST_DIR, f), "rb") as fh:
            h.update(fh.read())
    h.update(" ".join(HOST_FLAGS).encode())
    out_dir = _build_dir()
    lib = os.path.join(out_dir, f"{HOST_PREFIX}{h.hexdigest()[:16]}.so")
    if os.path.isfile(lib):
        return lib
    t0 = time.time()
    tmp = lib + f".{os.getpid()}.tmp"
    _run([_cxx(), *HOST_FLAGS, "-o", tmp, *[os.path.join(HOST_DIR, f) for f in srcs]],
         "compiling the host library")
    os.replace(tmp, lib)
    for f in os.listdir(out_dir):
        if f.startswith(HOST_PREFIX) and f.endswith(".so") and f != os.path.basename(lib):
            try:
                os.remove(os.path.join(out_dir, f))
            except OSError:
                pass
    if verbose:
        _say(f"built {os.path.basename(lib)} in {time.time() - t0:.0f} s")
    return lib


def load_host_library() -> ctypes.CDLL:
    with _lock:
        path = build_host_library()
        if path not in _loaded:
            _loaded[path] = ctypes.CDLL(path)
        return _loaded[path]
