"""Compiling the CUDA sources of this folder for sm_100a with nvcc and loading the result
with ctypes.

A module is a set of ``.cu`` files plus preprocessor definitions (the tensor-core attention
kernels are compiled for one head size at a time, so a model compiles what it needs and no
more).  Objects and libraries are kept in ``_build/`` beside the sources, named by a hash of
the sources, headers and flags; a library that is already there is loaded without nvcc.  If
that folder cannot be written, a per-user folder under the system's temporary directory is
used.  Nothing here falls back to another implementation: without a library, and without
nvcc to make one, loading fails with an error that says so.
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
from typing import Dict, Iterable, Tuple

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

_loaded: Dict[Tuple[str, Tuple[Tuple[str, str], ...]], ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[pico_engine build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("PICO_ENGINE_NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("the CUDA kernels are not built and nvcc was not found (looked at PICO_ENGINE_NVCC, PATH, "
                     "CUDA_HOME and /usr/local/cuda); this library has no other implementation to fall back on")


def build_dir() -> str:
    d = os.path.join(HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"pico_engine_b200-build-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _headers() -> list[str]:
    return sorted(os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h")))


def _digest(paths: Iterable[str], flags: Iterable[str]) -> str:
    h = hashlib.sha256()
    for p in paths:
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update("\0".join(flags).encode())
    return h.hexdigest()[:16]


def _run(cmd: list[str], what: str) -> None:
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=HERE)
    while True:
        try:
            out, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"... still {what} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{out}")


def library_path(name: str, sources: Iterable[str], defines: Dict[str, str] | None = None) -> str:
    """Path of the library of module ``name``, compiling it first if it is not there yet."""
    defines = dict(defines or {})
    srcs = [os.path.join(HERE, s) for s in sources]
    dflags = [f"-D{k}={v}" for k, v in sorted(defines.items())]
    flags = ARCH_FLAGS + NVCC_FLAGS + dflags
    tag = _digest(srcs + _headers(), flags)
    out_dir = build_dir()
    lib = os.path.join(out_dir, f"libpico_{name}.{tag}.so")
    if os.path.isfile(lib):
        return lib
    nvcc = find_nvcc()
    _say(f"compiling module {name!r} ({len(srcs)} file(s){', ' + ' '.join(dflags) if dflags else ''}) for sm_100a")

    def compile_one(src: str) -> str:
        obj = os.path.join(out_dir, f"{name}.{os.path.basename(src)}.{tag}.{os.getpid()}.o")
        _run([nvcc] + flags + ["-c", src, "-o", obj], f"compiling {os.path.basename(src)}")
        _say(f"compiled {os.path.basename(src)}")
        return obj

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = f"{lib}.{os.getpid()}.tmp"
    _run([nvcc] + ARCH_FLAGS + ["-shared", "-o", tmp] + objs, f"linking {os.path.basename(lib)}")
    os.replace(tmp, lib)
    for old in os.listdir(out_dir):                        # libraries of earlier versions of these sources
        if old.startswith(f"libpico_{name}.") and old.endswith(".so") and os.path.join(out_dir, old) != lib:
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    for o in objs:
        try:
            os.remove(o)
        except OSError:
            pass
    _say(f"built {os.path.basename(lib)}")
    return lib


def load(name: str, sources: Iterable[str], defines: Dict[str, str] | None = None) -> ctypes.CDLL:
    key = (name, tuple(sorted((defines or {}).items())))
    with _lock:
        if key not in _loaded:
            _loaded[key] = ctypes.CDLL(library_path(name, sources, defines))
        return _loaded[key]
