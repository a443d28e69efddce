"""Compiles the CUDA sources for sm_100a with nvcc and loads them through ctypes.

Each ``csrc/<module>.cu`` becomes one shared library that is built on first use
(or all at once by :func:`build_all`) and cached beside the sources under a name
that carries a hash of the source, the shared header and the flags, so an edited
kernel is rebuilt and a stale library is never loaded.  There is no fallback: if
a library cannot be built or loaded, the operation that needs it raises.
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
from typing import Dict, Iterable, List

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


class KernelBuildError(RuntimeError):
    pass


_DIR_LOCK = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("SKYLA_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found: the CUDA kernels cannot be compiled "
                           "(set SKYLA_NVCC or put nvcc on PATH)")


_BUILD_DIR = None


def _build_dir() -> str:
    global _BUILD_DIR
    if _BUILD_DIR is None:
        with _DIR_LOCK:
            if _BUILD_DIR is None:
                _BUILD_DIR = _find_build_dir()
    return _BUILD_DIR


def _find_build_dir() -> str:
    cands = [os.environ.get("SKYLA_BUILD_DIR"), os.path.join(CSRC, "_build"),
             os.path.join(tempfile.gettempdir(), f"skyla_kernel_b200_build_{os.getuid()}")]
    for d in cands:
        if not d:
            continue
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
            return d
        except OSError:
            continue
    raise KernelBuildError("no writable folder for the compiled kernels (set SKYLA_BUILD_DIR)")


def modules() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(module: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in [os.path.join(CSRC, module + ".cu")] + _headers():
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def library_path(module: str, build_dir: str = None) -> str:
    return os.path.join(build_dir or _build_dir(), f"skyla_{module}_{_digest(module)}.so")


def _say(msg: str) -> None:
    print(f"[skyla] {msg}", file=sys.stderr, flush=True)


def compile_module(module: str, verbose: bool = True) -> str:
    """Build one library if its cached copy is absent; returns its path."""
    src = os.path.join(CSRC, module + ".cu")
    if not os.path.isfile(src):
        raise KernelBuildError(f"no kernel source {src}")
    bdir = _build_dir()
    out = library_path(module, bdir)
    if os.path.isfile(out):
        return out
    tmp = f"{out}.{os.getpid()}.{threading.get_ident()}.tmp"
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, src]
    if verbose:
        _say(f"compiling {module}.cu for sm_100a ...")
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=bdir)
    while True:
        try:
            log, _ = proc.communicate(timeout=15)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                _say(f"  still compiling {module}.cu ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {module}.cu:\n{log}")
    os.replace(tmp, out)
    # drop libraries of older versions of this source
    prefix = f"skyla_{module}_"
    for f in os.listdir(bdir):
        if f.startswith(prefix) and f.endswith(".so") and os.path.join(bdir, f) != out:
            try:
                os.remove(os.path.join(bdir, f))
            except OSError:
                pass
    if verbose:
        _say(f"  {module}.cu done in {time.time() - t0:.1f} s")
    return out


def build_all(names: Iterable[str] = None, jobs: int = None, verbose: bool = True) -> Dict[str, str]:
    """Compile the named modules (default: all) in parallel."""
    names = list(names) if names is not None else modules()
    todo = [n for n in names if not os.path.isfile(library_path(n))]
    if todo and verbose:
        _say(f"{len(todo)} CUDA source file(s) to compile: {', '.join(todo)}")
    jobs = jobs or min(len(todo) or 1, os.cpu_count() or 4, 8)
    with ThreadPoolExecutor(max_workers=jobs) as ex:
        list(ex.map(lambda n: compile_module(n, verbose), todo))
    return {n: library_path(n) for n in names}


_LIBS: Dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


def load(module: str) -> ctypes.CDLL:
    """The loaded library of a module; compiles it first if need be."""
    lib = _LIBS.get(module)
    if lib is not None:
        return lib
    with _LOCK:
        lib = _LIBS.get(module)
        if lib is None:
            path = compile_module(module)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from None
            lib.skyla_error_message.restype = ctypes.c_char_p
            _LIBS[module] = lib
    return lib
