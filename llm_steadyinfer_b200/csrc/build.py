"""Builds the CUDA sources of this folder for sm_100a and loads them with ctypes.

Every ``<name>.cu`` becomes one shared library ``_build/<name>-<digest>.so`` next to the
sources (or, when that folder cannot be written, under the system temporary folder).
A library is compiled the first time one of its kernels is needed, so a run compiles
only what its model uses; while nvcc works a line is printed every few seconds.
There is no fallback: a missing compiler or a failed build raises.
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
from typing import Dict, List, Optional

CSRC_DIR = os.path.dirname(os.path.abspath(__file__))
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

_libs: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def kernel_sources() -> List[str]:
    return sorted(f[:-3] for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of this package cannot be built")


def _included_sources(name: str) -> List[str]:
    """Other .cu files that <name>.cu pulls in with #include "x.cu"."""
    out = []
    with open(os.path.join(CSRC_DIR, name + ".cu"), "r", encoding="utf-8") as f:
        for line in f:
            line = line.strip()
            if line.startswith("#include") and line.endswith('.cu"'):
                out.append(line.split('"')[1])
    return out


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(os.environ.get("SI_NVCC_EXTRA", "").encode())      # other flags, another library
    own = [name + ".cu"] + _included_sources(name)
    for fn in sorted(os.listdir(CSRC_DIR)):
        if fn in own or fn.endswith(".cuh") or fn.endswith(".h"):
            with open(os.path.join(CSRC_DIR, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    return h.hexdigest()[:16]


_build_dir_cached: Optional[str] = None


def _build_dir() -> str:
    global _build_dir_cached
    if _build_dir_cached is None:
        _build_dir_cached = _find_build_dir()
    return _build_dir_cached


def _find_build_dir() -> str:
    d = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.unlink(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llm_steadyinfer_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"{name}-{_digest(name)}.so")


def _compile(name: str, out: str, verbose: bool) -> None:
    src = os.path.join(CSRC_DIR, name + ".cu")
    if not os.path.isfile(src):
        raise BuildError(f"no CUDA source {src}")
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", CSRC_DIR, "-o", tmp, src]
    extra = os.environ.get("SI_NVCC_EXTRA")
    if extra:
        cmd[1:1] = extra.split()
    t0 = time.time()
    if verbose:
        print(f"[build] compiling {name}.cu for sm_100a ...", file=sys.stderr, flush=True)
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    stop = threading.Event()

    def tick():
        while not stop.wait(10.0):
            print(f"[build] still compiling {name}.cu ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)

    th = threading.Thread(target=tick, daemon=True)
    th.start()
    try:
        log, _ = proc.communicate()
    finally:
        stop.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise BuildError(f"nvcc failed on {name}.cu (exit {proc.returncode}):\n"
                         f"{' '.join(cmd)}\n{log.decode(errors='replace')}")
    os.replace(tmp, out)
    for old in os.listdir(os.path.dirname(out)):             # libraries of earlier source versions
        if old.startswith(name + "-") and old.endswith(".so") and old != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), old))
            except OSError:
                pass
    if verbose:
        print(f"[build] {name}.cu done in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def load(name: str, verbose: bool = True) -> ctypes.CDLL:
    """Return the loaded library of ``<name>.cu``, compiling it first when needed."""
    lib = _libs.get(name)
    if lib is not None:
        return lib
    with _lock:
        lib = _libs.get(name)
        if lib is not None:
            return lib
        path = library_path(name)
        if not os.path.isfile(path):
            _compile(name, path, verbose)
        try:
            lib = ctypes.CDLL(path)
        except OSError as e:
            raise BuildError(f"cannot load {path}: {e}") from None
        _libs[name] = lib
        return lib


def prebuild(names, verbose: bool = True) -> None:
    """Compile those of ``names`` that have no up-to-date library, several at a time: what a model needs
    is known when it is built, and its first step need not wait for one compiler run after the other."""
    build_all(verbose, names=sorted(set(names)))


def build_all(verbose: bool = True, jobs: Optional[int] = None, names: Optional[List[str]] = None) -> List[str]:
    """Compile every source (or every one of ``names``) that has no up-to-date library; returns the
    library paths."""
    names = kernel_sources() if names is None else list(names)
    todo = [n for n in names if n not in _libs and not os.path.isfile(library_path(n))]
    errors: List[str] = []

    _build_dir()

    def work(n):
        try:
            _compile(n, library_path(n), verbose)
        except Exception as e:      # a thread must not fail silently
            errors.append(f"{n}.cu: {e}")

    jobs = jobs or min(len(todo), os.cpu_count() or 1, 8) or 1
    pending = list(todo)
    threads: List[threading.Thread] = []
    while pending or threads:
        while pending and len(threads) < jobs:
            t = threading.Thread(target=work, args=(pending.pop(0),))
            t.start()
            threads.append(t)
        threads[0].join()
        threads.pop(0)
    if errors:
        raise BuildError("\n\n".join(errors))
    return [library_path(n) for n in names]
