"""Compiling the CUDA sources of this package for sm_100a, and loading them.

Each ``.cu`` file beside this one becomes one shared library of plain
``extern "C"`` functions, built with ``nvcc`` alone (no torch headers, so a file
compiles in seconds) and loaded with ``ctypes``.  A library is built the first
time something in it is called, so a run compiles what its model needs and
nothing else; ``build_all`` compiles everything (the "does it build" check).

Libraries go to ``synaptix_b200/_build/`` inside the source tree, named after a
hash of the source text and the flags, so an edited source is rebuilt and a
stale library is never loaded.  If that folder cannot be written (a read-only
checkout), a per-user folder under the system's temporary directory is used.
While ``nvcc`` runs, a line goes to standard error every few seconds.

The reference compiles its kernels at run time through NVRTC with a disk cache
(crates/synaptix-kernels-cuda/src/kernels/compile.rs:14-184); this is the
ahead-of-time counterpart for one architecture (sm_100a), with no fallback.
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
PKG_DIR = os.path.dirname(CSRC_DIR)

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# library name -> (source file, extra flags)
LIBRARIES: Dict[str, tuple] = {
    "generic": ("generic.cu", []),
    "sampling": ("sampling.cu", []),
    "decode": ("decode.cu", []),
    "attention": ("attention.cu", []),
    "attn_decode": ("attn_decode.cu", []),
    "attn_tc": ("attn_tc.cu", []),
    "gemm_tc": ("gemm_tc.cu", []),
    "gemm_ws": ("gemm_ws.cu", []),
}


# host-only C++ (the kernels' plain counterparts for the CPU): library name -> source file, compiled with the C++ compiler
HOST_LIBRARIES: Dict[str, str] = {"reference": "reference.cpp"}
HOST_FLAGS = ["-O2", "-std=c++17", "-shared", "-fPIC"]


class KernelsUnavailable(RuntimeError):
    """The CUDA kernels cannot be built or loaded; nothing falls back to anything else."""


def find_nvcc() -> str:
    for cand in (shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelsUnavailable("nvcc was not found (looked at PATH, $CUDA_HOME/bin, "
                             "/usr/local/cuda/bin); the kernels of this package must be compiled for sm_100a")


_BUILD_DIR: Optional[str] = None
_BUILD_DIR_LOCK = threading.Lock()


def _build_dir() -> str:
    global _BUILD_DIR
    with _BUILD_DIR_LOCK:
        if _BUILD_DIR is None:
            d = os.path.join(PKG_DIR, "_build")
            try:
                os.makedirs(d, exist_ok=True)
                fd, probe = tempfile.mkstemp(prefix=".w", dir=d)
                os.close(fd)
                os.remove(probe)
            except OSError:
                uid = os.getuid() if hasattr(os, "getuid") else 0
                d = os.path.join(tempfile.gettempdir(), f"synaptix_b200-build-{uid}")
                os.makedirs(d, exist_ok=True)
            _BUILD_DIR = d
        return _BUILD_DIR


def _source_hash(name: str) -> str:
    src, extra = LIBRARIES[name]
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS + list(extra)).encode())
    for fn in sorted(os.listdir(CSRC_DIR)):
        if fn == src or fn.endswith((".cuh", ".h")):
            with open(os.path.join(CSRC_DIR, fn), "rb") as f:
                h.update(fn.encode())
                h.update(f.read())
    return h.hexdigest()[:12]


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libsx_{name}-{_source_hash(name)}.so")


def _say(msg: str) -> None:
    print(f"[synaptix_b200] {msg}", file=sys.stderr, flush=True)


def build_library(name: str, verbose: bool = True, ptxas_info: bool = False) -> str:
    """Compile one library if its up-to-date file is not there yet; return its path."""
    out = library_path(name)
    if os.path.isfile(out) and not ptxas_info:
        return out
    src, extra = LIBRARIES[name]
    nvcc = find_nvcc()
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_info else []) + \
          ["-I", CSRC_DIR, "-o", tmp, os.path.join(CSRC_DIR, src)] + list(extra)
    if verbose:
        _say(f"compiling csrc/{src} for sm_100a ...")
    t0 = time.time()
    stop = threading.Event()

    def heartbeat():
        while not stop.wait(10.0):
            _say(f"  still compiling csrc/{src} ({time.time() - t0:.0f} s)")

    th = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        th.start()
    try:
        # nvcc needs a writable temporary directory and no HOME
        env = dict(os.environ)
        env.setdefault("TMPDIR", tempfile.gettempdir())
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    finally:
        stop.set()
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelsUnavailable(f"nvcc failed on csrc/{src}:\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    # drop older builds of the same library
    prefix = f"libsx_{name}-"
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(prefix) and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    if verbose:
        _say(f"  built {os.path.basename(out)} in {time.time() - t0:.1f} s")
    if ptxas_info:
        print(proc.stdout)
    return out


def build_all(verbose: bool = True) -> List[str]:
    """Compile every library of the package (in parallel), the host-only ones after them."""
    names = [n for n, (src, _) in LIBRARIES.items() if os.path.isfile(os.path.join(CSRC_DIR, src))]
    out: Dict[str, str] = {}
    errs: List[BaseException] = []

    def one(n):
        try:
            out[n] = build_library(n, verbose=verbose)
        except BaseException as e:  # noqa: BLE001 - reported below
            errs.append(e)

    threads = [threading.Thread(target=one, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errs:
        raise errs[0]
    return [out[n] for n in names] + [build_host_library(n, verbose=verbose) for n in HOST_LIBRARIES]


def build_host_library(name: str, verbose: bool = True) -> str:
    """Compile a host-only C++ library (no CUDA in it, no GPU needed to run it); return its path."""
    src = HOST_LIBRARIES[name]
    with open(os.path.join(CSRC_DIR, src), "rb") as f:
        digest = hashlib.sha256(" ".join(HOST_FLAGS).encode() + f.read()).hexdigest()[:12]
    out = os.path.join(_build_dir(), f"libsx_{name}-{digest}.so")
    if os.path.isfile(out):
        return out
    cxx = shutil.which("g++") or shutil.which("c++") or shutil.which("clang++")
    if cxx is None:
        raise KernelsUnavailable(f"no C++ compiler (g++, c++, clang++) was found to build csrc/{src}")
    tmp = f"{out}.{os.getpid()}.tmp"
    cmd = [cxx] + HOST_FLAGS + ["-o", tmp, os.path.join(CSRC_DIR, src)]
    if verbose:
        _say(f"compiling csrc/{src} for the host ...")
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise KernelsUnavailable(f"{cxx} failed on csrc/{src}:\n{' '.join(cmd)}\n{proc.stdout}")
    os.replace(tmp, out)
    prefix = f"libsx_{name}-"
    for fn in os.listdir(os.path.dirname(out)):
        if fn.startswith(prefix) and fn.endswith(".so") and os.path.join(os.path.dirname(out), fn) != out:
            try:
                os.remove(os.path.join(os.path.dirname(out), fn))
            except OSError:
                pass
    return out


_LOADED: Dict[str, ctypes.CDLL] = {}
_LOCK = threading.Lock()


def load_host_library(name: str) -> ctypes.CDLL:
    with _LOCK:
        key = "host:" + name
        lib = _LOADED.get(key)
        if lib is None:
            lib = _LOADED[key] = ctypes.CDLL(build_host_library(name))
        return lib


def load_library(name: str) -> ctypes.CDLL:
    """The library, compiled if need be.  Raises ``KernelsUnavailable``; never substitutes."""
    with _LOCK:
        lib = _LOADED.get(name)
        if lib is None:
            path = build_library(name)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelsUnavailable(f"cannot load {path}: {e}") from e
            _LOADED[name] = lib
        return lib
