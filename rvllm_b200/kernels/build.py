"""Compiling the CUDA sources under csrc/ for sm_100a and loading them with ctypes.

Each source file becomes one shared library, built with nvcc on its first use and kept in a
build folder beside the sources (or under the temporary folder when the package folder is
read-only).  A library's file name carries a hash of its source, headers, defines and flags,
so a changed source is rebuilt and an unchanged one is reused.  While nvcc runs, a line is
printed every few seconds.  There is no fallback: a library that cannot be built or loaded
raises `KernelError`.
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
from typing import Dict, Iterable, Optional, Sequence, Tuple

from ..errors import KernelError

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--shared", "-Xcompiler", "-fPIC"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def find_nvcc() -> str:
    for cand in (os.environ.get("RVLLM_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelError("nvcc was not found (looked at $RVLLM_NVCC, PATH and /usr/local/cuda/bin): "
                      "the CUDA kernels cannot be built")


def build_dir() -> str:
    """`csrc/_build` when writable, else a per-user folder under the temporary directory."""
    override = os.environ.get("RVLLM_BUILD_DIR")
    candidates = [override] if override else []
    candidates.append(os.path.join(CSRC_DIR, "_build"))
    candidates.append(os.path.join(tempfile.gettempdir(), f"rvllm_b200_build_{os.getuid()}"))
    for d in candidates:
        try:
            os.makedirs(d, exist_ok=True)
            fd, probe = tempfile.mkstemp(prefix=".w", dir=d)
            os.close(fd)
            os.unlink(probe)
            return d
        except OSError:
            continue
    raise KernelError(f"no writable build folder among {candidates}")


def _headers() -> Sequence[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _digest(source: str, defines: Sequence[str]) -> str:
    h = hashlib.sha256()
    for name in [source, *_headers()]:
        with open(os.path.join(CSRC_DIR, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(" ".join(defines).encode())
    return h.hexdigest()[:16]


def library_path(source: str, defines: Sequence[str] = ()) -> str:
    stem = os.path.splitext(source)[0]
    tag = "".join("_" + d.replace("=", "").replace("-D", "") for d in defines)
    return os.path.join(build_dir(), f"librvllm_{stem}{tag}_{_digest(source, defines)}.so")


def compile_library(source: str, defines: Sequence[str] = (), verbose: bool = True) -> str:
    """Build `csrc/<source>` if its library is not there yet; return the library's path."""
    out = library_path(source, defines)
    if os.path.exists(out):
        return out
    nvcc = find_nvcc()
    tmp = f"{out}.tmp{os.getpid()}"
    cmd = [nvcc, *NVCC_FLAGS, *defines, "-I", CSRC_DIR, "-o", tmp, os.path.join(CSRC_DIR, source)]
    if verbose:
        print(f"[rvllm_b200] compiling {source} {' '.join(defines)} for sm_100a ...", file=sys.stderr, flush=True)
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            log, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            if verbose:
                print(f"[rvllm_b200] ... still compiling {source} ({time.time() - t0:.0f} s)",
                      file=sys.stderr, flush=True)
    if proc.returncode != 0:
        try:
            os.unlink(tmp)
        except OSError:
            pass
        raise KernelError(f"nvcc failed for {source} (exit {proc.returncode}):\n{' '.join(cmd)}\n{log}")
    os.replace(tmp, out)
    # older builds of the same source and defines are of no use any more
    stem = os.path.basename(out).rsplit("_", 1)[0] + "_"
    for name in os.listdir(os.path.dirname(out)):
        if name.startswith(stem) and name.endswith(".so") and len(name) == len(os.path.basename(out)) \
                and name != os.path.basename(out):
            try:
                os.unlink(os.path.join(os.path.dirname(out), name))
            except OSError:
                pass
    if verbose:
        print(f"[rvllm_b200] built {os.path.basename(out)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return out


def load_library(source: str, defines: Sequence[str] = ()) -> ctypes.CDLL:
    key = source + "|" + " ".join(defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            path = compile_library(source, defines)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelError(f"cannot load {path}: {e}") from None
            _loaded[key] = lib
        return lib


def all_sources() -> Sequence[str]:
    return sorted(f for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))
