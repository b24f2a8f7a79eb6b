"""Builds the CUDA sources of `csrc/` into shared libraries, one per source file,
each at its first use.

`nvcc -gencode arch=compute_100a,code=sm_100a -shared` straight to a `.so` that
is loaded with ctypes; there is no framework header in the kernels, so a file
compiles in seconds.  The library is kept beside the package (`lib/`) under a
name that carries a hash of its sources and flags, so a changed source is
rebuilt and a fresh checkout compiles only what the model at hand needs.  If
the package folder cannot be written, a per-user folder under the system's
temporary directory is used instead.  While a file compiles, a line is printed
to stderr at the start and every few seconds.
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
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
_LIB_DIR = os.path.join(os.path.dirname(_HERE), "lib")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]

# Host-only sources (C++, no device code): compiled by the same nvcc call, which hands them
# to the host compiler.
HOST_SOURCES = {"host_step": "host_step.cpp", "host_cache": "host_cache.cpp"}

# source file -> extra headers whose change must trigger a rebuild
MODULES: Dict[str, List[str]] = {
    "host_step": [],
    "host_cache": [],
    "elementwise": ["common.cuh"],
    "gemm_simt": ["common.cuh"],
    "attention_generic": ["common.cuh"],
    "sampling": ["common.cuh", "no_alloc_argmax.h"],
}

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def register_module(name: str, headers: List[str]) -> None:
    MODULES[name] = list(headers)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels of crucible_b200 cannot be built")


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for fn in [_source(name)] + MODULES[name]:
        with open(os.path.join(CSRC, fn), "rb") as f:
            h.update(fn.encode())
            h.update(f.read())
    return h.hexdigest()[:16]


def _source(name: str) -> str:
    return HOST_SOURCES.get(name, name + ".cu")


def _writable_dir() -> str:
    try:
        os.makedirs(_LIB_DIR, exist_ok=True)
        probe = os.path.join(_LIB_DIR, f".probe-{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return _LIB_DIR
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"crucible_b200-lib-{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def library_path(name: str) -> str:
    """Path of the built library of module `name`, building it if needed."""
    if name not in MODULES:
        raise BuildError(f"no CUDA module named {name!r}; known: {sorted(MODULES)}")
    fname = f"cb_{name}-{_digest(name)}.so"
    in_tree = os.path.join(_LIB_DIR, fname)
    if os.path.exists(in_tree):
        return in_tree
    out_dir = _writable_dir()
    target = os.path.join(out_dir, fname)
    if os.path.exists(target):
        return target
    for old in os.listdir(out_dir):
        if old.startswith(f"cb_{name}-") and old.endswith(".so"):
            try:
                os.remove(os.path.join(out_dir, old))
            except OSError:
                pass
    tmp = os.path.join(out_dir, f".{fname}.{os.getpid()}.tmp")
    cmd = [_nvcc()] + NVCC_FLAGS + ["-I", CSRC, "-o", tmp, os.path.join(CSRC, _source(name))]
    print(f"[crucible_b200] compiling {_source(name)} for sm_100a (first use) ...",
          file=sys.stderr, flush=True)
    t0 = time.time()
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, env=env)
    out_chunks: List[bytes] = []
    reader = threading.Thread(target=lambda: out_chunks.append(proc.stdout.read()), daemon=True)
    reader.start()
    while True:
        try:
            proc.wait(timeout=5)
            break
        except subprocess.TimeoutExpired:
            print(f"[crucible_b200] ... still compiling {_source(name)} ({time.time() - t0:.0f} s)",
                  file=sys.stderr, flush=True)
    reader.join()
    log = b"".join(out_chunks).decode(errors="replace")
    if proc.returncode != 0:
        try:
            os.remove(tmp)
        except OSError:
            pass
        raise BuildError(f"nvcc failed on {_source(name)}:\n{log}")
    os.replace(tmp, target)
    print(f"[crucible_b200] built {name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
    return target


def load(name: str) -> ctypes.CDLL:
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            lib = ctypes.CDLL(library_path(name))
            _loaded[name] = lib
        return lib


def build_all() -> List[str]:
    return [library_path(name) for name in sorted(MODULES)]
