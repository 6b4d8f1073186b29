"""Compiling the CUDA sources of ``csrc/`` for sm_100a and loading them.

Each ``.cu`` file becomes one shared library with a plain C interface (raw
device pointers and a stream), so nothing here needs PyTorch's headers and a
file compiles in seconds.  Libraries are built on first use, into
``csrc/_build/`` inside the package (or a per-user temporary folder if that is
not writable), and rebuilt when a source, a header or a flag changes.  There is
no fallback: if nvcc or the GPU is missing, the first kernel call raises.
"""
from __future__ import annotations

import ctypes
import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from typing import Dict, List, Optional

CSRC = os.path.normpath(os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "csrc"))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-shared"]

# library name -> its source file; headers are shared by all.
LIBRARIES: Dict[str, str] = {
    "elementwise": "elementwise.cu",
    "gemm_f32": "gemm_f32.cu",
    "attention_simple": "attention_simple.cu",
    "sampling": "sampling.cu",
    "gemm_bf16_mma": "gemm_bf16_mma.cu",
    "gemm_bf16_skinny": "gemm_bf16_skinny.cu",
    "gemm_bf16_tcgen05": "gemm_bf16_tcgen05.cu",
    "gemm_bf16_swapab": "gemm_bf16_swapab.cu",
    "attention_bf16": "attention_bf16.cu",
    "attention_tcgen05": "attention_tcgen05.cu",
    "attention_decode_static": "attention_decode_static.cu",
}
# sources a library's file includes textually (they count for staleness)
INCLUDED_SOURCES: Dict[str, List[str]] = {"attention_decode_static.cu": ["attention_bf16.cu"]}


class KernelBuildError(RuntimeError):
    pass


def _find_nvcc() -> str:
    for cand in (os.environ.get("CUDA_HOME"), os.environ.get("CUDA_PATH"), "/usr/local/cuda"):
        if cand and os.path.exists(os.path.join(cand, "bin", "nvcc")):
            return os.path.join(cand, "bin", "nvcc")
    found = shutil.which("nvcc")
    if found:
        return found
    raise KernelBuildError("nvcc was not found (looked in $CUDA_HOME, /usr/local/cuda and PATH); "
                           "the kernels of this library cannot be built")


def _headers() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest(source: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in [source] + INCLUDED_SOURCES.get(source, []) + _headers():
        h.update(name.encode())
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


_BUILD_DIR: Optional[str] = None
_BUILD_DIR_LOCK = threading.Lock()


def build_dir() -> str:
    """``csrc/_build`` inside the package if it can be written, else a per-user
    folder under the system's temporary directory."""
    global _BUILD_DIR
    with _BUILD_DIR_LOCK:
        if _BUILD_DIR is None:
            in_tree = os.path.join(CSRC, "_build")
            try:
                os.makedirs(in_tree, exist_ok=True)
                fd, probe = tempfile.mkstemp(prefix=".probe", dir=in_tree)
                os.close(fd)
                os.remove(probe)
                _BUILD_DIR = in_tree
            except OSError:
                alt = os.path.join(tempfile.gettempdir(), f"go_tinygrad_b200_build_{os.getuid()}")
                os.makedirs(alt, exist_ok=True)
                _BUILD_DIR = alt
        return _BUILD_DIR


def _say(msg: str) -> None:
    print(f"[go-tinygrad_b200] {msg}", file=sys.stderr, flush=True)


def _compile(name: str, out_path: str) -> None:
    src = os.path.join(CSRC, LIBRARIES[name])
    tmp = f"{out_path}.{os.getpid()}.tmp"
    cmd = [_find_nvcc()] + NVCC_FLAGS + ["-I", CSRC, src, "-o", tmp]
    _say(f"compiling {LIBRARIES[name]} for sm_100a ...")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  still compiling {LIBRARIES[name]} ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    finally:
        done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"nvcc failed on {LIBRARIES[name]}:\n{proc.stdout}")
    os.replace(tmp, out_path)
    _say(f"  built {os.path.basename(out_path)} in {time.time() - t0:.1f} s")


def ensure_built(name: str) -> str:
    """Path of the up-to-date shared library `name`, compiling it if needed."""
    if name not in LIBRARIES:
        raise KeyError(f"unknown kernel library {name!r}; known: {sorted(LIBRARIES)}")
    bdir = build_dir()
    path = os.path.join(bdir, f"gtg_{name}_{_digest(LIBRARIES[name])}.so")
    if os.path.exists(path):
        return path
    lock_path = os.path.join(bdir, f".{name}.lock")
    with open(lock_path, "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if not os.path.exists(path):
                for old in os.listdir(bdir):       # drop stale builds of the same library
                    if old.startswith(f"gtg_{name}_") and old.endswith(".so"):
                        try:
                            os.remove(os.path.join(bdir, old))
                        except OSError:
                            pass
                _compile(name, path)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)
    return path


_LOADED: Dict[str, ctypes.CDLL] = {}


def library(name: str) -> ctypes.CDLL:
    lib = _LOADED.get(name)
    if lib is None:
        lib = ctypes.CDLL(ensure_built(name))
        _LOADED[name] = lib
    return lib


def build_all(names: Optional[List[str]] = None) -> List[str]:
    """Compile every library (in parallel); returns their paths."""
    names = list(LIBRARIES) if names is None else names
    paths: Dict[str, str] = {}
    errors: List[BaseException] = []

    def work(n):
        try:
            paths[n] = ensure_built(n)
        except BaseException as e:  # noqa: BLE001 - reported below
            errors.append(e)

    threads = [threading.Thread(target=work, args=(n,)) for n in names]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return [paths[n] for n in names]
