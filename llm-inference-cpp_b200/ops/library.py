"""Builds and loads the library's CUDA kernels (``csrc/*.cu``) as one shared object.

The kernels are plain ``extern "C"`` launchers compiled by ``nvcc`` for sm_100a and
called through ``ctypes``; there is no other backend.  The object is built in-tree
(``csrc/_build/<hash>/``) at the first call that needs it and reused while the
sources are unchanged; when the tree is read-only it goes to a per-user temporary
folder instead.  A missing compiler or a failed build raises: nothing falls back
to the CPU or to library model code.
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

CSRC = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")
LIB_NAME = "libllmi_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]

_lock = threading.Lock()
_lib = None


class KernelLibraryError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[llmi_b200] {msg}", file=sys.stderr, flush=True)


def _sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    for cand in (os.environ.get("LLMI_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise KernelLibraryError("nvcc not found: the CUDA kernels of this library cannot be built "
                             "(set LLMI_NVCC or put nvcc on PATH)")


def _source_hash() -> str:
    h = hashlib.sha256()
    for name in _sources() + _headers():
        with open(os.path.join(CSRC, name), "rb") as f:
            h.update(name.encode())
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_root() -> str:
    in_tree = os.path.join(CSRC, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        root = os.path.join(tempfile.gettempdir(), f"llmi_b200_build_{os.getuid()}")
        os.makedirs(root, exist_ok=True)
        return root


def library_path() -> str:
    return os.path.join(_build_root(), _source_hash(), LIB_NAME)


def build(verbose: bool = True) -> str:
    """Compile every kernel source for sm_100a (if not built yet) and return the .so path."""
    path = library_path()
    if os.path.exists(path):
        return path
    nvcc = _find_nvcc()
    out_dir = os.path.dirname(path)
    os.makedirs(out_dir, exist_ok=True)
    srcs = _sources()
    if verbose:
        _say(f"building {len(srcs)} CUDA sources for sm_100a into {out_dir} (first call only)")
    t0 = time.time()
    done = [0]

    def compile_one(name: str) -> str:
        obj = os.path.join(out_dir, name[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", os.path.join(CSRC, name), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelLibraryError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
        done[0] += 1
        if verbose:
            _say(f"  compiled {name} ({done[0]}/{len(srcs)}, {time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = path + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelLibraryError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, path)
    for name in os.listdir(os.path.dirname(out_dir)):      # builds of older sources are of no use any more
        stale = os.path.join(os.path.dirname(out_dir), name)
        if stale != out_dir and os.path.isdir(stale) and len(name) == 16:
            shutil.rmtree(stale, ignore_errors=True)
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f} s")
    return path


def load() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _lib
    with _lock:
        if _lib is None:
            _lib = ctypes.CDLL(build())
        return _lib
