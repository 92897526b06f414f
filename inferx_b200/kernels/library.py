"""Builds and loads the sm_100a kernel library.

The kernels are plain CUDA sources under ``inferx_b200/csrc`` with C entry
points; they are compiled with nvcc into one shared library that is loaded with
``ctypes``.  The library is built at first use (a fresh checkout has no built
files), into ``inferx_b200/csrc/_build`` when that folder can be written and
otherwise into a per-user folder under the system's temporary directory.  A
progress line is printed every few seconds while nvcc runs.  There is no
fallback: if the library cannot be built or loaded, using any kernel raises.
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
from typing import List, Optional

CSRC_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "csrc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


class KernelLibraryError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[inferx_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    cand = [os.environ.get("INFERX_NVCC"), shutil.which("nvcc"),
            os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
            "/usr/local/cuda/bin/nvcc"]
    for c in cand:
        if c and os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise KernelLibraryError(
        "nvcc not found (looked at $INFERX_NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
        "the sm_100a kernels cannot be built and there is no other execution path")


def sources() -> List[str]:
    return sorted(
        os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(
        os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))


def _digest() -> str:
    h = hashlib.sha256()
    for path in sources() + _headers():
        h.update(os.path.basename(path).encode())
        with open(path, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    override = os.environ.get("INFERX_BUILD_DIR")
    if override:
        os.makedirs(override, exist_ok=True)
        return override
    in_tree = os.path.join(CSRC_DIR, "_build")
    try:
        os.makedirs(in_tree, exist_ok=True)
        probe = os.path.join(in_tree, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return in_tree
    except OSError:
        pass
    d = os.path.join(tempfile.gettempdir(), f"inferx_b200-{os.getuid()}")
    os.makedirs(d, exist_ok=True)
    return d


def _run(cmd: List[str], what: str) -> None:
    p = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        raise KernelLibraryError(f"{what} failed ({' '.join(cmd)}):\n{p.stdout}")


def library_path() -> str:
    return os.path.join(_build_dir(), f"libinferx_b200_{_digest()}.so")


def build(verbose: bool = True) -> str:
    """Compile every kernel source for sm_100a; returns the library path."""
    out = library_path()
    if os.path.isfile(out):
        return out
    nvcc = find_nvcc()
    bdir = os.path.dirname(out)
    srcs = sources()
    tag = _digest()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA sources for sm_100a into {bdir} (first use only)")
    objs = [os.path.join(bdir, f"{os.path.basename(s)[:-3]}_{tag}.o") for s in srcs]
    done = [0]
    stop = threading.Event()

    def ticker():
        t0 = time.time()
        while not stop.wait(5.0):
            _say(f"  still compiling: {done[0]}/{len(srcs)} sources done, "
                 f"{time.time() - t0:.0f}s elapsed")

    def compile_one(pair):
        src, obj = pair
        _run([nvcc] + NVCC_FLAGS + ["-I", CSRC_DIR, "-c", src, "-o", obj],
             f"nvcc {os.path.basename(src)}")
        done[0] += 1

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            list(pool.map(compile_one, zip(srcs, objs)))
        tmp = out + f".tmp{os.getpid()}"
        _run([nvcc, "-shared", "-o", tmp] + objs, "link")
        os.replace(tmp, out)
        for f in os.listdir(bdir):   # libraries of older sources
            if f.startswith("libinferx_b200_") and f.endswith(".so") and \
                    os.path.join(bdir, f) != out:
                try:
                    os.remove(os.path.join(bdir, f))
                except OSError:
                    pass
    finally:
        stop.set()
        for o in objs:
            try:
                os.remove(o)
            except OSError:
                pass
    if verbose:
        _say(f"built {out}")
    return out


_lib: Optional[ctypes.CDLL] = None
_lock = threading.Lock()


def load() -> ctypes.CDLL:
    """The loaded kernel library; builds it first if needed."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            # torch brings the CUDA runtime the library links against
            import torch  # noqa: F401
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelLibraryError(f"cannot load kernel library {path}: {e}") from None
    return _lib
