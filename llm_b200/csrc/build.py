"""Builds the kernel library for sm_100a with nvcc and loads it with ctypes.

The kernels have a C interface and use no torch headers, so a file compiles in
seconds.  The library is built in-tree (llm_b200/csrc/_build) at the first call,
or in a temporary folder when the tree is read-only, and rebuilt when a source or
a flag changes.  While nvcc runs, a line is printed now and then.
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

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_NAME = "libllm_b200_kernels.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


class KernelBuildError(RuntimeError):
    pass


def sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _find_nvcc() -> str:
    for cand in (os.environ.get("LLM_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $LLM_B200_NVCC, PATH and /usr/local/cuda/bin)")


def _digest() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources() + _headers():
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _build_dir() -> str:
    d = os.environ.get("LLM_B200_BUILD_DIR") or os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"llm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[llm_b200] {msg}", file=sys.stderr, flush=True)


def library_path() -> str:
    return os.path.join(_build_dir(), LIB_NAME)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compile what is stale and return the path of the shared library."""
    bdir = _build_dir()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "sources.sha256")
    digest = _digest()
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    nvcc = _find_nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)")
    t0 = time.time()
    done = []
    stop = threading.Event()

    def ticker():
        while not stop.wait(10.0):
            _say(f"  ... still compiling: {len(done)}/{len(srcs)} files done after {time.time() - t0:.0f} s")

    def compile_one(name: str) -> str:
        obj = os.path.join(bdir, name[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", _HERE, "-c", os.path.join(_HERE, name), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {name}:\n{r.stdout}\n{r.stderr}")
        done.append(name)
        if verbose:
            _say(f"  compiled {name} ({len(done)}/{len(srcs)}, {time.time() - t0:.0f} s)")
        return obj

    th = threading.Thread(target=ticker, daemon=True)
    if verbose:
        th.start()
    try:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(digest)
    finally:
        stop.set()
    if verbose:
        _say(f"kernel library ready after {time.time() - t0:.0f} s")
    return lib


_LIB = None
_LOCK = threading.Lock()


def load() -> ctypes.CDLL:
    """The kernel library, built if needed.  Raises if it cannot be had: there is no
    other implementation to fall back to."""
    global _LIB
    with _LOCK:
        if _LIB is None:
            path = build()
            try:
                _LIB = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            _LIB.llmk_last_error.restype = ctypes.c_char_p
        return _LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
