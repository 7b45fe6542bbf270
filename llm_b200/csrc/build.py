"""Builds the kernel libraries for sm_100a with nvcc and loads them with ctypes.

The kernels have a C interface and use no torch headers, so a file compiles in
seconds.  There are two libraries: the plain one (everything a float32 model needs,
and what a bfloat16 model runs on the CUDA cores) and the tensor-core one (bfloat16
products and attention), which is only built and loaded when a bfloat16 model asks for
it.  A library is built in-tree (llm_b200/csrc/_build) at its first use, or in a
temporary folder when the tree is read-only, and rebuilt when a source or a flag
changes.  While nvcc runs, a line is printed now and then.
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
GROUPS = {
    # group -> (library file, sources); runtime.cu (error text, switches) is linked into both
    "plain": (LIB_NAME, ["runtime.cu", "rows.cu", "gemm_simt.cu", "rope_cache.cu", "attention_generic.cu",
                         "attention_decode.cu", "sampling.cu"]),
    "tensor": ("libllm_b200_tensor.so", ["runtime.cu", "gemm_tc.cu", "attention_tc.cu", "attention_decode_mma.cu"]),
    # host side of the runtime (page pool, step metadata, scheduler): plain C++, built with g++, needs no CUDA
    "host": ("libllm_b200_host.so", ["host/page_pool.cpp", "host/scheduler.cpp"]),
}
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


# extra nvcc flags from the environment (for experiments, e.g. -DNAME=1); part of the build's digest
NVCC_FLAGS += os.environ.get("LLM_B200_NVCC_FLAGS", "").split()


class KernelBuildError(RuntimeError):
    pass


def sources(group: str = None):
    """The CUDA files of a group, or of all groups."""
    if group is not None:
        return list(GROUPS[group][1])
    every = sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))
    every += sorted("host/" + f for f in os.listdir(os.path.join(_HERE, "host")) if f.endswith(".cpp"))
    listed = {f for _, files in GROUPS.values() for f in files}
    stray = [f for f in every if f not in listed]
    if stray:
        raise KernelBuildError(f"CUDA files that belong to no library: {stray}")
    return every


def _headers():
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _find_cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++")):
        if cand and (os.path.isfile(cand) or shutil.which(cand)):
            return shutil.which(cand) or cand
    raise KernelBuildError("no C++ compiler found (looked at $CXX, g++ and c++ on PATH)")


def _find_nvcc() -> str:
    for cand in (os.environ.get("LLM_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $LLM_B200_NVCC, PATH and /usr/local/cuda/bin)")


def _digest(group: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for name in sources(group) + (_headers() if group != "host" else []):
        h.update(name.encode())
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()


_BUILD_DIR = None
_DIR_LOCK = threading.Lock()


def _build_dir() -> str:
    """Where objects and libraries go; chosen once per process."""
    global _BUILD_DIR
    with _DIR_LOCK:
        if _BUILD_DIR is None:
            _BUILD_DIR = _choose_build_dir()
        return _BUILD_DIR


def _choose_build_dir() -> str:
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


def library_path(group: str = "plain") -> str:
    return os.path.join(_build_dir(), GROUPS[group][0])


def build(force: bool = False, verbose: bool = True, group: str = None) -> str:
    """Compile what is stale of one library (or, without a group, of both) and return the path of
    the shared library (of the plain one when both are built)."""
    if group is None:
        sources()                                   # every file belongs to a library
        with ThreadPoolExecutor(max_workers=len(GROUPS)) as pool:      # the libraries side by side
            paths = list(pool.map(lambda g: build(force, verbose, g), GROUPS))
        return paths[0]
    if group == "host":
        return _build_host(force, verbose)
    bdir = _build_dir()
    lib = os.path.join(bdir, GROUPS[group][0])
    stamp = os.path.join(bdir, f"{group}.sha256")
    digest = _digest(group)
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    nvcc = _find_nvcc()
    srcs = sources(group)
    if verbose:
        _say(f"compiling the {group} kernel library: {len(srcs)} CUDA files for sm_100a into {bdir} (first use only)")
    t0 = time.time()
    done = []
    stop = threading.Event()

    def ticker():
        while not stop.wait(10.0):
            _say(f"  ... still compiling: {len(done)}/{len(srcs)} files done after {time.time() - t0:.0f} s")

    def compile_one(name: str) -> str:
        obj = os.path.join(bdir, f"{group}_{name[:-3]}.o")      # a file that both libraries carry is compiled for each
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
        _say(f"{group} kernel library ready after {time.time() - t0:.0f} s")
    return lib


def _build_host(force: bool, verbose: bool) -> str:
    """The host library: C++ files compiled and linked by g++ in one go (a second or two)."""
    bdir = _build_dir()
    name, srcs = GROUPS["host"]
    lib = os.path.join(bdir, name)
    stamp = os.path.join(bdir, "host.sha256")
    h = hashlib.sha256(" ".join(CXX_FLAGS).encode())
    for f in sorted("host/" + n for n in os.listdir(os.path.join(_HERE, "host")) if n.endswith((".cpp", ".h"))):
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(f.encode() + fh.read())
    digest = h.hexdigest()
    if not force and os.path.isfile(lib) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return lib
    t0 = time.time()
    tmp = lib + f".tmp{os.getpid()}"
    cmd = [_find_cxx(), *CXX_FLAGS, "-shared", "-o", tmp, *[os.path.join(_HERE, f) for f in srcs]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise KernelBuildError(f"{cmd[0]} failed on the host library:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib)
    with open(stamp, "w") as f:
        f.write(digest)
    if verbose:
        _say(f"host library ready after {time.time() - t0:.0f} s")
    return lib


_LIBS = {}
_LOCK = threading.Lock()


def load(group: str = "plain") -> ctypes.CDLL:
    """A kernel library, built if needed.  Raises if it cannot be had: there is no
    other implementation to fall back to."""
    lib = _LIBS.get(group)
    if lib is not None:
        return lib
    with _LOCK:
        if group not in _LIBS:
            path = build(group=group)
            try:
                lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
            if group != "host":
                lib.llmk_last_error.restype = ctypes.c_char_p
            _LIBS[group] = lib
        return _LIBS[group]


def load_host() -> ctypes.CDLL:
    """The host library (page pool, step metadata); needs a C++ compiler, no GPU."""
    return load("host")


def load_tensor() -> ctypes.CDLL:
    """The tensor-core library (bfloat16 products and attention)."""
    return load("tensor")


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
