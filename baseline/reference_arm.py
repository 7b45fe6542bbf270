"""The reference arm: the unmodified reference (zhan-wei-919/llm) built with nvcc and driven
through its own public API by baseline/ref_harness.cu.

The reference is a header-only C++/CUDA tree with no setup.py or pyproject.toml, so pip has
nothing to install; what its own programs do instead is `nvcc -O3 -std=c++17 -arch=...` on one
.cu file that includes the headers (model/llm/test/bench_tiny_llama_load.cu:21-23).  This module
does the same: a copy of the tree under baseline/_ref (never edited), the harness compiled
against it for sm_100a, a checkpoint of the TinyLlama shape written for it, and the harness run
as a child process that speaks one command and one JSON line at a time.  Nothing of llm_b200's
engine or kernels is loaded in that process; this side only writes the checkpoint file.
"""
from __future__ import annotations

import hashlib
import json
import os
import select
import shutil
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_TREE = os.path.join(HERE, "_ref")
BUILD_DIR = os.path.join(HERE, "_build")
HARNESS_SRC = os.path.join(HERE, "ref_harness.cu")
HARNESS_BIN = os.path.join(BUILD_DIR, "ref_harness")
UPSTREAM = os.environ.get("LLM_B200_REFERENCE", "/root/reference")

# TinyLlama 1.1B, the one shape the reference's attention kernel exists for
# (kernel/attention/Attention.h:12-19; model/llm/tiny_llama.cpp:17-21)
MODEL = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=5632,
             num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
             vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048,
             tie_word_embeddings=False)


class ReferenceUnavailable(RuntimeError):
    """The reference cannot be built or run here; str() is the one-line reason."""


def _say(msg: str) -> None:
    print(f"[reference arm] {msg}", file=sys.stderr, flush=True)


def ensure_tree() -> str:
    """baseline/_ref: a verbatim copy of the reference's tree (without its .git)."""
    marker = os.path.join(REF_TREE, "runtime", "LLM.h")
    if os.path.isfile(marker):
        return REF_TREE
    if not os.path.isfile(os.path.join(UPSTREAM, "runtime", "LLM.h")):
        raise ReferenceUnavailable(f"no copy of the reference under baseline/_ref and none at {UPSTREAM}")
    shutil.copytree(UPSTREAM, REF_TREE, ignore=shutil.ignore_patterns(".git"), dirs_exist_ok=True)
    return REF_TREE


def _tree_digest() -> str:
    h = hashlib.sha256()
    with open(HARNESS_SRC, "rb") as f:
        h.update(f.read())
    for root, dirs, files in os.walk(REF_TREE):
        dirs.sort()
        for name in sorted(files):
            if name.endswith((".h", ".cuh")):
                with open(os.path.join(root, name), "rb") as f:
                    h.update(name.encode() + f.read())
    return h.hexdigest()


def build_harness(verbose: bool = True) -> str:
    """Compile the harness against the copy of the reference (about 20 s; kept until a source changes)."""
    ensure_tree()
    os.makedirs(BUILD_DIR, exist_ok=True)
    stamp = HARNESS_BIN + ".sha256"
    digest = _tree_digest()
    if os.path.isfile(HARNESS_BIN) and os.path.isfile(stamp) and open(stamp).read().strip() == digest:
        return HARNESS_BIN
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isfile(nvcc):
        raise ReferenceUnavailable("nvcc not found: the reference harness cannot be compiled")
    if verbose:
        _say("compiling the reference with nvcc for sm_100a (about 20 s, first use only)")
    tmp = HARNESS_BIN + f".tmp{os.getpid()}"
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-Xcompiler", "-pthread",
           "-I", REF_TREE, HARNESS_SRC, "-o", tmp]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        tail = (r.stderr or r.stdout).strip().splitlines()[-1:] or ["no output"]
        raise ReferenceUnavailable(f"nvcc failed on the reference: {tail[0][:200]}")
    os.replace(tmp, HARNESS_BIN)
    with open(stamp, "w") as f:
        f.write(digest)
    return HARNESS_BIN


def write_weights(folder: str, layers: int = 22, seed: int = 20240531) -> str:
    """model.safetensors for the reference: the seeded random tensors of llm_b200's random-weights
    mode at the TinyLlama shape, EVERY tensor stored as bfloat16.  The reference copies a tensor's
    bytes as they are (runtime/LLM.h:140-143) into storage of its compute type, so the norm gains,
    which llm_b200 stores in float32, must be bfloat16 here."""
    import torch

    root = os.path.dirname(HERE)
    if root not in sys.path:
        sys.path.insert(0, root)
    from llm_b200.weights.loader import expected_tensors, random_tensor
    from llm_b200.weights.safetensors_io import write_safetensors

    cfg = dict(MODEL, num_hidden_layers=layers)
    os.makedirs(folder, exist_ok=True)
    tensors = {name: random_tensor(name, info, seed).to(torch.bfloat16) for name, info in expected_tensors(cfg).items()}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(dict(cfg, torch_dtype="bfloat16"), f)
    path = os.path.join(folder, "model.safetensors")
    write_safetensors(path, tensors, metadata={"format": "pt", "seed": str(seed)})
    return path


class Harness:
    """One run of the harness: commands in, JSON lines out."""

    def __init__(self, weights: str, max_seqs: int = 8, max_tokens: int = 512, max_seq_len: int = 2048,
                 layers: int = 22, timeout: float = 600.0):
        self.timeout = timeout
        binary = build_harness()
        self.proc = subprocess.Popen(
            [binary, "--weights", weights, "--max-seqs", str(max_seqs), "--max-tokens", str(max_tokens),
             "--max-seq-len", str(max_seq_len), "--layers", str(layers)],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, bufsize=1)
        self.ready = self._read()
        if self.ready.get("mode") != "ready":
            self.close()
            raise ReferenceUnavailable(f"the reference did not start: {json.dumps(self.ready)[:200]}")

    def _read(self) -> dict:
        ready, _, _ = select.select([self.proc.stdout], [], [], self.timeout)
        if not ready:
            self.proc.kill()
            return {"error": f"no answer from the harness within {self.timeout:.0f} s"}
        line = self.proc.stdout.readline()
        if not line:
            rc = self.proc.wait()
            err = (self.proc.stderr.read() or "").strip().splitlines()[-1:] or [""]
            return {"error": f"the harness exited with code {rc}: {err[0][:160]}"}
        try:
            return json.loads(line)
        except json.JSONDecodeError:
            return {"error": f"unreadable line: {line.strip()[:160]}"}

    def command(self, text: str) -> dict:
        self.proc.stdin.write(text.strip() + "\n")
        self.proc.stdin.flush()
        return self._read()

    def close(self) -> None:
        if self.proc.poll() is None:
            try:
                self.proc.stdin.close()
                self.proc.wait(timeout=60)
            except (OSError, subprocess.TimeoutExpired):
                self.proc.kill()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


if __name__ == "__main__":
    t0 = time.time()
    print(build_harness(), f"({time.time() - t0:.0f} s)")
