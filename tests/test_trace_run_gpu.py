"""bin/trace_run as a user runs it: a subprocess fed JSON lines, logits read back from
the files it writes, compared with the plain implementation."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_llama
import replay
from tiny import CONFIGS, TOL, load_plain_weights, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_mixed_trace(tmp_path, dtype):
    cfg, page = CONFIGS["B"]
    d = make_model_dir(tmp_path, "B", dtype)
    w = load_plain_weights(d)
    reqs = {f"q{i}": random_tokens(n, cfg["vocab_size"], 50 + i) for i, n in enumerate([9, 70, 64, 33, 101])}
    steps = replay.steps_mixed(reqs)
    lines = [json.dumps({"step": i, **st}) for i, st in enumerate(steps)]
    # the most tokens alive at once, each request rounded up to 64
    live, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            live[e["id"]] = live.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // 64) * 64 for n in live.values()))
        for rid in st["end"]:
            del live[rid]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                           "--out", str(out), "--max-tokens", str(peak), "--kv-block-size", str(page)],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.split("\n") if l] == [f"done {i}" for i in range(len(steps))]
    got = {}
    for i, st in enumerate(steps):
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = out / f"{i}.f32"
        if not wanted:
            assert not path.exists()
            continue
        arr = np.fromfile(path, dtype="<f4").reshape(wanted, cfg["vocab_size"])
        at = 0
        for e in st["entries"]:
            got.setdefault(e["id"], []).append(torch.from_numpy(arr[at:at + len(e["want"])].copy()))
            at += len(e["want"])
    for rid, toks in reqs.items():
        ref = plain_llama.forward(cfg, w, toks)
        g = torch.cat(got[rid]).double()
        assert g.shape == ref.shape
        assert float((g - ref).abs().max() / ref.abs().max()) < TOL[dtype]
