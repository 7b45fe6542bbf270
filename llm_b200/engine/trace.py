"""Trace replay: feeds given token ids through the engine step by step and writes
the logits that are asked for.  It samples nothing and has no forward pass, cache or
loader of its own: it drives Engine.step, the step that generation uses.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, <out>/<step>.f32 holds the logits at the
wanted places, in the order of the entries and of `want`, little-endian float32
[wanted, vocab].  After every step the line `done <step>` is printed and flushed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def _parse_args(argv):
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__,
                                formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens that live requests hold at any time (each rounded up to 64)")
    p.add_argument("--kv-block-size", type=int, default=16)
    p.add_argument("--max-live", type=int, default=8, help="most requests alive at once")
    return p.parse_args(argv)


def main(argv=None, stdin=None, stdout=None) -> int:
    args = _parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    os.makedirs(args.out, exist_ok=True)

    from ..config.engine_options import EngineOptions
    from ..config.model_config import load_config
    from .engine import Engine, StepEntry

    _arch, cfg = load_config(args.model)
    max_pos = getattr(cfg, "max_position_embeddings")
    page = args.kv_block_size
    if args.max_tokens <= 0:
        raise SystemExit("--max-tokens must be positive")
    pool_tokens = (args.max_tokens + 63) // 64 * 64
    per_step = min(max(pool_tokens, 64), 8192)
    options = EngineOptions(
        dtype=args.dtype, kv_block_size=page, max_num_seqs=args.max_live,
        max_num_batched_tokens=per_step, max_logit_rows=per_step, max_seq_len=max_pos,
        num_kv_blocks=pool_tokens // page, use_cuda_graphs=False)
    engine = Engine(args.model, options)

    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        if entries:
            logits = engine.step(entries)
            engine.check_status()          # a step whose kernels reported a failure writes no logits
            if logits.shape[0]:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(args.out, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(args.out, f"{step}.f32"))
        for rid in rec.get("end", []):
            engine.release(rid)
        print(f"done {step}", file=stdout, flush=True)
    engine.check_status()
    return 0


if __name__ == "__main__":
    sys.exit(main())
