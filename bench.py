"""Serving benchmark of the engine on one B200: decode tokens per second of a
TinyLlama-1.1B-shaped model with seeded random weights (bfloat16), plus prefill
throughput, the decode step's share of the HBM roofline and decode at batch 1 and 64.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A "step" is one decode step of the whole batch.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Layer sizes of the benchmark model (TinyLlama 1.1B).
MODEL = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=5632,
             num_hidden_layers=22, num_attention_heads=32, num_key_value_heads=4, head_dim=64,
             vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=2048,
             tie_word_embeddings=False)
FULL_LAYERS = 22
PROMPT_LEN = 512          # decode starts from 512-token prompts
NEW_TOKENS = 256          # and the benchmark definition generates 256 tokens
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# The larger shapes of the benchmark definition: layer sizes only, random weights.
LLAMA2_7B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=11008,
                 num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=32, head_dim=128,
                 vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0, max_position_embeddings=4096,
                 tie_word_embeddings=False)
LLAMA3_8B = dict(architectures=["LlamaForCausalLM"], hidden_size=4096, intermediate_size=14336,
                 num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                 vocab_size=128256, rms_norm_eps=1e-5, rope_theta=500000.0, max_position_embeddings=8448,   # 8,000 + 256 positions are used
                 tie_word_embeddings=False)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except Exception:
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples, self.proc, self.index = [], None, index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        sm, mx, reasons = [], [], set()
        for p in self.samples:
            try:
                sm.append(int(float(p[0]))); mx.append(int(float(p[1])))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def matmul_params(cfg, layers):
    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    QN = cfg["num_attention_heads"] * cfg["head_dim"]
    KN = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = H * (QN + 2 * KN) + QN * H + 3 * H * I
    return per_layer * layers, V * H


def decode_bytes(cfg, layers, batch, ctx_tokens):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    body, head = matmul_params(cfg, layers)
    norms = (2 * layers + 1) * cfg["hidden_size"] * 4
    weights = (body + head) * 2 + norms + batch * cfg["hidden_size"] * 2      # embedding: one row per request
    kv = 2 * layers * cfg["num_key_value_heads"] * cfg["head_dim"] * 2 * ctx_tokens
    return weights + kv


def prefill_flops(cfg, layers, tokens, head_rows=1):
    body, head = matmul_params(cfg, layers)
    QN = cfg["num_attention_heads"] * cfg["head_dim"]
    attn = layers * 2 * 2 * QN * tokens * (tokens + 1) / 2        # QK^T and PV over the causal half
    return 2.0 * body * tokens + 2.0 * head * head_rows + attn


def generate_point(cfg, prompts, new_tokens, max_seqs, chunk, peaks, seed=20240531, llm=None):
    """One workload through LLM.generate and the scheduler: the requests all at once, prompts taken
    in portions of at most `chunk` tokens a step beside the decoded tokens of the others.  Timed on
    the host around generate() (tokens in, tokens out), after one untimed run of the same
    requests.  Fractions: the steps that only decode against the HBM roofline (weights once + the
    live cache per step), the steps that bring prompt portions against the tensor peak."""
    import torch

    from llm_b200.engine.llm import LLM
    from llm_b200.engine.scheduler import SchedulerConfig
    layers = cfg["num_hidden_layers"]
    longest = max(len(p) for p in prompts) + new_tokens
    own = llm is None
    if own:
        pages = sum(-(-(len(p) + new_tokens) // 16) for p in prompts) + 64
        llm = LLM(None, dtype="bfloat16", max_num_seqs=max_seqs, max_num_batched_tokens=chunk, max_seq_len=longest,
                  eos_token_id=-1, kv_block_size=16, num_kv_blocks=pages, random_config=cfg, random_seed=seed,
                  random_on_device=True)
    else:
        keep = llm.scheduler_config
        llm.scheduler_config = SchedulerConfig(max_seqs, chunk, -1)
    try:
        llm.generate(prompts, max_new_tokens=new_tokens)               # untimed: kernels built, graphs captured
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        gen = llm.generate(prompts, max_new_tokens=new_tokens)
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        st = llm.last_stats
        counters = dict(llm.engine.counters)
        free_pages = [llm.engine.cache.num_free_pages(g) for g in range(llm.engine.cache.num_groups)]
    finally:
        if not own:
            llm.scheduler_config = keep
    n_prompt = sum(len(p) for p in prompts)
    n_new = sum(len(g) for g in gen)
    out = {"requests": len(prompts), "prompt_tokens": n_prompt, "new_tokens": n_new, "max_num_seqs": max_seqs,
           "chunk": chunk, "wall_s": round(wall, 4), "tok_s": round(n_new / wall, 1),
           "total_tok_s": round((n_new + n_prompt) / wall, 1), "steps": st["steps"],
           "preemptions": st["preemptions"], "free_pages_after": free_pages,
           "graph_captures": counters["graph_captures"], "graph_replays": counters["graph_replays"]}
    if st["decode_steps"]:
        # every request decodes in these steps; their mean context is taken as prompt + half of the new tokens
        batch = st["decode_tokens"] / st["decode_steps"]
        ctx = batch * (n_prompt / len(prompts) + new_tokens / 2.0)
        bytes_step = decode_bytes(cfg, layers, batch, ctx)
        ms = st["decode_seconds"] / st["decode_steps"] * 1e3
        out["decode"] = {"steps": st["decode_steps"], "batch": round(batch, 2), "ms_per_step": round(ms, 4),
                         "tok_s": round(st["decode_tokens"] / st["decode_seconds"], 1),
                         "frac_hbm": round(bytes_step / (ms / 1e3) / 1e9 / peaks["hbm_gbs"], 4)}
    if st["prompt_steps"]:
        fl = sum(prefill_flops(cfg, layers, len(p)) for p in prompts)
        out["prefill"] = {"steps": st["prompt_steps"], "tokens": st["prompt_step_tokens"],
                          "tok_s": round(st["prompt_step_tokens"] / st["prompt_seconds"], 1),
                          "frac_tensor": round(fl / st["prompt_seconds"] / (peaks["bf16_tflops"] * 1e12), 4)}
    if own:
        del llm
        import gc
        gc.collect()
        torch.cuda.empty_cache()
    return out


def float32_check(cfg, seed, peaks):
    """The whole model in true 32-bit against the plain implementation on one short prompt, and
    the bfloat16 engine against the 32-bit engine (error and greedy token)."""
    import gc

    import torch

    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import plain_llama
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    from llm_b200.weights.loader import expected_tensors, random_tensor
    t0 = time.perf_counter()
    w = {}
    for name, info in expected_tensors(cfg).items():
        t = random_tensor(name, info, seed)
        w[name] = t.to(torch.bfloat16).float() if info.kind == "matrix" else t        # as a bfloat16 checkpoint stores them
    toks = [int(x) for x in torch.randint(0, cfg["vocab_size"], (24,), generator=torch.Generator().manual_seed(3))]
    ref = plain_llama.forward(cfg, w, toks, rows=[len(toks) - 1])[0]
    rows = {}
    for dtype in ("float32", "bfloat16"):
        eng = Engine(None, EngineOptions(dtype=dtype, kv_block_size=16, max_num_seqs=2, max_num_batched_tokens=64,
                                         max_seq_len=64, num_kv_blocks=8), random_config=cfg, tensors=w)
        rows[dtype] = eng.step([StepEntry("c", toks, [len(toks) - 1])])[0].double().cpu()
        eng.check_status()
        del eng
        gc.collect()
        torch.cuda.empty_cache()
    scale = float(ref.abs().max())
    return {"layers": cfg["num_hidden_layers"], "prompt_tokens": len(toks),
            "float32_vs_plain": float((rows["float32"] - ref).abs().max() / scale),
            "bfloat16_vs_float32": float((rows["bfloat16"] - rows["float32"]).abs().max() / scale),
            "top1_plain": int(ref.argmax()), "top1_float32": int(rows["float32"].argmax()),
            "top1_bfloat16": int(rows["bfloat16"].argmax()), "seconds": round(time.perf_counter() - t0, 1)}


def reference_arm(args, warmup: int) -> int:
    """The same measurements on the unmodified reference: its tree compiled with nvcc (it has no
    Python package to install) and driven through Scheduler -> PipelineDriver -> LLM::inference by
    baseline/ref_harness.cu, on the same seeded random checkpoint.  Nothing of llm_b200's engine or
    kernels runs in that process."""
    import shutil
    import tempfile

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    import reference_arm as ref

    def unavailable(why: str) -> int:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0

    if args.layers != FULL_LAYERS or args.batch > 64:
        return unavailable(f"the reference arm runs the full model at batch <= 64 (asked: {args.layers} layers, batch {args.batch})")
    peaks = load_peaks()
    folder = tempfile.mkdtemp(prefix="llm_b200_ref_")
    try:
        try:
            ref.build_harness()
            t0 = time.time()
            weights = ref.write_weights(folder, FULL_LAYERS, seed=20240531)
            write_s = time.time() - t0
        except ref.ReferenceUnavailable as e:
            return unavailable(str(e))
        out = {"metric": "decode tok/s at batch 8 (TinyLlama 1.1B shape, bf16, random weights)", "unit": "tok/s",
               "n_gpus": 1, "steps": args.steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak",
               "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights and token ids",
               "impl": "reference"}
        points, extra = {}, {}
        # the reference's own sizes (model/llm/tiny_llama.cpp:19): 8 sequences, 512 tokens per step.
        # Its driver keeps two batches in flight, so requests whose prompts ended in different
        # steps decode as two alternating groups (each reading every weight for part of the batch).
        with ref.Harness(weights, max_seqs=max(8, args.batch), max_tokens=512, max_seq_len=2048) as h:
            sampler = ClockSampler()
            sampler.start()
            stock = h.command(f"decode {args.batch} {PROMPT_LEN} {warmup} {args.steps}")
            clocks = sampler.stop()
            if "ms_per_step" not in stock:
                return unavailable("the reference's decode run failed: " + json.dumps(stock)[:200])
            load_s = h.ready.get("load_s")
            if not args.no_points:
                b1 = h.command(f"decode 1 {PROMPT_LEN} {warmup} {min(args.steps, 128)}")
                points["decode_b1"] = round(b1["tok_s_device"], 1) if "tok_s_device" in b1 else b1
                ld = h.command("load 32 128 128")       # its own benchmark (model/llm/test/bench_tiny_llama_load.cu:27-28)
                extra["shapes"] = {"load_32x128_128": dict(ld, max_num_seqs=8, chunk=512) if "tok_s" in ld else ld}
        head, mode = stock, "stock sizes (8 sequences, 512 tokens a step): two alternating groups in flight"
        # the same code with larger constructor arguments: every prompt of the batch in ONE step, so
        # that the batch decodes whole (and is waited for each step); batch 64; a 2,048-token step
        big_tokens = max(PREFILL_TOKENS, args.batch * PROMPT_LEN)
        with ref.Harness(weights, max_seqs=64, max_tokens=big_tokens, max_seq_len=2 * PREFILL_TOKENS) as h:
            whole = h.command(f"decode {args.batch} {PROMPT_LEN} {warmup} {args.steps}")
            points["decode_whole_batch"] = {k: whole.get(k) for k in ("tok_s_device", "tok_s_e2e", "ms_per_step", "batches_per_step")}
            points["decode_two_groups"] = {k: stock.get(k) for k in ("tok_s_device", "tok_s_e2e", "ms_per_step", "batches_per_step")}
            if whole.get("tok_s_e2e", 0) > stock["tok_s_e2e"]:
                head, mode = whole, f"all prompts in one step ({big_tokens} tokens a step): the batch decodes whole"
            if not args.no_points:
                b64 = h.command(f"decode 64 {PROMPT_LEN} {warmup} {min(args.steps, 128)}")
                points["decode_b64"] = round(b64["tok_s_device"], 1) if "tok_s_device" in b64 else b64
                pf = h.command(f"prefill {PREFILL_TOKENS} 2 5")
                if "ms" in pf:
                    fl = prefill_flops(MODEL, FULL_LAYERS, PREFILL_TOKENS, head_rows=PREFILL_TOKENS)
                    out["prefill"] = {"value": round(pf["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pf["ms"], 3),
                                      "frac": round(fl / (pf["ms"] / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                                      "peak_tflops": peaks["bf16_tflops"], "peak_source": peaks["source"],
                                      "note": "LM head on all rows, as the reference runs it"}
                else:
                    out["prefill"] = pf
        ms = head["ms_per_step"]
        mean_ctx = (head["ctx_min"] + head["ctx_max"]) / 2.0 - args.steps / 2.0
        step_bytes = decode_bytes(MODEL, FULL_LAYERS, args.batch, args.batch * mean_ctx)
        achieved = step_bytes / (ms / 1e3) / 1e9
        out.update({"value": round(args.batch / (ms / 1e3), 1), "ms_per_step": round(ms, 4),
                    "ms_per_step_with_gaps": round(head["ms_per_step_span"], 4), "clocks": clocks,
                    "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                                 "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
                                 "bytes_per_step": int(step_bytes)},
                    "e2e": {"value": round(head["tok_s_e2e"], 1), "unit": "tok/s",
                            "h2d_bytes_per_step": head["h2d_bytes_per_step"], "d2h_bytes_per_step": head["d2h_bytes_per_step"],
                            "decode_steps": args.steps},
                    "points": points})
        out.update(extra)
        out["config"] = {"model": "TinyLlama-1.1B shape", "layers": FULL_LAYERS, "layers_full": FULL_LAYERS,
                         "hidden": MODEL["hidden_size"], "heads": MODEL["num_attention_heads"],
                         "kv_heads": MODEL["num_key_value_heads"], "head_dim": MODEL["head_dim"],
                         "intermediate": MODEL["intermediate_size"], "vocab": MODEL["vocab_size"],
                         "global_batch": args.batch, "prompt_len": PROMPT_LEN, "new_tokens": args.steps,
                         "seq_len": MODEL["max_position_embeddings"], "kv_block": 16, "parallelism": "none (1 GPU)",
                         "l2": "inputs larger than L2 (2.2 GB of weights per step)", "cuda_graphs": True,
                         "load_s": load_s, "reference_mode": mode}
        out["build"] = "nvcc -O3 -std=c++17 sm_100a on a verbatim copy of the reference (baseline/_ref)"
        out["ctx_at_end"] = [head["ctx_min"], head["ctx_max"]]
        out["checkpoint_write_s"] = round(write_s, 1)
        print(json.dumps(out))
        return 0
    finally:
        shutil.rmtree(folder, ignore_errors=True)


def decode_attention_sweep(args, peaks, torch, ops) -> int:
    """The decode attention kernel alone: one query token per request over `ctx` cached keys, pages
    in shuffled order, several sets of pages in turn so that no launch finds its keys in L2; timed
    as one CUDA graph of all launches.  Bytes are the keys and values that a launch has to read."""
    import math
    n_heads, n_kv, hs = (int(x) for x in args.heads.split(","))
    page, dev = 16, "cuda:0"
    cases = [(args.batch, args.ctx)] if args.ctx else [(b, c) for b in (1, 8, 64) for c in (512, 2048, 8192, 32768)
                                                       if b * c * 4 * n_kv * hs <= 2.2e9]
    print(f"decode attention, {n_heads} query heads, {n_kv} kv heads, head size {hs}, pages of {page}; "
          f"peak {peaks['hbm_gbs']:.0f} GB/s ({peaks['source']})")
    for batch, ctx in cases:
        per_req = -(-ctx // page)
        nbytes = batch * ctx * 4 * n_kv * hs
        sets = min(64, max(2, math.ceil(300e6 / nbytes)))
        k_pages = torch.randn(sets * batch * per_req, n_kv, page, hs, device=dev, dtype=torch.bfloat16)
        v_pages = torch.randn_like(k_pages)
        tables = torch.randperm(sets * batch * per_req, device=dev).to(torch.int32).view(sets, batch, per_req).contiguous()
        kv_lens = torch.full((batch,), ctx, dtype=torch.int32, device=dev)
        q = torch.randn(batch, n_heads * hs, device=dev, dtype=torch.bfloat16)
        out = torch.empty_like(q)
        call = lambda i: ops.paged_attention_decode(out, q, k_pages, v_pages, tables[i % sets], kv_lens, batch, n_heads, n_kv,
                                                    hs, 0, 1.0 / math.sqrt(hs), max_keys=ctx)
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        n = max(sets, 8)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                call(i)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); graph.replay(); b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / n * 1e3
        gbs = nbytes / us / 1e3
        print(f"batch {batch:3d} context {ctx:6d} ranges {ops.decode_splits(batch, n_kv, ctx):2d}: {us:8.1f} us a launch, "
              f"{nbytes / 1e6:7.1f} MB, {gbs:7.1f} GB/s = {gbs / peaks['hbm_gbs']:.2f} of the peak")
        del k_pages, v_pages, tables
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=NEW_TOKENS)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS)
    ap.add_argument("--no-points", action="store_true", help="skip prefill and the batch 1 / 64 points")
    ap.add_argument("--no-shapes", action="store_true",
                    help="skip the runs at the Llama-2-7B and Llama-3-8B shapes, the many-request load and the 32-bit check")
    ap.add_argument("--mode", default="all",
                    choices=["all", "decode", "prefill", "timeline", "timeline_prefill", "decode_attention"],
                    help="decode / prefill: only that measurement, for small profiling runs (not the benchmark line); "
                         "timeline: the kernels of one decode layer with their start and end inside the step's CUDA graph; "
                         "decode_attention: the decode attention kernel alone over batches and context lengths "
                         "(--batch with --ctx: that one case)")
    ap.add_argument("--ctx", type=int, default=0, help="decode_attention: the context length of the one case to run")
    ap.add_argument("--prompt-tokens", type=int, default=PREFILL_TOKENS, help="timeline_prefill: tokens of the prompt step")
    ap.add_argument("--heads", default="32,4,64", help="decode_attention: query heads, kv heads, head size")
    args = ap.parse_args()

    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return reference_arm(args, warmup)

    import numpy as np
    import torch

    from llm_b200.csrc import ops
    from llm_b200.engine.engine import StepEntry
    from llm_b200.engine.llm import LLM

    peaks = load_peaks()
    if args.mode == "decode_attention":
        return decode_attention_sweep(args, peaks, torch, ops)
    cfg = dict(MODEL, num_hidden_layers=args.layers)
    if args.mode != "all":
        args.no_points = True
    max_batch = max(64, args.batch) if not args.no_points else args.batch
    t_load = time.time()
    # a token budget that takes the whole batch's prompts in one step, so that in the end-to-end run
    # every request starts to decode in the same step and the batch stays whole to the last token
    llm = LLM(None, dtype="bfloat16", max_num_seqs=max_batch, max_num_batched_tokens=max(PREFILL_TOKENS, args.batch * PROMPT_LEN),
              max_seq_len=MODEL["max_position_embeddings"], eos_token_id=-1, kv_block_size=16,
              random_config=cfg, random_seed=20240531)
    eng = llm.engine
    use_graphs = eng.options.use_cuda_graphs
    load_s = time.time() - t_load
    rng = np.random.default_rng(1)

    def prompt(n):
        return [int(x) for x in rng.integers(0, cfg["vocab_size"], size=n)]

    def prefill_requests(batch):
        """Put `batch` requests of PROMPT_LEN tokens into the cache, a few per step."""
        ids = [f"b{batch}_{i}" for i in range(batch)]
        per_step = PREFILL_TOKENS // PROMPT_LEN
        for i in range(0, batch, per_step):
            eng.step([StepEntry(r, prompt(PROMPT_LEN), []) for r in ids[i:i + per_step]])
        return ids

    def timed_decode(batch, steps, warm):
        """Device time of `steps` decode steps of `batch` requests (tokens are given, nothing is
        read back inside the region).  Returns (ms per step, launches per step, context at the end)."""
        ids = prefill_requests(batch)
        toks = rng.integers(0, cfg["vocab_size"], size=(warm + steps, batch))
        entries = lambda k: [StepEntry(r, [int(toks[k, j])], [0]) for j, r in enumerate(ids)]
        for k in range(warm):
            eng.step(entries(k))
        torch.cuda.synchronize()
        l0 = ops.launch_count()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for k in range(warm, warm + steps):
            eng.step(entries(k))
        stop.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(stop) / steps
        launches = (ops.launch_count() - l0) / steps
        ctx_end = PROMPT_LEN + warm + steps
        for r in ids:
            eng.release(r)
        return ms, launches, ctx_end

    out = {"metric": "decode tok/s at batch 8 (TinyLlama 1.1B shape, bf16, random weights)", "unit": "tok/s",
           "n_gpus": 1, "steps": args.steps, "warmup": warmup, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "bf16", "data": "synthetic: seeded random weights and token ids",
           "impl": "ours"}

    if args.mode == "prefill":
        reps = []
        for k in range(max(3, args.steps)):
            rid = f"p{k}"
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([StepEntry(rid, prompt(PREFILL_TOKENS), [PREFILL_TOKENS - 1])])
            b.record()
            torch.cuda.synchronize()
            reps.append(a.elapsed_time(b))
            eng.release(rid)
        print(json.dumps({"mode": "prefill", "layers": args.layers, "tokens": PREFILL_TOKENS, "ms": reps}))
        return 0
    if args.mode in ("timeline", "timeline_prefill"):
        # When each kernel of a step starts and ends inside the replayed CUDA graph (CUPTI through
        # torch.profiler): the kernels overlap (programmatic dependent launch), so the step's time
        # is the chain of their ENDS, not the sum of their durations.  timeline: a decode step of
        # --batch requests; timeline_prefill: a prompt of PREFILL_TOKENS tokens in one step.
        import collections

        from torch.profiler import ProfilerActivity, profile
        if args.mode == "timeline":
            ids = prefill_requests(args.batch)
            toks = rng.integers(0, cfg["vocab_size"], size=(warmup + 4, args.batch))
            entries = lambda k: [StepEntry(r, [int(toks[k, j])], [0]) for j, r in enumerate(ids)]
            run = lambda k: eng.step(entries(k))
        else:
            def run(k):
                eng.step([StepEntry(f"p{k}", prompt(args.prompt_tokens), [args.prompt_tokens - 1])])
                eng.release(f"p{k}")
        for k in range(warmup):
            run(k)
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for k in range(warmup, warmup + 4):
                run(k)
            torch.cuda.synchronize()
        on_gpu = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.name]
        evs = [e for e in on_gpu if "Memcpy" not in e.name and "Memset" not in e.name]
        evs.sort(key=lambda e: e.time_range.start)
        per_step = len(evs) // 4
        step = evs[2 * per_step:3 * per_step]
        span = step[-1].time_range.end - step[0].time_range.start
        # what lies between two steps launched back to back: the copies and fills of the step, the graph's start
        gap0, gap1 = evs[2 * per_step - 1].time_range.end, step[0].time_range.start
        between = [e for e in on_gpu if gap0 <= e.time_range.start < gap1 and ("Memcpy" in e.name or "Memset" in e.name)]
        print(f"{gap1 - gap0:.1f} us from the last end of the step before to this step's first start; in between: "
              + ", ".join(f"{e.name.split('(')[0].strip()} {e.time_range.start - gap0:.1f}..{e.time_range.end - gap0:.1f}" for e in between))
        what = f"batch {args.batch}" if args.mode == "timeline" else f"prompt of {args.prompt_tokens} tokens"
        print(f"{what}, {args.layers} layers: {per_step} kernels a step, {span:.1f} us from the first start to the last end")
        agg = collections.OrderedDict()
        prev_end = None
        for e in step:
            name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:48]
            gain = e.time_range.end - (prev_end if prev_end is not None else e.time_range.start)
            prev_end = max(prev_end or 0, e.time_range.end)
            d = agg.setdefault(name, [0, 0.0, 0.0])
            d[0] += 1; d[1] += e.time_range.end - e.time_range.start; d[2] += max(gain, 0.0)
        print(f"{'kernel':50s} {'launches':>8s} {'mean duration us':>17s} {'end after previous end us (sum)':>32s}")
        for name, (n, dur, gain) in agg.items():
            print(f"{name:50s} {n:8d} {dur / n:17.2f} {gain:32.1f}")
        base = step[0].time_range.start
        first = min(9, per_step - 1)
        print("the second layer, microseconds from the step's first kernel: start .. end")
        for e in step[first:first + 9]:
            name = e.name.replace("(anonymous namespace)::", "").replace("void ", "").split("(")[0][:60]
            print(f"  {e.time_range.start - base:9.2f} .. {e.time_range.end - base:9.2f}  {name}")
        return 0
    if args.mode == "decode":
        ms, launches, _ = timed_decode(args.batch, args.steps, warmup)
        print(json.dumps({"mode": "decode", "layers": args.layers, "batch": args.batch, "ms_per_step": ms,
                          "launches_per_step": launches}))
        return 0

    # ---- headline: decode at the default batch, device-timed ----
    sampler = ClockSampler()
    sampler.start()
    ms, launches, ctx_end = timed_decode(args.batch, args.steps, warmup)
    clocks = sampler.stop()
    value = args.batch / (ms / 1e3)
    mean_ctx = PROMPT_LEN + warmup + (args.steps + 1) / 2.0
    step_bytes = decode_bytes(cfg, args.layers, args.batch, args.batch * mean_ctx)
    achieved = step_bytes / (ms / 1e3) / 1e9
    out.update({"value": round(value, 1), "ms_per_step": round(ms, 4), "gpu_launches": int(round(launches * args.steps)),
                "clocks": clocks,
                "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": round(achieved / peaks["hbm_gbs"], 4), "peak_source": peaks["source"],
                             "bytes_per_step": int(step_bytes)}})

    # ---- end to end: the same decode through LLM.generate, host tokens in and out ----
    prompts = [prompt(PROMPT_LEN) for _ in range(args.batch)]
    llm.generate(prompts, max_new_tokens=args.steps + 1)             # warm-up: the same shapes, so that their graphs exist
    gen = llm.generate(prompts, max_new_tokens=args.steps + 1)
    st = llm.last_stats
    e2e_value = st["decode_tokens"] / st["decode_seconds"] if st["decode_seconds"] > 0 else None
    out["e2e"] = {"value": round(e2e_value, 1) if e2e_value else None, "unit": "tok/s",
                  "h2d_bytes_per_step": int(st["h2d_bytes_per_step"]), "d2h_bytes_per_step": int(st["d2h_bytes_per_step"]),
                  "decode_steps": st["decode_steps"], "generated": sum(len(g) for g in gen),
                  "host_us_per_step": {k[:-8]: round(st[k] / max(st["steps"], 1) * 1e6, 1)
                                       for k in ("sched_seconds", "launch_seconds", "wait_seconds", "update_seconds")}}

    # ---- prefill of 2,048 tokens ----
    if not args.no_points:
        reps = []
        for k in range(5):
            rid = f"p{k}"
            tokens = prompt(PREFILL_TOKENS)              # the request's token ids exist before the step is asked for
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            eng.step([StepEntry(rid, tokens, [PREFILL_TOKENS - 1])])
            b.record()
            torch.cuda.synchronize()
            reps.append(a.elapsed_time(b))
            eng.release(rid)
        pms = sorted(reps[2:])[len(reps[2:]) // 2]
        fl = prefill_flops(cfg, args.layers, PREFILL_TOKENS)
        out["prefill"] = {"value": round(PREFILL_TOKENS / (pms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(pms, 3),
                          "frac": round(fl / (pms / 1e3) / (peaks["bf16_tflops"] * 1e12), 4),
                          "peak_tflops": peaks["bf16_tflops"], "peak_source": peaks["source"]}
        points = {}
        for b in (1, 64):
            pm, _, _ = timed_decode(b, min(args.steps, 128), warmup)
            points[f"decode_b{b}"] = round(b / (pm / 1e3), 1)
        out["points"] = points

    out["counters"] = dict(eng.counters, preemptions=llm.last_stats.get("preemptions", 0),
                           free_pages=[eng.cache.num_free_pages(g) for g in range(eng.cache.num_groups)],
                           pages=[eng.cache.group_spec(g).num_pages for g in range(eng.cache.num_groups)])

    # ---- the other workloads of the benchmark definition, each through LLM.generate and the scheduler ----
    if not (args.no_points or args.no_shapes) and args.layers == FULL_LAYERS:
        shapes = {}

        def attempt(name, fn):
            try:
                shapes[name] = fn()
            except Exception as e:                   # a shape that cannot run here must not take the headline with it
                shapes[name] = {"error": f"{type(e).__name__}: {str(e)[:200]}"}

        # the reference's own load (model/llm/test/bench_tiny_llama_load.cu:27-28): 32 requests of
        # 128 + 128 tokens, at most 8 live, 512 tokens a step
        attempt("load_32x128_128", lambda: generate_point(cfg, [prompt(128) for _ in range(32)], 128, 8, 512, peaks, llm=llm))
        del llm, eng
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        # Llama-2-7B shape: 32 requests, prompts of 128 to 2,048 tokens, 128 new tokens each, one mixed batch
        lens7 = [int(x) for x in rng.integers(128, 2049, size=32)]
        attempt("llama2_7b_mixed", lambda: generate_point(
            LLAMA2_7B, [[int(x) for x in rng.integers(0, 32000, size=n)] for n in lens7], 128, 32, 2048, peaks))
        # Llama-3-8B shape: 8 requests of 8,000 tokens taken 2,048 a step, then 256 new tokens at batch 8
        attempt("llama3_8b_long", lambda: generate_point(
            LLAMA3_8B, [[int(x) for x in rng.integers(0, 128256, size=8000)] for _ in range(8)], 256, 8, 2048, peaks))
        attempt("float32_check", lambda: float32_check(dict(MODEL), 20240531, peaks))
        out["shapes"] = shapes

    out["config"] = {"model": "TinyLlama-1.1B shape", "layers": args.layers, "layers_full": FULL_LAYERS,
                     "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                     "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                     "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                     "global_batch": args.batch, "prompt_len": PROMPT_LEN, "new_tokens": args.steps,
                     "seq_len": MODEL["max_position_embeddings"], "kv_block": 16, "parallelism": "none (1 GPU)",
                     "l2": "inputs larger than L2 (2.2 GB of weights per step)", "cuda_graphs": use_graphs,
                     "load_s": round(load_s, 1)}
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
