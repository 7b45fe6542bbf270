"""The plain implementation (and the engine) against the reference's own model on the GPU.

The reference (zhan-wei-919/llm) runs one shape, TinyLlama 1.1B in bfloat16, so this test writes
two layers of that width with seeded random weights (every tensor in bfloat16, which is what
the reference's loader expects), lets the unmodified reference compute the logits at the last
row of three prompts (baseline/ref_harness.cu, built by nvcc against a verbatim copy of its
tree), and compares them with tests/plain_llama.py on the same weights and with the bfloat16
engine.  Skipped where no copy of the reference tree can be had."""
import os
import sys

import numpy as np
import pytest
import torch

import plain_llama
from tiny import random_tokens

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "baseline"))

LAYERS = 2
PROMPT_LENGTHS = (7, 61, 200)       # one tile, a ragged tile, several tiles of the reference's kernels


@pytest.fixture(scope="module")
def reference_logits(tmp_path_factory):
    import reference_arm as ref
    try:
        ref.build_harness()
    except ref.ReferenceUnavailable as e:
        pytest.skip(str(e))
    folder = str(tmp_path_factory.mktemp("ref_model"))
    weights = ref.write_weights(folder, LAYERS, seed=77)
    cfg = dict(ref.MODEL, num_hidden_layers=LAYERS)
    prompts = [random_tokens(n, cfg["vocab_size"], 100 + n) for n in PROMPT_LENGTHS]
    rows = []
    with ref.Harness(weights, max_seqs=8, max_tokens=512, max_seq_len=2048, layers=LAYERS, timeout=300) as h:
        for i, p in enumerate(prompts):
            path = os.path.join(folder, f"logits_{i}.f32")
            answer = h.command("logits " + path + " " + " ".join(str(t) for t in p))
            assert answer.get("mode") == "logits" and "refused" not in answer and "error" not in answer, answer
            rows.append((torch.from_numpy(np.fromfile(path, dtype=np.float32).astype(np.float64)), answer["next_token"]))
    return folder, cfg, prompts, rows


def test_plain_implementation_matches_the_reference_model(reference_logits):
    from llm_b200.weights.safetensors_io import SafetensorsFile
    folder, cfg, prompts, rows = reference_logits
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    w = {n: f.tensor(n).clone() for n in f.names()}
    for p, (got, token) in zip(prompts, rows):
        want = plain_llama.forward(cfg, w, p)[-1]
        # the reference rounds every activation, its residual stream and its logits to bfloat16
        # (8 bits of mantissa): the same bound as the engine's bfloat16 path
        err = float((got - want).abs().max() / want.abs().max())
        assert err < 3e-2, (len(p), err)
        # its greedy token is the plain implementation's, or one whose logit is within that bound of it
        assert float(want.max() - want[token]) <= 3e-2 * float(want.abs().max())


def test_engine_matches_the_reference_model(reference_logits):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    folder, cfg, prompts, rows = reference_logits
    eng = Engine(folder, EngineOptions(dtype="bfloat16", kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=512,
                                       max_seq_len=512, num_kv_blocks=64))
    for i, (p, (ref_row, _)) in enumerate(zip(prompts, rows)):
        got = eng.step([StepEntry(f"r{i}", p, [len(p) - 1])])[0].double().cpu()
        eng.release(f"r{i}")
        err = float((got - ref_row).abs().max() / ref_row.abs().max())
        assert err < 3e-2, (len(p), err)
    eng.check_status()
