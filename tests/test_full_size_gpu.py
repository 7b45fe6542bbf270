"""The layer sizes of the benchmark's model (TinyLlama 1.1B: hidden 2048, 32 query and 4 kv
heads of 64, intermediate 5632, vocabulary 32000), three layers of it with seeded random
weights, against the plain implementation: the kernels at the sizes they are measured at,
in 32-bit and in bfloat16, prompt portions and single tokens."""
import pytest
import torch

import plain_llama
from tiny import TOL, random_tokens

pytestmark = pytest.mark.gpu

CONFIG = dict(architectures=["LlamaForCausalLM"], hidden_size=2048, intermediate_size=5632, num_hidden_layers=3,
              num_attention_heads=32, num_key_value_heads=4, vocab_size=32000, rms_norm_eps=1e-5, rope_theta=10000.0,
              max_position_embeddings=2048, tie_word_embeddings=False)


@pytest.fixture(scope="module")
def reference():
    from llm_b200.weights.loader import expected_tensors, random_tensor
    toks = random_tokens(300, CONFIG["vocab_size"], 5)
    w = {}
    for name, info in expected_tensors(CONFIG).items():
        t = random_tensor(name, info, 0)
        w[name] = t.to(torch.bfloat16).float() if info.kind == "matrix" else t      # as stored: matrices in bfloat16
    return toks, plain_llama.forward(CONFIG, w, toks)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_match_plain(reference, dtype):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    toks, ref = reference
    eng = Engine(None, EngineOptions(dtype=dtype, kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=512,
                                     max_seq_len=512, num_kv_blocks=40), random_config=CONFIG, random_seed=0)
    # a portion of more than 128 rows (the many-row products and the tcgen05 attention), a short
    # one (the swapped products), then single tokens (the decode kernels, replayed from a graph)
    rows = [eng.step([StepEntry("a", toks[:200], list(range(200)))]).double().cpu().clone(),
            eng.step([StepEntry("a", toks[200:270], list(range(70)))]).double().cpu().clone()]
    for t in toks[270:]:
        rows.append(eng.step([StepEntry("a", [t], [0])]).double().cpu().clone())
    got = torch.cat(rows)
    err = (got - ref).abs().max(dim=1).values / ref.abs().max()
    bad = torch.nonzero(err > TOL[dtype])
    assert bad.numel() == 0, f"first differing position {int(bad[0])}: {float(err[int(bad[0])]):.3e}"
    eng.check_status()
