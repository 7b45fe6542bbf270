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


# ---- the shapes that the benchmark times, two layers of them, against the plain implementation ----

CONFIG2 = dict(CONFIG, num_hidden_layers=2)


@pytest.fixture(scope="module")
def weights2():
    from llm_b200.weights.loader import expected_tensors, random_tensor
    w = {}
    for name, info in expected_tensors(CONFIG2).items():
        t = random_tensor(name, info, 3)
        w[name] = t.to(torch.bfloat16).float() if info.kind == "matrix" else t
    return w


def _engine2(dtype, **kw):
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    opts = dict(dtype=dtype, kv_block_size=16, max_num_seqs=4, max_num_batched_tokens=2048, max_seq_len=2048,
                num_kv_blocks=140, poison_freed_pages=True)
    opts.update(kw)
    return Engine(None, EngineOptions(**opts), random_config=CONFIG2, random_seed=3)


def _check_rows(got, ref, dtype, what):
    err = (got.double().cpu() - ref).abs().max(dim=1).values / ref.abs().max()
    bad = torch.nonzero(err > TOL[dtype])
    assert bad.numel() == 0, f"{what}: first differing row {int(bad[0])}: {float(err[int(bad[0])]):.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_step_of_2048_rows_then_decoding_past_1024_keys(weights2, dtype):
    """The prefill the benchmark times (2,048 rows in one step: the pair kernels with rotation in
    the epilogue over 8 row tiles, the whole attention grid), and decoding with more than 1,024
    keys behind it (several ranges per request, the graph of a longer key bucket)."""
    from llm_b200.engine.engine import StepEntry
    toks = random_tokens(2048, CONFIG2["vocab_size"], 11)
    want = sorted(set([0, 1, 15, 16, 127, 128, 129, 255, 256, 1023, 1024, 1025, 2046, 2047] + list(range(40, 2048, 97))))
    ref = plain_llama.forward(CONFIG2, weights2, toks, rows=want)
    eng = _engine2(dtype)
    _check_rows(eng.step([StepEntry("p", toks, want)]), ref, dtype, "2,048 rows in one step")
    eng.release("p")
    # 1,500 tokens in portions of 512, then single tokens from position 1,500 on
    head, tail = 1500, 24
    ref_tail = plain_llama.forward(CONFIG2, weights2, toks[:head + tail], rows=range(head - 1, head + tail))
    rows = []
    for a in range(0, head, 512):
        part = toks[a:min(a + 512, head)]
        out = eng.step([StepEntry("q", part, [len(part) - 1] if a + 512 >= head else [])])
        if out.shape[0]:
            rows.append(out.double().cpu().clone())
    for t in toks[head:head + tail]:
        rows.append(eng.step([StepEntry("q", [t], [0])]).double().cpu().clone())
    _check_rows(torch.cat(rows), ref_tail, dtype, "decoding past 1,024 keys")
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_decode_batch_of_64(weights2, dtype):
    """64 requests of ragged lengths decoded together (the products' 64-row tile, one range per
    request in the attention), prompts taken 16 requests a step."""
    from llm_b200.engine.engine import StepEntry
    lens = [3 + (7 * i) % 45 for i in range(64)]
    reqs = [random_tokens(n + 3, CONFIG2["vocab_size"], 500 + i) for i, n in enumerate(lens)]
    eng = _engine2(dtype, max_num_seqs=64, num_kv_blocks=64 * 4 + 2)
    for a in range(0, 64, 16):
        eng.step([StepEntry(i, reqs[i][:lens[i]], []) for i in range(a, a + 16)])
    got = [eng.step([StepEntry(i, [reqs[i][lens[i] + k]], [0]) for i in range(64)]).double().cpu().clone() for k in range(3)]
    for i in range(64):
        ref = plain_llama.forward(CONFIG2, weights2, reqs[i], rows=range(lens[i], lens[i] + 3))
        _check_rows(torch.stack([g[i] for g in got]), ref, dtype, f"request {i} of {lens[i]} tokens")
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_with_pages_used_again(weights2, dtype):
    """Up to four live requests, portions of some beside decoded tokens of others, a pool that
    holds four requests at most, freed pages poisoned."""
    import replay
    lens = [130, 300, 47, 260, 90, 200]
    reqs = {f"r{i}": random_tokens(n, CONFIG2["vocab_size"], 700 + i) for i, n in enumerate(lens)}
    pool = sum(-(-n // 16) for n in sorted(lens, reverse=True)[:4]) + 1
    eng = _engine2(dtype, num_kv_blocks=pool, max_num_batched_tokens=512, use_cuda_graphs=False)
    got = replay.run_steps(eng, replay.steps_mixed(reqs, prefill_sizes=(150, 2, 24, 130)))
    for rid, toks in reqs.items():
        _check_rows(got[rid], plain_llama.forward(CONFIG2, weights2, toks), dtype, f"mixed, request {rid}")
    eng.cache.check()
    eng.check_status()
