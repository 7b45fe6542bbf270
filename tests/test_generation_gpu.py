"""Generation through the Python entry point and the command line: long decoding, the first
tokens of a sequence, temperature sampling against the plain sampler, running out of pages,
CUDA graphs on and off."""
import os
import random
import subprocess
import sys

import pytest
import torch

import plain_llama as pl
from tiny import CONFIGS, TOL, load_plain_weights, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    root = tmp_path_factory.mktemp("gen")
    return lambda name, dtype: make_model_dir(root, name, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_long_decode_and_first_tokens(folders, name, dtype):
    """Three prompt tokens, then 180 tokens decoded one by one across many pages; every step's
    logits against the plain implementation, the first positions included."""
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    cfg, page = CONFIGS[name]
    d = folders(name, dtype)
    w = load_plain_weights(d)
    toks = random_tokens(183, cfg["vocab_size"], 77)
    ref = pl.forward(cfg, w, toks)
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=2, max_num_batched_tokens=64,
                                  num_kv_blocks=-(-183 // page) + 1, use_cuda_graphs=True))
    rows = [eng.step([StepEntry("x", toks[:3], [0, 1, 2])]).double().cpu().clone()]
    for t in toks[3:]:
        rows.append(eng.step([StepEntry("x", [t], [0])]).double().cpu().clone())
    got = torch.cat(rows)
    err = (got - ref).abs().max(dim=1).values / ref.abs().max()
    bad = torch.nonzero(err > TOL[dtype])
    assert bad.numel() == 0, f"first differing position {int(bad[0])}: {float(err[int(bad[0])]):.3e}"
    assert eng.counters["graph_replays"] > 100


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_matches_plain_sampler(folders, dtype):
    from llm_b200 import LLM
    cfg, page = CONFIGS["B"]
    d = folders("B", dtype)
    w = load_plain_weights(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 900 + n) for n in (1, 40, 64, 97)]
    llm = LLM(d, dtype=dtype, max_num_seqs=4, max_num_batched_tokens=24, kv_block_size=page, num_kv_blocks=64,
              eos_token_id=-1)
    got = llm.generate(prompts, max_new_tokens=12, temperature=0.8, seed=5)
    again = llm.generate(prompts, max_new_tokens=12, temperature=0.8, seed=5)
    other = llm.generate(prompts, max_new_tokens=12, temperature=0.8, seed=6)
    assert got == again and got != other
    for rid, (p, g) in enumerate(zip(prompts, got)):
        ids = list(p)
        for tok in g:
            row = pl.forward(cfg, w, ids)[-1]
            u = pl.uniform_for(5, rid, len(ids))
            want = pl.sample_temperature(row, 0.8, u)
            if tok != want:
                # only a draw within rounding of a boundary of the cumulative distribution may differ
                c = torch.cumsum(torch.softmax(row / 0.8, -1), -1)
                edge = min(abs(u - float(c[min(tok, want)])), abs(u - float(c[max(tok, want) - 1])))
                assert abs(tok - want) == 1 and edge < (1e-5 if dtype == "float32" else 2e-2), (rid, len(ids), tok, want)
            ids.append(tok)


def test_running_out_of_pages_preempts_and_still_matches(folders):
    """A pool too small for all requests at once: decoding preempts and recomputes, and greedy
    output still equals the plain implementation's."""
    from llm_b200 import LLM
    cfg, page = CONFIGS["A"]
    d = folders("A", "float32")
    w = load_plain_weights(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 40 + n) for n in (30, 29, 31, 12)]
    llm = LLM(d, dtype="float32", max_num_seqs=4, max_num_batched_tokens=32, kv_block_size=page, num_kv_blocks=8,
              eos_token_id=-1, use_cuda_graphs=False)
    got = llm.generate(prompts, max_new_tokens=28)
    assert llm.last_num_preemptions > 0
    for p, g in zip(prompts, got):
        assert g == pl.greedy_generate(cfg, w, p, 28)
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages(0) == 8


def test_cuda_graphs_change_nothing_and_eos_stops(folders):
    from llm_b200 import LLM
    cfg, page = CONFIGS["D"]
    d = folders("D", "bfloat16")
    prompts = [random_tokens(n, cfg["vocab_size"], 70 + n) for n in (9, 50, 3)]
    a = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=40, eos_token_id=-1,
            use_cuda_graphs=True).generate(prompts, max_new_tokens=20)
    llm = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=40, eos_token_id=-1,
              use_cuda_graphs=False)
    b = llm.generate(prompts, max_new_tokens=20)
    assert a == b
    # stop at a token: the first request's fifth token as eos
    eos = b[0][4]
    first = b[0].index(eos)
    llm2 = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=40, eos_token_id=eos,
               use_cuda_graphs=False)
    c = llm2.generate(prompts[:1], max_new_tokens=20)
    assert c[0] == b[0][:first + 1]


def test_command_line(folders, tmp_path):
    d = folders("A", "float32")
    w = load_plain_weights(d)
    cfg, _ = CONFIGS["A"]
    prompts = [[5, 17, 3, 200], [1, 2, 3, 4, 5, 6, 7, 8, 9]]
    text = "\n".join(" ".join(str(t) for t in p) for p in prompts) + "\n"
    proc = subprocess.run([sys.executable, "-m", "llm_b200", "--model", d, "--dtype", "float32", "--max-new-tokens", "6",
                           "--eos-token-id", "-1", "--num-kv-blocks", "16", "--max-num-seqs", "2",
                           "--max-num-batched-tokens", "16"], input=text, capture_output=True, text=True, cwd=ROOT,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = dict(l.split(": ") for l in proc.stdout.strip().split("\n"))
    for i, p in enumerate(prompts):
        assert [int(x) for x in lines[str(i)].split()] == pl.greedy_generate(cfg, w, p, 6)
    # the same requests named on the command line and in a file instead of standard input
    listed = tmp_path / "prompts.txt"
    listed.write_text(" ".join(str(t) for t in prompts[1]) + "\n")
    proc = subprocess.run([sys.executable, "-m", "llm_b200", "--model", d, "--dtype", "float32", "--max-new-tokens", "6",
                           "--eos-token-id", "-1", "--num-kv-blocks", "16", "--max-num-seqs", "2",
                           "--prompt-ids", ",".join(str(t) for t in prompts[0]), "--prompt-file", str(listed)],
                          stdin=subprocess.DEVNULL, capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert dict(l.split(": ") for l in proc.stdout.strip().split("\n")) == lines


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_lookahead_changes_nothing(folders, dtype):
    """Launching a decode step before the previous step's tokens are read gives the same tokens,
    also when a request ends on a token and when sampling with a temperature."""
    from llm_b200 import LLM
    cfg, page = CONFIGS["D"]
    d = folders("D", dtype)
    prompts = [random_tokens(n, cfg["vocab_size"], 170 + n) for n in (9, 50, 3, 130)]
    mk = lambda la, eos: LLM(d, dtype=dtype, max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=60,
                             eos_token_id=eos, lookahead=la)
    base = mk(False, -1).generate(prompts, max_new_tokens=24)
    llm = mk(True, -1)
    assert llm.generate(prompts, max_new_tokens=24) == base
    assert llm.last_stats["lookahead_steps"] >= 20
    eos = base[1][6]
    assert mk(True, eos).generate(prompts, max_new_tokens=24) == mk(False, eos).generate(prompts, max_new_tokens=24)
    assert mk(True, -1).generate(prompts, max_new_tokens=12, temperature=0.7, seed=2) == \
        mk(False, -1).generate(prompts, max_new_tokens=12, temperature=0.7, seed=2)
    llm.engine.cache.check()


def _same_or_near_tie(cfg, w, prompts, got, want):
    """Two bfloat16 runs that batch the same requests differently (other kernels, other split counts)
    may part ways at a near-tie: the first differing token must be one of the plain logits."""
    for p, g, wnt in zip(prompts, got, want):
        assert len(g) == len(wnt)
        if g != wnt:
            k = next(i for i, (a, b) in enumerate(zip(g, wnt)) if a != b)
            row = pl.forward(cfg, w, list(p) + g[:k])[-1]
            assert abs(float(row[g[k]] - row[wnt[k]])) <= TOL["bfloat16"] * float(row.abs().max()), (k, g[k], wnt[k])


def test_a_given_up_wait_is_reported_by_the_step_function(folders):
    """The tensor-core kernels bound their waits; one that gives up stores a code in a word of the
    engine's status block and writes zeros.  The word is set here from the host (no kernel is made
    to wait): check_status, generate and the server's emit then refuse to pass tokens on."""
    from llm_b200 import LLM
    from llm_b200.csrc import ops
    from llm_b200.engine.engine import StepError
    cfg, page = CONFIGS["D"]
    llm = LLM(folders("D", "bfloat16"), dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=40,
              eos_token_id=-1)
    eng = llm.engine
    prompts = [random_tokens(20, cfg["vocab_size"], 3)]
    assert len(llm.generate(prompts, max_new_tokens=4)[0]) == 4          # a clean run raises nothing
    # the word the product kernels are given while this engine steps is a word of its status block
    eng.status[1] = 8
    ops.set_error_block(eng.status)
    try:
        assert ops.gemm_tc_take_error() == 8 and int(eng.status[1]) == 0
    finally:
        ops.set_error_block(None)
    eng.status[1] = 5
    with pytest.raises(StepError, match="tensor-core product .persistent kernel.*MMA issuer"):
        eng.check_status()
    eng.check_status()                                                    # reported once, then clear
    eng.status[2] = 12
    with pytest.raises(StepError, match="tensor-core attention.*key/value tile"):
        llm.generate(prompts, max_new_tokens=2)
    eng.status[2] = 13
    emitted = []
    feed = iter(prompts)
    with pytest.raises(StepError, match="the scores"):
        llm.server(lambda wait: next(feed, None), lambda rid, toks: emitted.append(toks), max_new_tokens=3)
    assert emitted == []


def test_server_runs_ahead_like_generate(folders):
    """The serving loop (what the command line runs) launches decode steps one ahead of the host,
    as generate does, and emits the same tokens; requests that arrive while others decode join."""
    from llm_b200 import LLM
    cfg, page = CONFIGS["D"]
    d = folders("D", "bfloat16")
    prompts = [random_tokens(n, cfg["vocab_size"], 270 + n) for n in (9, 50, 3, 130)]
    llm = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=64, num_kv_blocks=60, eos_token_id=-1)
    base = llm.generate(prompts, max_new_tokens=24)
    calls = {"n": 0}
    waiting = list(prompts)

    def receive(wait):
        calls["n"] += 1
        # two prompts at once, the others only after some steps have run
        if wait or calls["n"] in (2, 9, 15):
            return waiting.pop(0) if waiting else None
        return None

    got = {}
    llm.server(receive, lambda rid, toks: got.__setitem__(rid, toks), max_new_tokens=24)
    _same_or_near_tie(cfg, load_plain_weights(d), prompts, [got[i] for i in range(4)], base)
    assert llm.last_stats["lookahead_steps"] >= 10
    llm.engine.cache.check()


@pytest.mark.parametrize("name", ["D", "E"])
def test_preemption_in_bfloat16_with_graphs_and_lookahead(folders, name):
    """So few pages that decoding preempts and recomputes, with CUDA graphs and the one-step
    lookahead on: the tokens equal those of a pool that holds everything."""
    from llm_b200 import LLM
    cfg, page = CONFIGS[name]
    d = folders(name, "bfloat16")
    prompts = [random_tokens(n, cfg["vocab_size"], 340 + n) for n in (30, 29, 31, 12)]
    roomy = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=32, kv_block_size=page, num_kv_blocks=64,
                eos_token_id=-1)
    want = roomy.generate(prompts, max_new_tokens=40)
    assert roomy.last_num_preemptions == 0
    tight_pages = -(-(31 + 40) // page) * 2 + 1        # two requests fit whole, four do not
    tight = LLM(d, dtype="bfloat16", max_num_seqs=4, max_num_batched_tokens=32, kv_block_size=page,
                num_kv_blocks=tight_pages, eos_token_id=-1, use_cuda_graphs=True, lookahead=True)
    got = tight.generate(prompts, max_new_tokens=40)
    assert tight.last_num_preemptions > 0
    assert tight.last_stats["lookahead_steps"] > 0 and tight.engine.counters["graph_replays"] > 0
    _same_or_near_tie(cfg, load_plain_weights(d), prompts, got, want)
    tight.engine.cache.check()
    assert tight.engine.cache.num_free_pages(0) == tight_pages


@pytest.mark.parametrize("seed", range(20))
def test_random_generations_match_plain(folders, seed):
    """Random prompts through LLM.generate and the scheduler with random limits: live requests,
    token budget, a pool between what the longest request needs and what all need (so some runs
    preempt and recompute), an end token or none, graphs and the one-step lookahead on or off.
    The greedy tokens equal the plain implementation's, up to a near-tie of two logits."""
    from llm_b200 import LLM
    rng = random.Random(9000 + seed)
    name = ["D", "E", "A", "B", "C", "F", "G"][seed % 7]
    dtype = "float32" if seed % 2 else "bfloat16"
    cfg, page = CONFIGS[name]
    d = folders(name, dtype)
    w = load_plain_weights(d)
    new = rng.randint(1, 24)
    prompts = [random_tokens(rng.randint(1, min(cfg["max_position_embeddings"] - new, 90)), cfg["vocab_size"], seed * 50 + i)
               for i in range(rng.randint(1, 7))]
    max_seqs = rng.randint(1, 6)
    need_one = -(-(max(len(p) for p in prompts) + new) // page)
    pool = need_one + rng.randint(0, need_one * (max_seqs - 1) + 2)
    eos = rng.choice([-1, -1, rng.randrange(cfg["vocab_size"])])
    llm = LLM(d, dtype=dtype, max_num_seqs=max_seqs, max_num_batched_tokens=rng.choice([16, 24, 64, 512]), kv_block_size=page,
              num_kv_blocks=pool, eos_token_id=eos, use_cuda_graphs=rng.random() < 0.7, lookahead=rng.random() < 0.7)
    got = llm.generate(prompts, max_new_tokens=new)
    for p, g in zip(prompts, got):
        want = pl.greedy_generate(cfg, w, p, new, eos_token_id=None if eos < 0 else eos)
        if g != want:
            k = next((i for i, (a, b) in enumerate(zip(g, want)) if a != b), min(len(g), len(want)))
            assert k < len(g) and k < len(want), (g, want)
            row = pl.forward(cfg, w, list(p) + want[:k])[-1]
            assert abs(float(row[g[k]] - row[want[k]])) <= TOL[dtype] * float(row.abs().max()), (k, g, want)
    llm.engine.cache.check()
    assert llm.engine.cache.num_free_pages(0) == pool
