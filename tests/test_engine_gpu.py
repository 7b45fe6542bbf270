"""GPU tests of the whole engine against the plain implementation: every way of
cutting the work, in 32-bit and in bfloat16."""
import random

import pytest
import torch

import plain_llama
import replay
from tiny import CONFIGS, TOL, load_plain_weights, make_model_dir, max_err, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 40, 64, 97, 130], "C": [3, 50, 81, 120],
           "D": [2, 129, 300, 47, 260], "E": [33, 290, 131, 380], "F": [4, 150, 61, 280], "G": [9, 140, 77, 230]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("models")
    cache = {}

    def get(name, dtype, peaked=False):
        key = (name, dtype, peaked)
        if key not in cache:
            d = make_model_dir(root, name, dtype, peaked=peaked)
            w = load_plain_weights(d)
            cfg, page = CONFIGS[name]
            reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], 100 + i) for i, n in enumerate(LENGTHS[name])}
            ref = {rid: plain_llama.forward(cfg, w, toks) for rid, toks in reqs.items()}
            cache[key] = (d, cfg, page, reqs, ref)
        return cache[key]
    return get


def make_engine(model_dir, dtype, page, num_blocks, max_tokens=512, max_seqs=4, poison=True):
    """poison: pages that go back to the pool are overwritten with a huge value, so that a kernel
    that reads a page its request does not hold gives logits that are far off."""
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine
    return Engine(model_dir, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_seqs,
                                           max_num_batched_tokens=max_tokens, num_kv_blocks=num_blocks,
                                           use_cuda_graphs=False, poison_freed_pages=poison))


def compare(got, ref, dtype, what):
    for rid, r in ref.items():
        assert got[rid].shape == r.shape, f"{what}: {rid} shape {got[rid].shape} vs {r.shape}"
        # the first wrong row, to point at the place (a page's edge, a portion's start, ...)
        err_rows = (got[rid].double() - r).abs().max(dim=1).values / r.abs().max()
        bad = torch.nonzero(err_rows > TOL[dtype])
        assert bad.numel() == 0, (f"{what}: request {rid} first differs at position {int(bad[0])} "
                                  f"(err {float(err_rows[int(bad[0])]):.3e}, limit {TOL[dtype]:.1e})")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F", "G"])
def test_every_cut_matches_plain(models, name, dtype):
    d, cfg, page, reqs, ref = models(name, dtype)
    longest = max(len(t) for t in reqs.values())
    pages_one = (longest + page - 1) // page
    # whole, tail decode and portions: one request at a time, a pool barely larger than the longest
    eng = make_engine(d, dtype, page, pages_one + 1)
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, dtype, "whole")
    compare(replay.run_steps(eng, replay.steps_tail_decode(reqs)), ref, dtype, "tail decode")
    compare(replay.run_steps(eng, replay.steps_portions(reqs)), ref, dtype, "portions")
    eng.cache.check()
    assert all(eng.cache.num_free_pages(g) == eng.cache.group_spec(g).num_pages for g in range(eng.cache.num_groups))
    # mixed: up to four live, so few pages that freed ones are used again
    lens = sorted((len(t) for t in reqs.values()), reverse=True)
    pool = sum((n + page - 1) // page for n in lens[:4]) + 1
    eng = make_engine(d, dtype, page, pool)
    compare(replay.run_steps(eng, replay.steps_mixed(reqs)), ref, dtype, "mixed")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C", "D", "E"])
def test_every_cut_matches_plain_with_peaked_attention(models, name, dtype):
    """The same cuts on weights whose attention is peaked (a few keys carry each row), where one
    wrong key, page or window edge moves a logit by far more than the bound; freed pages poisoned."""
    d, cfg, page, reqs, ref = models(name, dtype, peaked=True)
    longest = max(len(t) for t in reqs.values())
    eng = make_engine(d, dtype, page, (longest + page - 1) // page + 1)
    compare(replay.run_steps(eng, replay.steps_whole(reqs)), ref, dtype, "whole")
    compare(replay.run_steps(eng, replay.steps_tail_decode(reqs)), ref, dtype, "tail decode")
    compare(replay.run_steps(eng, replay.steps_portions(reqs)), ref, dtype, "portions")
    lens = sorted((len(t) for t in reqs.values()), reverse=True)
    eng = make_engine(d, dtype, page, sum((n + page - 1) // page for n in lens[:4]) + 1)
    compare(replay.run_steps(eng, replay.steps_mixed(reqs)), ref, dtype, "mixed")
    eng.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_at_a_context_of_thousands_of_keys(tmp_path_factory, dtype):
    """A prompt of 5,100 tokens in portions of 1,024 (the prompt attention over a long cache), then
    70 tokens one by one from replayed graphs (the decode attention cut into dozens of ranges, the
    count of keys crossing a bucket's edge), with peaked attention so that a lost or doubled range
    of keys would show; every decoded position against the plain implementation."""
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    cfg, page = CONFIGS["H"]
    d = make_model_dir(tmp_path_factory.mktemp("long"), "H", dtype, peaked=True)
    n, tail = 5170, 70
    toks = random_tokens(n, cfg["vocab_size"], 77)
    rows = list(range(n - tail, n))
    ref = plain_llama.forward(cfg, load_plain_weights(d), toks, rows=rows)
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=2, max_num_batched_tokens=1024,
                                  num_kv_blocks=n // page + 3, use_cuda_graphs=True, poison_freed_pages=True))
    head = n - tail
    for at in range(0, head, 1024):
        eng.step([StepEntry("x", toks[at:min(at + 1024, head)], [])])
    got = torch.stack([eng.step([StepEntry("x", [t], [0])])[0].double().cpu() for t in toks[head:]])
    eng.check_status()
    err_rows = (got - ref).abs().max(dim=1).values / ref.abs().max()
    bad = torch.nonzero(err_rows > TOL[dtype])
    assert bad.numel() == 0, f"first differs at position {head + int(bad[0])}: {float(err_rows[int(bad[0])]):.3e}"
    assert eng.counters["graph_replays"] >= tail - 4


@pytest.mark.parametrize("seed", range(24))
def test_random_workloads_match_plain(tmp_path_factory, seed):
    """Random requests cut into random steps: portions of 1 to 160 tokens beside single tokens, up to
    eight live, requests that sit a step out, entries in shuffled order, wanted rows picked at
    random, a pool that only just holds the live requests (so pages are used again, poisoned in
    between), graphs on or off; every wanted row against the plain implementation."""
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    rng = random.Random(4000 + seed)
    name = ["D", "E", "A", "C", "G", "H"][seed % 6]
    dtype = "float32" if seed % 3 == 2 else "bfloat16"
    cfg, page = CONFIGS[name]
    d = make_model_dir(tmp_path_factory.mktemp("random"), name, dtype, peaked=seed % 2 == 0)
    w = load_plain_weights(d)
    lens = [rng.randint(1, min(cfg["max_position_embeddings"], 500)) for _ in range(rng.randint(3, 7))]
    reqs = {f"r{i}": random_tokens(n, cfg["vocab_size"], seed * 100 + i) for i, n in enumerate(lens)}
    ref = {rid: plain_llama.forward(cfg, w, toks) for rid, toks in reqs.items()}
    max_live = rng.randint(1, 8)
    pool = sum((n + page - 1) // page for n in sorted(lens, reverse=True)[:max_live]) + rng.randint(0, 3)
    budget = rng.choice([64, 200, 512])
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=max_live, max_num_batched_tokens=budget,
                                  num_kv_blocks=pool, use_cuda_graphs=rng.random() < 0.7, poison_freed_pages=True))
    pending, live = list(reqs.items()), []
    while pending or live:
        while pending and len(live) < max_live and rng.random() < 0.7:
            rid, toks = pending[0]
            held = sum((len(t) + page - 1) // page for _, t, _ in live)
            if held + (len(toks) + page - 1) // page > pool:
                break
            pending.pop(0)
            live.append([rid, toks, 0])
        entries, ended, left = [], [], budget
        for item in live:
            rid, toks, at = item
            if rng.random() < 0.15 and len(live) > 1:
                continue                                   # this request sits the step out
            n = min(1 if rng.random() < 0.45 else rng.randint(1, 160), len(toks) - at, left)
            if n <= 0:
                continue
            left -= n
            want = sorted(rng.sample(range(n), rng.randint(0, min(n, 6)))) if rng.random() < 0.8 else list(range(n))
            entries.append((rid, toks[at:at + n], want, at))
            item[2] = at + n
            if item[2] == len(toks):
                ended.append(rid)
        if not entries:
            continue
        rng.shuffle(entries)
        out = eng.step([StepEntry(rid, t, wnt) for rid, t, wnt, _ in entries]).double().cpu()
        row = 0
        for rid, t, wnt, at in entries:
            for k in wnt:
                err = float((out[row] - ref[rid][at + k]).abs().max() / ref[rid].abs().max())
                assert err <= TOL[dtype], (f"request {rid} position {at + k}: {err:.3e} in a step of "
                                           f"{[(r, len(tt), a) for r, tt, _, a in entries]}")
                row += 1
        for rid in ended:
            eng.release(rid)
        live = [it for it in live if it[0] not in ended]
    eng.check_status()
    eng.cache.check()


@pytest.mark.parametrize("seed", range(24))
def test_random_configurations_match_plain(tmp_path_factory, seed):
    """Random small configurations of the architecture: widths that are no powers of two (some with
    rows that are no multiples of 16 bytes), any numbers of heads and groups, head sizes from 6 to
    256, vocabularies, eps, theta, windows, tied heads, biases, page sizes; a prompt in two
    portions and then tokens one by one, in 32-bit or bfloat16, against the plain implementation."""
    import os

    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    from llm_b200.weights.loader import write_random_model
    rng = random.Random(700 + seed)
    n_kv, group = rng.choice([1, 1, 2, 3, 4, 5]), rng.choice([1, 1, 2, 3, 4, 8])
    hidden = rng.choice([64, 72, 96, 128, 160, 200, 256]) + (rng.choice([2, 4, 6]) if rng.random() < 0.3 else 0)
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=hidden, intermediate_size=rng.choice([100, 172, 200, 256, 344]),
               num_hidden_layers=rng.randint(1, 3), num_attention_heads=n_kv * group, num_key_value_heads=n_kv,
               head_dim=rng.choice([16, 32, 48, 64, 64, 80, 96, 100, 128, 128, 112, 6, 256]),
               vocab_size=rng.choice([97, 256, 301, 1000]), rms_norm_eps=rng.choice([1e-5, 1e-6, 1e-3]),
               rope_theta=rng.choice([10000.0, 500000.0, 100.0]), max_position_embeddings=rng.choice([64, 200, 520]),
               tie_word_embeddings=rng.random() < 0.3, hidden_act="silu")
    if rng.random() < 0.3:
        cfg["sliding_window"] = rng.randint(3, 90)
    cfg["attention_bias"], cfg["mlp_bias"] = rng.random() < 0.25, rng.random() < 0.25
    page = rng.choice([8, 16, 16, 32, 64])
    dtype = "float32" if seed % 2 else "bfloat16"
    d = os.path.join(str(tmp_path_factory.mktemp("cfg")), "model")
    write_random_model(d, cfg, seed, dtype)
    n = rng.randint(2, cfg["max_position_embeddings"])
    toks = random_tokens(n, cfg["vocab_size"], seed)
    ref = plain_llama.forward(cfg, load_plain_weights(d), toks)
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=2, max_num_batched_tokens=600,
                                  num_kv_blocks=n // page + 3, use_cuda_graphs=rng.random() < 0.6, poison_freed_pages=True))
    head = n - rng.randint(0, min(20, n - 1))
    cut = rng.randint(1, head)
    rows = [eng.step([StepEntry("x", toks[:cut], list(range(cut)))]).double().cpu().clone()]
    if cut < head:
        rows.append(eng.step([StepEntry("x", toks[cut:head], list(range(head - cut)))]).double().cpu().clone())
    for t in toks[head:]:
        rows.append(eng.step([StepEntry("x", [t], [0])]).double().cpu().clone())
    eng.check_status()
    err_rows = (torch.cat(rows) - ref).abs().max(dim=1).values / ref.abs().max()
    bad = torch.nonzero(err_rows > TOL[dtype])
    assert bad.numel() == 0, f"{cfg}, page {page}: first differs at position {int(bad[0])}: {float(err_rows[int(bad[0])]):.3e}"


def test_peaked_attention_shows_one_wrong_page(models):
    """What the peaked weights are for: two pages of values that trade places (the keys stay) move
    the bfloat16 logits of the next token far beyond the bound, while on the plain random weights,
    where every softmax is nearly uniform, the same fault stays inside it."""
    from llm_b200.engine.engine import StepEntry
    moved = {}
    for peaked in (False, True):
        d, cfg, page, reqs, ref = models("D", "bfloat16", peaked=peaked)
        toks = reqs["r2"]                                   # 300 tokens
        eng = make_engine(d, "bfloat16", page, 40, poison=False)
        eng.step([StepEntry("x", toks[:-1], [])])
        table = eng.cache.table(0, "x")
        a, b = table[-2], table[-4]
        for inst in range(len(eng.cache_storage.k)):
            v_pages = eng.cache_storage.pages(inst)[1]
            tmp = v_pages[a].clone()
            v_pages[a] = v_pages[b]
            v_pages[b] = tmp
        got = eng.step([StepEntry("x", toks[-1:], [0])])[0].double().cpu()
        moved[peaked] = float((got - ref["r2"][-1]).abs().max() / ref["r2"].abs().max())
    assert moved[False] < TOL["bfloat16"] and moved[True] > 3 * TOL["bfloat16"], moved


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_plain(models, dtype):
    from llm_b200 import LLM
    d, cfg, page, reqs, _ = models("A", dtype)
    w = load_plain_weights(d)
    prompts = [random_tokens(n, cfg["vocab_size"], 7 + n) for n in (5, 17, 33)]
    llm = LLM(d, dtype=dtype, max_num_seqs=4, max_num_batched_tokens=24, kv_block_size=page,
              num_kv_blocks=12, eos_token_id=-1, use_cuda_graphs=False)
    got = llm.generate(prompts, max_new_tokens=16)
    for p, g in zip(prompts, got):
        assert len(g) == 16
        if dtype == "float32":
            assert g == plain_llama.greedy_generate(cfg, w, p, 16)
        else:
            # bfloat16 may flip near-ties: every chosen token must be within rounding of the best
            ids = list(p)
            for tok in g:
                row = plain_llama.forward(cfg, w, ids)[-1]
                assert float(row.max() - row[tok]) <= 2 * TOL[dtype] * float(row.abs().max())
                ids.append(tok)
    llm.engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_recurring_prompt_shapes_replayed_from_graphs_match_plain(models, name, dtype):
    """With CUDA graphs on, a step shape (entries, tokens, wanted rows) that comes a second time is
    captured and replayed from then on, for prompt portions as for decoded tokens.  The same
    requests in portions of one size, twice over with pages used again, and mixed with decoded
    tokens of other requests: every logit against the plain implementation."""
    from llm_b200.config import EngineOptions
    from llm_b200.engine.engine import Engine, StepEntry
    d, cfg, page, reqs, ref = models(name, dtype)
    longest = max(len(t) for t in reqs.values())
    eng = Engine(d, EngineOptions(dtype=dtype, kv_block_size=page, max_num_seqs=4, max_num_batched_tokens=512,
                                  num_kv_blocks=2 * ((longest + page - 1) // page) + 2, use_cuda_graphs=True))
    chunk = 24
    for round_ in range(2):
        got = {}
        for rid, toks in reqs.items():
            rows = []
            for a in range(0, len(toks), chunk):
                part = toks[a:a + chunk]
                rows.append(eng.step([StepEntry(rid, part, list(range(len(part))))]).double().cpu().clone())
            got[rid] = torch.cat(rows)
            eng.release(rid)
        compare(got, ref, dtype, f"portions of {chunk}, round {round_}")
    assert eng.counters["graph_replays"] > 0 and eng.counters["graph_captures"] >= 1
    # a portion of one request beside a decoded token of another, the same shape again and again
    ids = list(reqs)
    long_id = max(ids, key=lambda r: len(reqs[r]))
    short_id = min(ids, key=lambda r: len(reqs[r]))
    before = eng.counters["graph_replays"]
    got = {long_id: [], short_id: []}
    lt, st = reqs[long_id], reqs[short_id]
    got[short_id].append(eng.step([StepEntry(short_id, st[:1], [0])]).double().cpu().clone())
    at, k = 0, 1
    while at < len(lt):
        part = lt[at:at + 16]
        entries = [StepEntry(long_id, part, list(range(len(part))))]
        if k < len(st):
            entries.append(StepEntry(short_id, [st[k]], [0]))
        out = eng.step(entries).double().cpu().clone()
        got[long_id].append(out[:len(part)])
        if k < len(st):
            got[short_id].append(out[len(part):])
            k += 1
        at += len(part)
    while k < len(st):
        got[short_id].append(eng.step([StepEntry(short_id, [st[k]], [0])]).double().cpu().clone())
        k += 1
    compare({r: torch.cat(v) for r, v in got.items()}, {r: ref[r] for r in got}, dtype, "portion beside a decoded token")
    if len(lt) >= 4 * 16 and len(st) > 4:
        assert eng.counters["graph_replays"] > before
    eng.cache.check()


def test_a_step_that_cannot_run_is_refused_whole(models):
    """Too many new requests, a request past max_seq_len, too few pages: the step is refused
    before any page or slot moves, and the engine goes on as if it had not been asked."""
    from llm_b200.cache import OutOfPages
    from llm_b200.engine.engine import StepEntry, StepError
    d, cfg, page, reqs, ref = models("A", "float32")
    eng = make_engine(d, "float32", page, num_blocks=4, max_seqs=2)
    toks = reqs["r2"]                                           # 33 tokens: three pages of 16
    first = eng.step([StepEntry("x", toks[:20], [19])]).double().cpu().clone()
    free = eng.cache.num_free_pages(0)
    with pytest.raises(OutOfPages):                             # "y" needs 3 pages, 2 are free; "x" would have fitted
        eng.step([StepEntry("x", toks[20:22], [1]), StepEntry("y", toks, [0])])
    with pytest.raises(StepError):                              # a third request: only two slots
        eng.step([StepEntry("x", toks[20:22], []), StepEntry("y", [1], []), StepEntry("z", [2], [])])
    with pytest.raises(StepError):                              # past the longest sequence the engine holds
        eng.step([StepEntry("x", [1] * (eng.max_seq_len - 19), [])])
    eng.cache.check()
    assert eng.cache.num_free_pages(0) == free and eng.cache.length("x") == 20 and not eng.cache.is_live("y")
    rest = eng.step([StepEntry("x", toks[20:], list(range(13)))]).double().cpu()
    got = torch.cat([first, rest])
    assert max_err(got, ref["r2"][19:]) < TOL["float32"]
