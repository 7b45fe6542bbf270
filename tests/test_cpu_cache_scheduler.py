"""CPU tests: the cache manager's invariants under random orders of requests, and the
scheduler's decisions (portions, budget, reserve, what happens when pages run out).
Scenarios follow the reference's host test runtime/test/test_scheduler_chunk.cpp."""
import random

import pytest

from llm_b200.cache import CacheError, CacheManager, GroupSpec, OutOfPages
from llm_b200.engine.scheduler import Scheduler, SchedulerConfig


def full_pool(pages=8, page=16, max_req=4, max_len=256):
    return CacheManager([GroupSpec("full", page, pages)], max_req, max_len)


def test_extend_release_and_tables():
    c = full_pool()
    c.admit("a")
    assert c.extend("a", 17) == 0 and c.length("a") == 17
    assert len(c.table(0, "a")) == 2 and c.num_free_pages(0) == 6
    assert c.extend("a", 15) == 17 and len(c.table(0, "a")) == 2      # 32 tokens: still two pages
    assert c.extend("a", 1) == 32 and len(c.table(0, "a")) == 3
    assert c.physical_slot(0, "a", 33) == c.table(0, "a")[2] * 16 + 1
    c.check()
    c.release("a")
    assert c.num_free_pages(0) == 8 and c.num_free_slots() == 4
    with pytest.raises(CacheError, match="not live"):
        c.release("a")
    with pytest.raises(CacheError):
        c.extend("a", 1)
    c.check()


def test_out_of_pages_changes_nothing():
    c = full_pool(pages=2)
    c.admit("a")
    c.extend("a", 20)
    c.admit("b")
    with pytest.raises(OutOfPages):
        c.extend("b", 16)
    assert c.length("b") == 0 and c.num_free_pages(0) == 0
    assert not c.can_extend("b", 1) and c.can_extend("a", 12) and not c.can_extend("a", 13)
    c.check()


def test_window_group_gives_pages_back_and_reuses_them():
    c = CacheManager([GroupSpec("full", 8, 40), GroupSpec("window", 8, 12, window=20)], 2, 300)
    c.admit("a")
    pos = 0
    for n in (30, 1, 1, 7, 25, 2, 60, 1):
        assert c.pages_needed("a", n)[1] <= c.num_free_pages(1)
        assert c.extend("a", n) == pos
        pos += n
        c.check()
        t = c.table(1, "a")
        lowest_key = max(0, pos - n - 20 + 1)          # first key the first new token could see
        for i, p in enumerate(t):
            if (i + 1) * 8 <= lowest_key:
                assert p == -1                         # out of every later window: given back
            else:
                assert p >= 0
        assert all(p >= 0 for p in c.table(0, "a"))     # the full group keeps everything
    # a window group never holds more than ceil((window + step) / page) + 1 pages per request
    assert sum(p >= 0 for p in c.table(1, "a")) <= 4
    c.release("a")
    assert c.num_free_pages(1) == 12 and c.num_free_pages(0) == 40
    c.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted(seed):
    rng = random.Random(seed)
    groups = [GroupSpec("full", 8, 30)] + ([GroupSpec("window", 8, 20, window=rng.choice([5, 16, 33]))] if seed % 2 else [])
    c = CacheManager(groups, 5, 200)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and c.num_free_slots():
            c.admit(next_id); live[next_id] = 0; next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 16, 40])
            if c.can_extend(rid, n):
                assert c.extend(rid, n) == live[rid]
                live[rid] += n
            else:
                before = [c.num_free_pages(g) for g in range(c.num_groups)]
                with pytest.raises(CacheError):
                    c.extend(rid, n)
                assert before == [c.num_free_pages(g) for g in range(c.num_groups)]
        elif live:
            rid = rng.choice(list(live))
            c.release(rid); del live[rid]
        c.check()
    for rid in list(live):
        c.release(rid)
    c.check()
    assert all(c.num_free_pages(g) == c.group_spec(g).num_pages for g in range(c.num_groups))
    assert c.num_free_slots() == 5


# ---- scheduler ---------------------------------------------------------------

def run_step(sched, cache, batch, token=7):
    """What the engine does with a batch, as far as the cache is concerned."""
    for e in batch.entries:
        if not cache.is_live(e.request_id):
            cache.admit(e.request_id)
        assert cache.extend(e.request_id, len(e.tokens)) == e.start
    cache.check()
    return sched.update(batch, {e.request_id: token for e in batch.entries if e.samples})


def test_prompt_is_cut_to_the_budget():
    c = full_pool(pages=16)
    s = Scheduler(c, SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=32))
    rid = s.add_request(list(range(80)), 2)
    sizes = []
    for _ in range(3):
        b = s.schedule()
        sizes.append([len(e.tokens) for e in b.entries])
        assert [e.samples for e in b.entries] == [len(sizes) == 3]
        run_step(s, c, b)
    assert sizes == [[32], [32], [16]]
    b = s.schedule()                                     # now it decodes
    assert [(e.request_id, len(e.tokens), e.start, e.samples) for e in b.entries] == [(rid, 1, 80, True)]
    done = run_step(s, c, b)
    assert [r.id for r in done] == [rid] and done[0].generated == [7, 7]
    assert c.num_free_pages(0) == 16 and c.num_free_slots() == 4 and s.num_requests() == 0


def test_short_prompts_share_a_batch_and_decode_rides_along():
    c = full_pool(pages=16)
    s = Scheduler(c, SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=32))
    a = s.add_request([1] * 5, 4)
    b_ = s.add_request([2] * 9, 4)
    big = s.add_request([3] * 40, 4)
    b = s.schedule()
    assert [(e.request_id, len(e.tokens)) for e in b.entries] == [(a, 5), (b_, 9), (big, 18)]
    assert [e.samples for e in b.entries] == [True, True, False]
    run_step(s, c, b)
    b = s.schedule()                                     # two decode tokens first, then the rest of the prompt
    assert [(e.request_id, len(e.tokens)) for e in b.entries] == [(a, 1), (b_, 1), (big, 22)]
    assert b.num_tokens <= 32
    run_step(s, c, b)
    b = s.schedule()
    assert sorted(len(e.tokens) for e in b.entries) == [1, 1, 1]


def test_rejects_what_can_never_run():
    c = full_pool(pages=4, max_len=100)
    s = Scheduler(c, SchedulerConfig(2, 32))
    assert s.add_request([], 4) == -1
    assert s.add_request([1] * 90, 20) == -1              # longer than max_seq_len
    assert s.add_request([1] * 60, 10) == -1              # 5 pages, the pool has 4
    assert s.add_request([1] * 60, 4) >= 0


def test_prefill_waits_for_pages_and_reserve():
    c = full_pool(pages=3)
    s = Scheduler(c, SchedulerConfig(4, 64))
    a = s.add_request([1] * 16, 8)                       # ends exactly on a page edge: needs its next page kept
    b_ = s.add_request([2] * 20, 4)
    b = s.schedule()
    assert [e.request_id for e in b.entries] == [a]      # b would leave no page for a's first decoded token
    run_step(s, c, b)
    b = s.schedule()
    assert [(e.request_id, len(e.tokens)) for e in b.entries] == [(a, 1)]
    run_step(s, c, b)
    for _ in range(6):
        run_step(s, c, s.schedule())
    assert s.num_requests() == 1 and c.num_free_pages(0) == 3
    b = s.schedule()
    assert [(e.request_id, len(e.tokens)) for e in b.entries] == [(b_, 20)]


def test_decode_preempts_the_latest_and_recomputes():
    c = full_pool(pages=4, page=16)
    s = Scheduler(c, SchedulerConfig(4, 64))
    a = s.add_request([1] * 30, 30)
    b_ = s.add_request([2] * 30, 30)
    run_step(s, c, s.schedule())                         # both prompts: 2 pages each, pool full
    assert c.num_free_pages(0) == 0
    for _ in range(2):                                    # positions 30 and 31 still fit in the held pages
        b = s.schedule()
        assert len(b.entries) == 2
        run_step(s, c, b)
    b = s.schedule()                                     # both need a third page and none is free
    assert s.num_preemptions == 1
    assert [(e.request_id, len(e.tokens)) for e in b.entries] == [(a, 1)]
    run_step(s, c, b)
    r = s.requests[b_]
    assert r.cached_len == 0 and len(r.token_ids) == 33 and not c.is_live(b_)
    b = s.schedule()                                     # a decodes; b's recompute needs 3 pages, 1 is free
    assert [e.request_id for e in b.entries] == [a]
    run_step(s, c, b)
    steps = 0
    finished = []
    while s.num_requests():
        b = s.schedule()
        assert not b.empty()
        finished += run_step(s, c, b)
        steps += 1
        assert steps < 200
    assert sorted(r.id for r in finished) == [a, b_]
    assert all(len(r.generated) == 30 for r in finished)
    assert c.num_free_pages(0) == 4 and c.num_free_slots() == 4


@pytest.mark.parametrize("seed", range(5))
def test_random_load_finishes_and_frees_everything(seed):
    rng = random.Random(seed)
    page = rng.choice([8, 16])
    groups = [GroupSpec("full", page, 12)] + ([GroupSpec("window", page, 10, window=24)] if seed % 2 else [])
    c = CacheManager(groups, 4, 160)
    s = Scheduler(c, SchedulerConfig(4, 24, eos_token_id=3))
    want = {}
    for _ in range(12):
        n, m = rng.randint(1, 70), rng.randint(1, 30)
        rid = s.add_request([rng.randint(4, 90) for _ in range(n)], m)
        if rid >= 0:
            want[rid] = m
    done = {}
    for _ in range(3000):
        if not s.num_requests():
            break
        b = s.schedule()
        assert not b.empty() and b.num_tokens <= 24 and len(b.entries) <= 4
        for r in run_step(s, c, b, token=rng.choice([3, 5, 5, 5, 5, 5, 5, 5])):
            done[r.id] = r
    assert set(done) == set(want)
    for rid, r in done.items():
        assert 1 <= len(r.generated) <= want[rid]
        assert r.generated[-1] == 3 or len(r.generated) == want[rid]
    assert all(c.num_free_pages(g) == c.group_spec(g).num_pages for g in range(c.num_groups))
    assert c.num_free_slots() == 4


def test_lookahead_placeholders_resolve_and_late_end():
    """A step accounted before its tokens are known: placeholders, then the real tokens; a request
    whose token was the end retires when the step it ran too far is accounted."""
    from llm_b200.engine.scheduler import PENDING_TOKEN
    c = full_pool(pages=16)
    s = Scheduler(c, SchedulerConfig(4, 64, eos_token_id=3))
    a = s.add_request([5] * 10, 6)
    b_ = s.add_request([6] * 4, 6)
    run_step(s, c, s.schedule(), token=9)                     # prompts; both sampled 9
    b1 = s.schedule()
    assert s.can_look_ahead(b1)
    for e in b1.entries:
        c.extend(e.request_id, 1)
    s.update_pending(b1)
    assert s.requests[a].token_ids[-1] == PENDING_TOKEN
    b2 = s.schedule()                                         # scheduled with the tokens still unknown
    assert [e.tokens for e in b2.entries] == [[PENDING_TOKEN], [PENDING_TOKEN]]
    for e in b2.entries:
        c.extend(e.request_id, 1)
    s.resolve(b1, {a: 7, b_: 3})                              # b's token was the end
    assert s.requests[a].token_ids[-1] == 7 and s.requests[b_].ended
    assert not s.can_look_ahead(b2)
    done = s.update(b2, {a: 8, b_: 8})
    assert [r.id for r in done] == [b_] and done[0].generated == [9, 3]
    assert s.requests[a].generated == [9, 7, 8] and not c.is_live(b_)
    c.check()
    # a request one token before its limit is not looked ahead
    b3 = s.schedule()
    run_step(s, c, b3, token=8)
    b4 = s.schedule()
    run_step(s, c, b4, token=8)
    b5 = s.schedule()                                         # generated 5 of 6: this step's token is the last
    assert not s.can_look_ahead(b5)


def test_request_ids_are_integers_or_names_and_the_scheduler_shares_the_pool():
    """The pool knows requests by a 64-bit key: integers are their own key, other ids get one.
    What the native scheduler releases is gone for the cache manager too."""
    c = full_pool(pages=8)
    c.admit("a"); c.admit(7); c.admit(("x", 1))
    c.extend("a", 3); c.extend(7, 20); c.extend(("x", 1), 1)
    assert sorted(map(str, c.live_requests())) == sorted(["a", "7", "('x', 1)"])
    assert c.length(7) == 20 and c.slot("a") != c.slot(7) and not c.is_live("b") and not c.is_live(8)
    with pytest.raises(CacheError):
        c.admit(7)
    c.release("a"); c.release(7); c.release(("x", 1))
    c.admit("a")                                          # a name may come back
    c.release("a")
    c.check()
    s = Scheduler(c, SchedulerConfig(4, 64))
    rid = s.add_request([1, 2, 3], 1)
    run_step(s, c, s.schedule())                          # finishes with its first token
    assert not c.is_live(rid) and c.num_free_slots() == 4 and rid not in s.requests
    c.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_load_with_lookahead_keeps_tokens_and_pages_straight(seed):
    """Random requests, steps accounted ahead of their tokens whenever the scheduler allows it:
    every request finishes with exactly the tokens it was given, in order, no placeholder is
    left, a request that met its end stops there, and every page and slot comes back."""
    from llm_b200.engine.scheduler import PENDING_TOKEN
    rng = random.Random(100 + seed)
    page = rng.choice([4, 8, 16])
    groups = [GroupSpec("full", page, rng.randint(10, 30))] + ([GroupSpec("window", page, 12, window=20)] if seed % 2 else [])
    c = CacheManager(groups, 4, 200)
    s = Scheduler(c, SchedulerConfig(4, 32, eos_token_id=3))
    limit, given = {}, {}
    for _ in range(10):
        n, m = rng.randint(1, 60), rng.randint(1, 25)
        rid = s.add_request([rng.randint(4, 90) for _ in range(n)], m)
        if rid >= 0:
            limit[rid], given[rid] = m, []
    done, pending = {}, None
    for _ in range(5000):
        if not s.num_requests():
            break
        b = s.schedule()
        assert not b.empty() and b.num_tokens <= 32 and len(b.entries) <= 4
        for e in b.entries:
            if not c.is_live(e.request_id):
                c.admit(e.request_id)
            assert c.extend(e.request_id, len(e.tokens)) == e.start
        c.check()
        toks = {e.request_id: rng.choice([3, 5, 6, 7, 8, 9, 10, 11, 12]) for e in b.entries if e.samples}
        if pending is not None:                           # the step before: its tokens arrive now
            s.resolve(*pending)
            pending = None
        if all(len(e.tokens) == 1 for e in b.entries) and s.can_look_ahead(b) and rng.random() < 0.8:
            s.update_pending(b)
            pending = (b, toks)
            for rid, t in toks.items():
                given[rid].append(t)
        else:
            for rid, t in toks.items():
                given[rid].append(t)
            for r in s.update(b, toks):
                done[r.id] = r
    assert pending is None and set(done) == set(limit)
    for rid, r in done.items():
        gen = r.generated
        assert PENDING_TOKEN not in gen and 1 <= len(gen) <= limit[rid]
        assert gen == given[rid][:len(gen)]               # what ran one step too far was dropped
        assert gen[-1] == 3 or len(gen) == limit[rid]
        assert 3 not in gen[:-1]
    assert all(c.num_free_pages(g) == c.group_spec(g).num_pages for g in range(c.num_groups))
    assert c.num_free_slots() == 4
    c.check()


def test_begin_step_uses_pages_that_a_later_entry_of_the_same_step_gives_back():
    """All or nothing: the step's page count nets what window entries give back, so an entry that
    takes pages may stand before the entry whose window frees them."""
    import numpy as np
    c = CacheManager([GroupSpec("window", 8, 6, window=8)], 3, 200)
    slots, starts = np.zeros(1, np.int32), np.zeros(1, np.int32)
    c.begin_step(["old"], np.array([40], np.int32), slots, starts)          # 5 of 6 pages held
    assert c.num_free_pages(0) == 1
    # "new" needs 2 pages, one is free; "old" gives back 4 (keys below 33 are out of sight) and takes 1
    slots, starts = np.zeros(2, np.int32), np.zeros(2, np.int32)
    c.begin_step(["new", "old"], np.array([16, 8], np.int32), slots, starts)
    assert list(starts) == [0, 40] and c.length("new") == 16 and c.length("old") == 48
    c.check()
    # and a step that does not fit changes nothing
    before = (c.num_free_pages(0), c.length("new"), c.length("old"), c.table(0, "old"))
    with pytest.raises(OutOfPages):
        c.begin_step(["new", "third"], np.array([8, 40], np.int32), slots, starts)
    assert before == (c.num_free_pages(0), c.length("new"), c.length("old"), c.table(0, "old"))
    assert not c.is_live("third")
    c.check()


def test_freed_pages_are_logged_for_the_poison_fill():
    c = CacheManager([GroupSpec("full", 8, 10), GroupSpec("window", 8, 10, window=8)], 2, 200)
    c.log_freed_pages(True)
    c.admit("a")
    c.extend("a", 30)
    held_full, held_win = c.table(0, "a"), c.table(1, "a")
    assert c.take_freed_pages(0) == [] and c.take_freed_pages(1) == []
    c.extend("a", 1)                       # keys below 23 are out of sight: two window pages go back
    assert sorted(c.take_freed_pages(1)) == sorted(held_win[:2]) and c.take_freed_pages(1) == []
    c.release("a")
    assert sorted(c.take_freed_pages(0)) == sorted(held_full)
    assert sorted(c.take_freed_pages(1)) == sorted(held_win[2:])
    c.check()


def test_ranges_of_the_decode_attention():
    """How many ranges the keys of a request are cut into (pure arithmetic, no device): always 1
    to 64; short contexts in ranges of at least about 128 keys and at most 16 of them; long ones
    in ranges of at least 256 keys, as many as give two CTAs per SM in one wave."""
    from llm_b200.csrc.ops import decode_splits
    sms = 148
    for entries in (1, 2, 3, 8, 24, 64, 300):
        for n_kv in (1, 4, 8):
            for keys in (1, 100, 520, 1024, 2048, 2049, 4096, 8192, 40000, 1 << 20):
                s = decode_splits(entries, n_kv, keys, sms)
                assert 1 <= s <= 64
                if keys <= 2048:
                    assert s <= 16 and (s == 1 or keys / s >= 64)
                else:
                    assert s == 1 or (keys / s >= 256 and s * entries * n_kv <= 2 * sms)
    assert decode_splits(8, 4, 520, sms) in (4, 5, 6)          # the benchmark's step: ranges of about 100 keys
    assert decode_splits(8, 4, 16384, sms) == 9                # 288 CTAs on 148 SMs
    assert decode_splits(1, 4, 1 << 20, sms) == 64


def test_plans_of_the_tensor_core_product_cover_k():
    """The planner's choices as arithmetic (no device): every plan splits K into parts that cover
    it exactly once; up to 23 rows run the swapped mode, 24 to 128 rows one CTA per tile of 128 or
    256 weight rows, and a limit on the CTAs is kept where K is split."""
    from llm_b200.csrc import ops
    for M in (1, 8, 16, 23, 24, 32, 64, 100, 128, 129, 300, 2048):
        for N, K in ((2560, 2048), (2048, 5632), (11264, 2048), (32000, 2048), (22016, 4096), (344, 200), (72, 1000)):
            for fused in (False, True):
                swap, tile, splits, per, mode = ops._plan_gemm(M, N, K, fused, True, True, 148, 0)
                kb = -(-K // 64)
                assert splits >= 1 and per >= 1 and splits * per >= kb and -(-kb // per) == splits, (M, N, K)
                assert swap == (M < ops.NORMAL_MODE_FROM_ROWS)
                if swap:
                    assert tile in (16, 32, 64, 128) and tile >= M
                elif M <= 128:
                    assert tile in (128, 256) and mode == 0
                else:
                    assert tile % 32 == 0 and 128 <= tile <= 256
    swap, tile, splits, per, mode = ops._plan_gemm(64, 2560, 2048, True, True, True, 148, 49)
    assert not swap and (splits == 1 or -(-2560 // tile) * splits <= 49)
