"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

Rules are those of the reference's Scheduler (runtime/Scheduler.h:81-283) with one
change: a step is one mixed batch instead of a prefill batch or a decode batch
(:103-108).  Decoding requests come first, one token each; what is left of
max_num_batched_tokens is filled with prompt portions in arrival order, a long
prompt cut to the budget and several short ones sharing it (:155-191).  A portion is
scheduled only if the free pages cover it plus a reserve of one page for every
running request that will sit on a page boundary (:170-171,222-232); a request that
does not fit stops the walk (head-of-line blocking, :171).

When pages run out: prompts wait; if the decoding requests themselves cannot all
take their next token, the one queued last is preempted: its pages and slot are
given back and it returns to the head of the prompt queue with everything it has
produced so far as its prompt, to be recomputed (:194,234-246).  A request whose
prompt plus max_new_tokens can never fit is refused at add_request (:89-91).

The pages themselves are taken inside Engine.step, as the reference takes them in
Engine::prepare (runtime/Engine.h:57); the scheduler only does the arithmetic, and
asks the cache manager for it, group by group.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from ..cache.manager import CacheManager

PREFILL, DECODE = "prefill", "decode"
PENDING_TOKEN = -1      # stands in a request's tokens for a token that is sampled but not read back yet


@dataclass
class SchedulerConfig:
    max_num_seqs: int
    max_num_batched_tokens: int
    eos_token_id: Optional[int] = None


@dataclass
class Request:
    id: int
    token_ids: List[int]
    prompt_len: int
    max_new_tokens: int
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False
    phase: str = PREFILL
    cached_len: int = 0          # tokens whose keys and values are in the cache
    num_preemptions: int = 0
    ended: bool = False          # its end was found after the next step had already been launched

    @property
    def generated(self) -> List[int]:
        return self.token_ids[self.prompt_len:]


@dataclass
class ScheduledEntry:
    request_id: int
    start: int                   # position of the first token
    tokens: List[int]
    samples: bool                # the step's last token of this entry yields the next token


@dataclass
class ScheduledBatch:
    entries: List[ScheduledEntry] = field(default_factory=list)

    def empty(self) -> bool:
        return not self.entries

    @property
    def num_tokens(self) -> int:
        return sum(len(e.tokens) for e in self.entries)


class Scheduler:
    def __init__(self, cache: CacheManager, cfg: SchedulerConfig):
        if cfg.max_num_seqs > cfg.max_num_batched_tokens:
            raise ValueError("max_num_seqs must not exceed max_num_batched_tokens")
        if cfg.max_num_seqs > cache.max_requests:
            raise ValueError("max_num_seqs exceeds the cache manager's request slots")
        self.cache, self.cfg = cache, cfg
        self._next_id = 0
        self.requests: Dict[int, Request] = {}
        self.prefill_ready: Deque[int] = deque()
        self.decode_ready: Deque[int] = deque()
        self.num_preemptions = 0

    # ---- admission ----
    def add_request(self, prompt: List[int], max_new_tokens: int, temperature: float = 0.0, seed: int = 0,
                    ignore_eos: bool = False) -> int:
        """Returns the request id, or -1 if the request can never run: empty prompt, longer
        than max_seq_len with its new tokens, or more pages than a whole group holds."""
        worst = len(prompt) + max_new_tokens
        if not prompt or max_new_tokens <= 0 or worst > self.cache.max_seq_len:
            return -1
        for g, need in enumerate(self.cache.pages_needed(None, worst, length=0)):
            if need > self.cache.group_spec(g).num_pages:
                return -1
        rid = self._next_id
        self._next_id += 1
        self.requests[rid] = Request(rid, list(prompt), len(prompt), max_new_tokens, temperature, seed, ignore_eos)
        self.prefill_ready.append(rid)
        return rid

    def num_requests(self) -> int:
        return len(self.requests)

    # ---- one step's batch ----
    def schedule(self) -> ScheduledBatch:
        """The next step's batch.  If nothing can run although requests wait, prompts that
        hold pages behind the head of the queue give them back (they are recomputed later),
        which always lets the head run: admission made sure that it fits alone."""
        batch = self._schedule_once()
        if batch.empty() and self.requests:
            head = self.prefill_ready[0] if self.prefill_ready else None
            freed = False
            for rid in reversed(self.prefill_ready):
                if rid != head and self.cache.is_live(rid):
                    self.cache.release(rid)
                    self.requests[rid].cached_len = 0
                    self.requests[rid].num_preemptions += 1
                    self.num_preemptions += 1
                    freed = True
            if freed:
                batch = self._schedule_once()
        return batch

    def _schedule_once(self) -> ScheduledBatch:
        batch = ScheduledBatch()
        cache, cfg = self.cache, self.cfg
        G = cache.num_groups
        promised = [0] * G

        def fits(needs, reserve=None) -> bool:
            return all(cache.num_free_pages(g) - promised[g] >= needs[g] + (reserve[g] if reserve else 0)
                       for g in range(G))

        # Decoding requests first; preempt from the back while they do not all fit.
        per_request = {}
        while self.decode_ready:
            needs = [0] * G
            first = list(self.decode_ready)[:cfg.max_num_seqs]
            for rid in first:
                k = per_request.get(rid)
                if k is None:
                    k = per_request[rid] = cache.pages_needed(rid, 1)
                for g in range(G):
                    needs[g] += max(k[g], 0)
            if fits(needs):
                break
            self._preempt_last_decode()
        for rid in list(self.decode_ready)[:cfg.max_num_seqs]:
            r = self.requests[rid]
            self.decode_ready.popleft()
            k = per_request[rid]
            for g in range(G):
                promised[g] += k[g]
            batch.entries.append(ScheduledEntry(rid, r.cached_len, [r.token_ids[-1]], True))
        budget = cfg.max_num_batched_tokens - batch.num_tokens

        # Prompt portions in arrival order.
        while self.prefill_ready and budget > 0 and len(batch.entries) < cfg.max_num_seqs:
            rid = self.prefill_ready[0]
            r = self.requests[rid]
            target = len(r.token_ids)
            chunk = min(target - r.cached_len, budget)
            is_final = r.cached_len + chunk == target
            live = cache.is_live(rid)
            if not live and cache.num_free_slots() - self._new_in(batch) <= 0:
                break
            needs = cache.pages_needed(rid if live else None, chunk, length=r.cached_len)
            reserve = self._decode_reserve(batch)
            if is_final:          # this request decodes next and may start on a fresh page
                for g in range(G):
                    if target % cache.group_spec(g).page_size == 0:
                        reserve[g] += 1
            if not fits(needs, reserve):
                break
            for g in range(G):
                promised[g] += needs[g]
            batch.entries.append(ScheduledEntry(rid, r.cached_len, r.token_ids[r.cached_len:r.cached_len + chunk],
                                                is_final))
            budget -= chunk
            if is_final:
                self.prefill_ready.popleft()
            else:
                break        # the rest of this prompt comes in the next step; nothing may overtake it
        return batch

    def _new_in(self, batch: ScheduledBatch) -> int:
        return sum(1 for e in batch.entries if not self.cache.is_live(e.request_id))

    def _decode_reserve(self, batch: ScheduledBatch) -> List[int]:
        """One page per request that, after this step, decodes from a page boundary."""
        G = self.cache.num_groups
        reserve = [0] * G
        in_batch = {e.request_id: e for e in batch.entries}
        for rid, r in self.requests.items():
            e = in_batch.get(rid)
            if e is not None:
                after = e.start + len(e.tokens)
                runs_on = e.samples
            else:
                after = r.cached_len
                runs_on = r.phase == DECODE
            if runs_on and after > 0:
                for g in range(G):
                    if after % self.cache.group_spec(g).page_size == 0:
                        reserve[g] += 1
        return reserve

    def _preempt_last_decode(self) -> None:
        rid = self.decode_ready.pop()
        r = self.requests[rid]
        if self.cache.is_live(rid):
            self.cache.release(rid)
        r.cached_len = 0
        r.phase = PREFILL
        r.num_preemptions += 1
        self.prefill_ready.appendleft(rid)
        self.num_preemptions += 1

    # ---- after the step ----
    def update(self, batch: ScheduledBatch, new_tokens: Dict[int, int]) -> List[Request]:
        """Account for a finished step.  new_tokens maps the id of every entry that samples
        to its next token.  Returns the requests that finished; their pages are free again."""
        done = []
        for e in batch.entries:
            r = self.requests.get(e.request_id)
            if r is None:
                continue
            r.cached_len = e.start + len(e.tokens)
            if not e.samples:
                continue
            if r.ended:                      # ran one step too far: that step's token is dropped
                self._retire(r, done)
                continue
            tok = int(new_tokens[e.request_id])
            r.token_ids.append(tok)
            if tok != PENDING_TOKEN and self._finished(r, tok):
                self._retire(r, done)
            else:
                r.phase = DECODE
                self.decode_ready.append(r.id)
        return done

    def _retire(self, r: Request, done: List[Request]) -> None:
        if self.cache.is_live(r.id):
            self.cache.release(r.id)
        del self.requests[r.id]
        done.append(r)

    # ---- one step of lookahead: the next step is launched before this step's tokens are read ----
    def can_look_ahead(self, batch: ScheduledBatch) -> bool:
        """Whether the step after `batch` can be scheduled before the tokens of `batch` are
        known: only decoding requests, nobody waiting to be admitted, nobody at its last token,
        and pages for one more token of each without preempting anyone."""
        if self.prefill_ready or not batch.entries:
            return False
        need = [0] * self.cache.num_groups
        for e in batch.entries:
            r = self.requests.get(e.request_id)
            if r is None or not e.samples or r.ended:
                return False
            if len(r.token_ids) - r.prompt_len + 2 > r.max_new_tokens:     # this step's token would be its last
                return False
            if self.cache.length(r.id) + 1 > self.cache.max_seq_len:
                return False
            for g, k in enumerate(self.cache.pages_needed(r.id, 1)):
                need[g] += max(k, 0)
        return all(need[g] <= self.cache.num_free_pages(g) for g in range(self.cache.num_groups))

    def update_pending(self, batch: ScheduledBatch) -> None:
        """update() for a step whose tokens are not known yet: every request gets a placeholder
        and goes on decoding.  Only after can_look_ahead(batch)."""
        done = self.update(batch, {e.request_id: PENDING_TOKEN for e in batch.entries})
        assert not done

    def resolve(self, batch: ScheduledBatch, new_tokens: Dict[int, int]) -> None:
        """The tokens of a step that was accounted with update_pending() have arrived.  A request
        that ends with its token is marked: it is already part of the step in flight and retires
        when that step is accounted."""
        eos = self.cfg.eos_token_id
        for e in batch.entries:
            r = self.requests.get(e.request_id)
            if r is None:
                continue
            tok = int(new_tokens[e.request_id])
            at = len(r.token_ids) - 1
            while at >= r.prompt_len and r.token_ids[at] != PENDING_TOKEN:
                at -= 1
            assert at >= r.prompt_len, "no pending token to resolve"
            r.token_ids[at] = tok
            if eos is not None and eos >= 0 and tok == eos and not r.ignore_eos:
                del r.token_ids[at + 1:]
                r.ended = True

    def _finished(self, r: Request, tok: int) -> bool:
        eos = self.cfg.eos_token_id
        hit_eos = eos is not None and eos >= 0 and tok == eos and not r.ignore_eos
        return hit_eos or len(r.token_ids) - r.prompt_len >= r.max_new_tokens
