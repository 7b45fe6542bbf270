"""The scheduler: admits requests, cuts prompts into portions under a token budget,
decodes, finishes and frees.

The scheduler itself is native (csrc/host/scheduler.cpp, C++ behind a C interface on top of the
native page pool, as the reference's scheduler is C++); this module is its Python face: the
batch and request types that the entry points work with, and a class that passes calls through.

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
Engine::prepare (runtime/Engine.h:57); the scheduler only does the arithmetic, group by group.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field
from typing import Dict, Iterator, List, Optional

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
    """A request as the scheduler has it at the moment of asking (a copy: it does not follow
    the scheduler's later steps)."""
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


@dataclass
class _Sampling:
    temperature: float
    seed: int
    ignore_eos: bool
    max_new_tokens: int


class _Requests:
    """scheduler.requests: the waiting and running requests by id, read from the native side."""

    def __init__(self, sched: "Scheduler"):
        self._s = sched

    def __contains__(self, rid) -> bool:
        return rid in self._s._sampling

    def __len__(self) -> int:
        return self._s.num_requests()

    def __iter__(self) -> Iterator[int]:
        return iter(list(self._s._sampling))

    def get(self, rid, default=None):
        return self._s._request(rid) or default

    def __getitem__(self, rid) -> Request:
        r = self._s._request(rid)
        if r is None:
            raise KeyError(rid)
        return r


class Scheduler:
    def __init__(self, cache: CacheManager, cfg: SchedulerConfig):
        if cfg.max_num_seqs > cfg.max_num_batched_tokens:
            raise ValueError("max_num_seqs must not exceed max_num_batched_tokens")
        if cfg.max_num_seqs > cache.max_requests:
            raise ValueError("max_num_seqs exceeds the cache manager's request slots")
        self.cache, self.cfg = cache, cfg
        self._lib, pool = cache.native
        lib = self._lib
        lib.llmh_sched_create.restype = ctypes.c_void_p
        lib.llmh_sched_add.restype = ctypes.c_longlong
        lib.llmh_sched_num_preemptions.restype = ctypes.c_longlong
        lib.llmh_sched_batch.restype = ctypes.POINTER(ctypes.c_int)
        lib.llmh_sched_finished.restype = ctypes.POINTER(ctypes.c_int)
        lib.llmh_sched_request.restype = ctypes.POINTER(ctypes.c_int)
        lib.llmh_sched_request.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.POINTER(ctypes.c_int),
                                           ctypes.POINTER(ctypes.c_int)]
        eos = cfg.eos_token_id if cfg.eos_token_id is not None else -1
        h = lib.llmh_sched_create(pool, cfg.max_num_seqs, cfg.max_num_batched_tokens, eos)
        if not h:
            raise ValueError("the scheduler refused this configuration")
        self._h = ctypes.c_void_p(h)
        n = cfg.max_num_seqs
        self._ids = (ctypes.c_longlong * n)()
        self._starts = (ctypes.c_int * n)()
        self._counts = (ctypes.c_int * n)()
        self._samples = (ctypes.c_int * n)()
        self._new = (ctypes.c_int * n)()
        self._sampling: Dict[int, _Sampling] = {}      # what only the sampler needs, by request id
        self.requests = _Requests(self)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.llmh_sched_destroy(h)

    # ---- admission ----
    def add_request(self, prompt: List[int], max_new_tokens: int, temperature: float = 0.0, seed: int = 0,
                    ignore_eos: bool = False) -> int:
        """Returns the request id, or -1 if the request can never run: empty prompt, longer
        than max_seq_len with its new tokens, or more pages than a whole group holds."""
        arr = (ctypes.c_int * max(len(prompt), 1))(*prompt)
        rid = int(self._lib.llmh_sched_add(self._h, arr, len(prompt), int(max_new_tokens), int(ignore_eos)))
        if rid >= 0:
            self._sampling[rid] = _Sampling(temperature, seed, ignore_eos, int(max_new_tokens))
        return rid

    def num_requests(self) -> int:
        return self._lib.llmh_sched_num_requests(self._h)

    @property
    def num_preemptions(self) -> int:
        return int(self._lib.llmh_sched_num_preemptions(self._h))

    @property
    def prefill_ready(self) -> List[int]:
        return self._queue(0)

    @property
    def decode_ready(self) -> List[int]:
        return self._queue(1)

    def _queue(self, which: int) -> List[int]:
        n = self._lib.llmh_sched_queue(self._h, which, self._ids, 0)
        out = (ctypes.c_longlong * max(n, 1))()
        self._lib.llmh_sched_queue(self._h, which, out, n)
        return list(out[:n])

    def _request(self, rid) -> Optional[Request]:
        n, fields = ctypes.c_int(), (ctypes.c_int * 6)()
        toks = self._lib.llmh_sched_request(self._h, int(rid), ctypes.byref(n), fields)
        if not toks:
            return None
        sp = self._sampling[rid]
        return Request(rid, toks[:n.value], fields[0], fields[1], sp.temperature, sp.seed, sp.ignore_eos,
                       DECODE if fields[2] else PREFILL, fields[3], fields[4], bool(fields[5]))

    def sampling_of(self, rid) -> _Sampling:
        """temperature, seed and ignore_eos of a waiting or running request."""
        return self._sampling[rid]

    # ---- one step's batch ----
    def schedule(self) -> ScheduledBatch:
        """The next step's batch.  If nothing can run although requests wait, prompts that
        hold pages behind the head of the queue give them back (they are recomputed later),
        which always lets the head run: admission made sure that it fits alone."""
        n_tokens = ctypes.c_int()
        n = self._lib.llmh_sched_schedule(self._h, ctypes.byref(n_tokens))
        toks = self._lib.llmh_sched_batch(self._h, self._ids, self._starts, self._counts, self._samples)
        batch = ScheduledBatch()
        at = 0
        for i in range(n):
            c = self._counts[i]
            batch.entries.append(ScheduledEntry(self._ids[i], self._starts[i], toks[at:at + c], bool(self._samples[i])))
            at += c
        return batch

    def _pack(self, batch: ScheduledBatch) -> int:
        n = len(batch.entries)
        if n > len(self._ids):
            raise ValueError("a batch of more entries than max_num_seqs")
        for i, e in enumerate(batch.entries):
            self._ids[i], self._starts[i], self._counts[i], self._samples[i] = e.request_id, e.start, len(e.tokens), e.samples
        return n

    # ---- after the step ----
    def update(self, batch: ScheduledBatch, new_tokens: Dict[int, int]) -> List[Request]:
        """Account for a finished step.  new_tokens maps the id of every entry that samples
        to its next token.  Returns the requests that finished; their pages are free again."""
        n = self._pack(batch)
        for i, e in enumerate(batch.entries):
            self._new[i] = int(new_tokens[e.request_id]) if e.samples and e.request_id in new_tokens else 0
        k = self._lib.llmh_sched_update(self._h, n, self._ids, self._starts, self._counts, self._samples, self._new)
        done = []
        rid, plen, nt, npre = ctypes.c_longlong(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        for i in range(k):
            toks = self._lib.llmh_sched_finished(self._h, i, ctypes.byref(rid), ctypes.byref(plen), ctypes.byref(nt),
                                                 ctypes.byref(npre))
            sp = self._sampling.pop(rid.value)
            done.append(Request(rid.value, toks[:nt.value], plen.value, sp.max_new_tokens, sp.temperature, sp.seed,
                                sp.ignore_eos, DECODE, nt.value, npre.value, True))
        return done

    # ---- one step of lookahead: the next step is launched before this step's tokens are read ----
    def can_look_ahead(self, batch: ScheduledBatch) -> bool:
        """Whether the step after `batch` can be scheduled before the tokens of `batch` are
        known: only decoding requests, nobody waiting to be admitted, nobody at its last token,
        and pages for one more token of each without preempting anyone."""
        n = self._pack(batch)
        return bool(self._lib.llmh_sched_can_look_ahead(self._h, n, self._ids, self._samples))

    def update_pending(self, batch: ScheduledBatch) -> None:
        """update() for a step whose tokens are not known yet: every request gets a placeholder
        and goes on decoding.  Only after can_look_ahead(batch)."""
        done = self.update(batch, {e.request_id: PENDING_TOKEN for e in batch.entries})
        assert not done

    def resolve(self, batch: ScheduledBatch, new_tokens: Dict[int, int]) -> None:
        """The tokens of a step that was accounted with update_pending() have arrived.  A request
        that ends with its token is marked: it is already part of the step in flight and retires
        when that step is accounted."""
        n = self._pack(batch)
        for i, e in enumerate(batch.entries):
            self._new[i] = int(new_tokens[e.request_id])
        rc = self._lib.llmh_sched_resolve(self._h, n, self._ids, self._new)
        assert rc == 0, "no pending token to resolve"
