"""The engine: a model on one GPU with its cache, and one step function.

step() takes a batch of (request, its next tokens, the places whose logits are
wanted): portions of prompts beside single decoded tokens, cut anywhere.  It runs
only those tokens, as one batch, against the cache that earlier steps left, and
returns float32 logits at the wanted places.  It is what the reference splits over
LLM::inference (runtime/LLM.h:205-219) and Engine::prepare (runtime/Engine.h:52-71),
with three differences: prompt portions and decoded tokens share a batch, the LM
head runs on wanted rows only, and sampling is a layer above.
"""
from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

import ctypes

import numpy as np
import torch

from ..cache.manager import CacheError, CacheManager, GroupSpec, OutOfPages
from ..cache.storage import CacheStorage, StateStorage, bytes_per_page
from ..config.engine_options import EngineOptions
from ..config.model_config import load_config, parse_config
from ..csrc import ops
from ..csrc.build import build as build_kernels, load as load_kernels
from ..parts.base import ResidualStream
from ..weights.loader import adopt_tensors, load_tensors, random_tensors_on_device
from .context import GroupView, LayerView, StepContext, Workspace
from .model import Model

_TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


class StepError(ValueError):
    """A batch that the step function refuses, or a step whose kernels reported a failure."""


@dataclass
class StepEntry:
    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)   # indices into tokens
    feed: Optional[int] = None      # take the (single) token from this row of step()'s feed_source, on the device


class _MetaLayout:
    """Offsets of the step's int32 metadata inside one buffer (one copy per step).  The block
    tables come last, entry by entry, so that a step of few entries copies a prefix."""

    def __init__(self, max_tokens: int, max_entries: int, max_rows: int, table_widths: List[int], base: int = 0):
        off = base
        self.base, self.max_tokens, self.max_entries, self.max_rows, self.widths = base, max_tokens, max_entries, max_rows, table_widths

        def take(n):
            nonlocal off
            start = off
            off += (n + 3) // 4 * 4          # keep every array 16-byte aligned
            return start

        self.cu_tokens = take(max_entries + 1)
        self.kv_lens = take(max_entries)
        self.state_slots = take(max_entries)
        self.token_ids = take(max_tokens)
        self.positions = take(max_tokens)
        self.token_entry = take(max_tokens)
        self.logit_rows = take(max_rows)
        self.feed_dst = take(max_entries)
        self.feed_src = take(max_entries)
        self.slot_map = [take(max_tokens) for _ in table_widths]
        self.block_table = [take(max_entries * w) for w in table_widths]
        self.end = off

    def used_end(self, n_entries: int) -> int:
        """One past the last word that a step of n_entries entries reads."""
        if not self.widths:
            return self.end
        return self.block_table[-1] + n_entries * self.widths[-1]


class _NativeLayout(ctypes.Structure):
    """The layout as the native step preparation takes it (StepLayout in csrc/host/page_pool.cpp)."""
    _fields_ = [(n, ctypes.c_int) for n in ("token_ids", "positions", "token_entry", "cu_tokens", "kv_lens", "state_slots",
                                            "logit_rows", "feed_dst", "feed_src", "n_groups")] + \
               [("block_table", ctypes.c_int * 16), ("slot_map", ctypes.c_int * 16)]

    @classmethod
    def of(cls, lay: "_MetaLayout") -> "_NativeLayout":
        if len(lay.block_table) > 16:
            raise ValueError("at most 16 cache groups")
        out = cls(lay.token_ids, lay.positions, lay.token_entry, lay.cu_tokens, lay.kv_lens, lay.state_slots,
                  lay.logit_rows, lay.feed_dst, lay.feed_src, len(lay.block_table))
        for g, (bt, sm) in enumerate(zip(lay.block_table, lay.slot_map)):
            out.block_table[g] = bt
            out.slot_map[g] = sm
        return out


class Engine:
    MAX_PROMPT_GRAPHS = 64        # captured shapes of steps that bring prompt portions
    MAX_GRAPHS = 512              # captured shapes in all; the one replayed longest ago goes first

    def __init__(self, model_dir: Optional[str], options: Optional[EngineOptions] = None, *,
                 random_config: Optional[dict] = None, random_seed: int = 0, random_on_device: bool = False,
                 tensors: Optional[Dict[str, torch.Tensor]] = None):
        """model_dir: a folder with config.json and model.safetensors.  Without a folder,
        random_config (the contents of a config.json) and random_seed give the same seeded
        random weights that write_random_model would have written, built in memory (with
        random_on_device other values of the same distributions, drawn by the GPU's generator).
        tensors: with random_config, the checkpoint's tensors by name, already in memory, instead
        of drawing them (checked against what the parts expect like a file's)."""
        self.options = options = options or EngineOptions()
        options.validate()
        if not torch.cuda.is_available():
            raise RuntimeError("llm_b200 needs a CUDA device: there is no CPU path")
        # the plain kernel library; a bfloat16 model also needs the tensor-core one (when both
        # have to be compiled first, they are compiled side by side)
        if options.dtype == "bfloat16":
            build_kernels()
            load_kernels("tensor")
        load_kernels()
        self.device = torch.device(options.device)
        torch.cuda.set_device(self.device)
        self.dtype = _TORCH_DTYPE[options.dtype]

        if model_dir is not None:
            self.arch, self.config = load_config(model_dir)
        elif random_config is not None:
            self.arch, self.config = parse_config(random_config)
        else:
            raise ValueError("Engine needs a model folder or a random_config")
        self.spec = self.arch.build_spec(self.config)
        self.model = Model(self.spec, self.dtype, self.device)
        if model_dir is not None:
            tensors = load_tensors(model_dir, self.model.parameters(), self.dtype, self.device)
        elif tensors is not None:
            tensors = adopt_tensors(tensors, self.model.parameters(), self.dtype, self.device)
        else:
            tensors = random_tensors_on_device(self.model.parameters(), random_seed, self.dtype, self.device,
                                               on_device=random_on_device)
        self.model.bind(tensors)
        del tensors

        self.max_seq_len = options.max_seq_len or self.spec.max_position
        if self.max_seq_len > self.spec.max_position:
            raise ValueError(f"max_seq_len {self.max_seq_len} exceeds the model's max_position "
                             f"{self.spec.max_position}")
        self.max_tokens = options.max_num_batched_tokens
        self.max_entries = options.max_num_seqs
        self.max_rows = options.max_logit_rows or self.max_tokens
        self.page_size = options.kv_block_size
        self.hidden, self.vocab = self.spec.hidden_size, self.spec.vocab_size

        self._init_cache()
        self._init_buffers()
        self._drop_graphs()
        self.counters = {"steps": 0, "tokens": 0, "graph_captures": 0, "graph_replays": 0}

    # ---- set-up -------------------------------------------------------------
    def _init_cache(self) -> None:
        opt, model = self.options, self.model
        per_seq_full = (self.max_seq_len + self.page_size - 1) // self.page_size
        pages: List[int] = []
        cap = {}
        for g, (kind, window) in enumerate(model.group_keys):
            if kind == "window":
                per_seq = (window + self.max_tokens + self.page_size - 1) // self.page_size + 2
                cap[g] = self.max_entries * min(per_seq, per_seq_full)
            else:
                cap[g] = self.max_entries * per_seq_full
        if opt.num_kv_blocks is not None:
            pages = [opt.num_kv_blocks for _ in model.group_keys]
        else:
            free, _total = torch.cuda.mem_get_info(self.device)
            budget = int(free * opt.gpu_memory_utilization) - self._activation_estimate()
            for g, (kind, _w) in enumerate(model.group_keys):
                if kind == "window":
                    pages.append(cap[g])
                    budget -= cap[g] * bytes_per_page(model.cache_instances, g, self.page_size, self.dtype)
                else:
                    pages.append(-1)
            for g, (kind, _w) in enumerate(model.group_keys):
                if pages[g] < 0:
                    per = bytes_per_page(model.cache_instances, g, self.page_size, self.dtype)
                    pages[g] = max(0, min(cap[g], budget // max(per, 1)))
            if any(p <= 0 for p in pages):
                raise RuntimeError("not enough free GPU memory for the cache pool")
        specs = [GroupSpec(kind, self.page_size, pages[g], window)
                 for g, (kind, window) in enumerate(model.group_keys)]
        self.cache = CacheManager(specs, self.max_entries, self.max_seq_len)
        self.cache_storage = CacheStorage(model.cache_instances, pages, self.page_size, self.dtype, self.device)
        self.state_storage = StateStorage(model.state_needs, self.max_entries, self.device)
        if opt.poison_freed_pages:
            self.cache.log_freed_pages(True)

    def _activation_estimate(self) -> int:
        widest = 4 * self.spec.hidden_size * 8          # a generous guess of scratch columns per row
        return self.options.max_num_batched_tokens * widest * 4 + (512 << 20)

    def _init_buffers(self) -> None:
        widths = [self.cache.table_width(g) for g in range(self.cache.num_groups)]
        # Two layouts in one buffer.  The small one holds a step in which every entry brings one token
        # (its per-token arrays are as long as the most entries), so that such a step copies a few
        # hundred words plus its entries' table rows instead of arrays sized for the token budget;
        # the large one holds every other step.  The reference likewise uploads only the used part
        # of each array (runtime/Engine.h:109-116).
        small = _MetaLayout(self.max_entries, self.max_entries, min(self.max_rows, self.max_entries), widths)
        large = _MetaLayout(self.max_tokens, self.max_entries, self.max_rows, widths, base=small.end)
        self.layout = large
        self._layouts = (small, large)
        self._host_ring = [torch.zeros(large.end, dtype=torch.int32).pin_memory() for _ in range(4)]
        self._host_events = [None] * len(self._host_ring)
        self._ring_at = 0
        self.meta = torch.zeros(large.end, dtype=torch.int32, device=self.device)
        # word 0: a token id outside the vocabulary; words 1 and 2: a tensor-core product or attention
        # kernel whose bounded wait gave up (the kernels write there while this engine's step runs)
        self.status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self.resid = torch.zeros((self.max_tokens, self.hidden), dtype=torch.float32, device=self.device)
        self.workspace = Workspace(self.max_tokens, self.device)
        self._head_rows = None
        self._logits = None
        self._step_views = [self._views_of(lay) for lay in self._layouts]       # (native layout, context, layer views)

    def _views_of(self, lay: "_MetaLayout"):
        """The device views of one layout: what the parts see of a step that uses it."""
        def dev(off, n):
            return self.meta[off:off + n]

        groups = {
            g: GroupView(page_size=self.page_size,
                         block_table=dev(lay.block_table[g], lay.max_entries * w).view(lay.max_entries, w),
                         slot_map=dev(lay.slot_map[g], lay.max_tokens),
                         kind=self.cache.group_spec(g).kind, window=self.cache.group_spec(g).window)
            for g, w in enumerate(lay.widths)
        }
        views = []
        for occ in self.model.occurrences:
            view = LayerView(owns_cache=occ.owns_cache)
            if occ.cache_instance is not None:
                inst = self.model.cache_instances[occ.cache_instance]
                view.group = groups[inst.group]
                view.k_pages, view.v_pages = self.cache_storage.pages(occ.cache_instance)
            if occ.state_instance is not None:
                view.state = self.state_storage.tensor(occ.state_instance)
            views.append(view)
        ctx = StepContext(
            n_tokens=0, n_entries=0, n_logit_rows=0,
            token_ids=dev(lay.token_ids, lay.max_tokens), positions=dev(lay.positions, lay.max_tokens),
            token_entry=dev(lay.token_entry, lay.max_tokens), cu_tokens=dev(lay.cu_tokens, lay.max_entries + 1),
            kv_lens=dev(lay.kv_lens, lay.max_entries), state_slots=dev(lay.state_slots, lay.max_entries),
            logit_rows=dev(lay.logit_rows, lay.max_rows), status=self.status,
            groups=groups, workspace=self.workspace)
        ctx.layer_views = views
        return _NativeLayout.of(lay), ctx, views

    def _drop_graphs(self) -> None:
        """Forget every captured step (their buffers' addresses changed, or none exist yet)."""
        self._graphs: "OrderedDict[tuple, tuple]" = OrderedDict()     # key -> (graph, kernel launches inside), by last use
        self._graph_seen: Dict[tuple, int] = {}          # how often a shape that is not yet captured has come
        self._prompt_graphs = 0

    def _logit_buffers(self, rows: int):
        if self._logits is None or self._logits.shape[0] < rows:
            n = max(rows, min(self.max_rows, 64))
            self._head_rows = torch.zeros((n, self.hidden), dtype=torch.float32, device=self.device)
            self._head_normed = torch.zeros((n, self.hidden), dtype=self.dtype, device=self.device)
            self._logits = torch.zeros((n, self.vocab), dtype=torch.float32, device=self.device)
            self._drop_graphs()          # captured graphs hold the old addresses
        return self._head_rows, self._head_normed, self._logits

    # ---- requests -----------------------------------------------------------
    def release(self, request_id: Hashable) -> None:
        """The request is finished: its pages and its state slot are given back."""
        self.cache.release(request_id)

    def is_live(self, request_id: Hashable) -> bool:
        return self.cache.is_live(request_id)

    # ---- the step -----------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], feed_source: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch; returns float32 logits [wanted rows, vocab] on the device, in
        the order of the entries and of their `want`.  The tensor is a view of a buffer
        that the next step overwrites.  Entries with `feed` take their token from
        feed_source (int32 on the device, e.g. what the sampler made of the previous step),
        so that a step can be launched before the host has seen the previous step's tokens."""
        ctx = self._prepare(entries, feed_source)
        return self._run(ctx)

    def _prepare(self, entries: Sequence[StepEntry], feed_source: Optional[torch.Tensor] = None) -> StepContext:
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_entries:
            raise StepError(f"{len(entries)} entries exceed max_num_seqs {self.max_entries}")
        seen = set()
        n_tokens = n_rows = 0
        token_arrays = []                                  # each entry's tokens, checked and converted once (an int for one token)
        for e in entries:
            if e.request_id in seen:
                raise StepError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request_id!r} brings no tokens")
            for w in e.want:
                if not (0 <= w < n):
                    raise StepError(f"request {e.request_id!r}: wanted place {w} is outside its {n} tokens")
            if e.feed is not None:
                if n != 1 or feed_source is None or not (0 <= e.feed < feed_source.numel()):
                    raise StepError(f"request {e.request_id!r}: a fed entry brings one token from a row of feed_source")
                token_arrays.append(0)
            elif n == 1:
                tok = e.tokens[0]
                if not (0 <= tok < self.vocab):
                    raise StepError(f"request {e.request_id!r}: token id outside [0, {self.vocab})")
                token_arrays.append(int(tok))
            else:
                try:
                    arr = np.asarray(e.tokens, dtype=np.int64)
                except (OverflowError, TypeError, ValueError):
                    raise StepError(f"request {e.request_id!r}: token ids must be integers in [0, {self.vocab})") from None
                if arr.ndim != 1 or int(arr.min()) < 0 or int(arr.max()) >= self.vocab:
                    raise StepError(f"request {e.request_id!r}: token id outside [0, {self.vocab})")
                token_arrays.append(arr)
            n_tokens += n
            n_rows += len(e.want)
        if n_tokens > self.max_tokens:
            raise StepError(f"{n_tokens} tokens exceed max_num_batched_tokens {self.max_tokens}")
        if n_rows > self.max_rows:
            raise StepError(f"{n_rows} wanted rows exceed the limit {self.max_rows}")

        cache = self.cache
        B = len(entries)
        which = 0 if n_tokens == B else 1                  # one token per entry: the small layout
        lay = self._layouts[which]
        native_layout, ctx, _views = self._step_views[which]
        host_t = self._next_host_buffer()
        ns = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=B)
        starts = np.empty(B, dtype=np.int32)
        slots = np.empty(B, dtype=np.int32)
        # all or nothing: the pool sees that every entry fits before any page moves, then admits
        # the new requests and takes the pages
        try:
            cache.begin_step([e.request_id for e in entries], ns, slots, starts)
        except OutOfPages:
            raise
        except CacheError as err:
            raise StepError(str(err)) from None
        T = n_tokens
        tokens = (np.asarray(token_arrays, dtype=np.int32) if T == B
                  else np.concatenate([np.atleast_1d(a) for a in token_arrays]).astype(np.int32, copy=False))
        want_counts = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=B)
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=n_rows)
        feeds = np.fromiter((-1 if (e.feed is None or feed_source is None) else e.feed for e in entries), dtype=np.int32, count=B)
        # the native routine writes tokens, positions, block tables, slot maps, wanted rows and the
        # rest of the step's metadata into the pinned block, from the pool's own tables
        lib, pool = cache.native
        ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)
        n_feed = lib.llmh_prepare_step(pool, ctypes.byref(native_layout), ctypes.c_void_p(host_t.data_ptr()), B,
                                       ptr(slots), ptr(ns), ptr(starts), ptr(tokens), ptr(want_counts), ptr(wants), ptr(feeds))
        if n_feed < 0:
            raise StepError(lib.llmh_pool_error(pool).decode("utf-8", "replace"))
        entry_tokens, entry_start, entry_slots = ns, starts, slots
        if self.options.poison_freed_pages:
            # everything freed since the last step (requests that ended or were preempted, pages a
            # window has passed) is overwritten before this step's kernels run: those launched
            # earlier, which may still read the pages, are ahead of the fill on the stream
            for g in range(cache.num_groups):
                self.cache_storage.poison(g, cache.take_freed_pages(g))
        fresh = cache.take_fresh_slots()
        if fresh:
            self.state_storage.zero_slots(fresh)
        a, b = lay.base, lay.used_end(B)
        self.meta[a:b].copy_(host_t[a:b], non_blocking=True)
        self.last_h2d_bytes = 4 * (b - a)
        ev = torch.cuda.Event()
        ev.record()
        self._host_events[self._ring_at] = ev
        if n_feed:
            ops.feed_tokens(ctx.token_ids, feed_source, self.meta[lay.feed_dst: lay.feed_dst + n_feed],
                            self.meta[lay.feed_src: lay.feed_src + n_feed], n_feed)

        ctx.n_tokens, ctx.n_entries, ctx.n_logit_rows = n_tokens, B, n_rows
        ctx.host_entry_tokens, ctx.host_entry_start, ctx.host_state_slots = entry_tokens, entry_start, entry_slots
        ctx.kv_bucket = (int((entry_start + entry_tokens).max()) + 255) // 256 * 256
        return ctx

    def _next_host_buffer(self) -> torch.Tensor:
        self._ring_at = (self._ring_at + 1) % len(self._host_ring)
        ev = self._host_events[self._ring_at]
        if ev is not None:
            ev.synchronize()
        return self._host_ring[self._ring_at]

    def _forward(self, ctx: StepContext) -> None:
        ops.set_stream(torch.cuda.current_stream().cuda_stream)     # looked up once per step, not per kernel
        if self.dtype == torch.bfloat16:
            ops.set_error_block(self.status)
        try:
            self._forward_on_stream(ctx)
        finally:
            ops.set_stream(None)
            if self.dtype == torch.bfloat16:
                ops.set_error_block(None)

    def _forward_on_stream(self, ctx: StepContext) -> None:
        stream = ResidualStream(self.resid, ctx.n_tokens)
        self.model.forward(ctx, stream, ctx.layer_views)
        if ctx.n_logit_rows:
            self.model.head.logits(stream, ctx, self.model.final_norm, self._logit_buffers(ctx.n_logit_rows))

    def _run(self, ctx: StepContext) -> torch.Tensor:
        R = ctx.n_logit_rows
        if R:
            self._logit_buffers(R)
        # The launch parameters of a step depend only on its numbers of entries, tokens and wanted
        # rows and, for a step of single tokens, on the bucket of the longest context; everything
        # else is read from the metadata buffer on the device.  So a step is captured once per such
        # key and replayed (the reference captures per GraphShape{batch, tokens} the same way,
        # runtime/LLM.h:63-72,192-201): steps of single tokens at once, other shapes when they come
        # a second time (a portion of the full token budget recurs, a ragged last portion does not).
        graphable = self.options.use_cuda_graphs and self.model.is_graph_safe(ctx)
        if graphable:
            key = (ctx.n_entries, ctx.n_tokens, R, ctx.kv_bucket if ctx.decode_only else 0)
            entry = self._graphs.get(key)
            if entry is None and not ctx.decode_only:
                seen = self._graph_seen.get(key, 0)
                self._graph_seen[key] = seen + 1
                if seen == 0 or self._prompt_graphs >= self.MAX_PROMPT_GRAPHS:
                    graphable = False
        if graphable:
            if entry is not None:
                self._graphs.move_to_end(key)
                entry[0].replay()
                ops.count_launches(entry[1])
                self.counters["graph_replays"] += 1
            else:
                self._forward(ctx)                       # this step's result; also sizes the scratch buffers
                torch.cuda.synchronize(self.device)
                before = ops.launch_count()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._forward(ctx)                   # recorded only; same inputs, same result when replayed
                self._graphs[key] = (graph, ops.launch_count() - before)
                while len(self._graphs) > self.MAX_GRAPHS:
                    old_key, _old = self._graphs.popitem(last=False)
                    if old_key[3] == 0:
                        self._prompt_graphs -= 1
                ops.count_launches(-(ops.launch_count() - before))
                self.counters["graph_captures"] += 1
                if not ctx.decode_only:
                    self._prompt_graphs += 1
        else:
            self._forward(ctx)
        self.counters["steps"] += 1
        self.counters["tokens"] += ctx.n_tokens
        return self._logits[:R] if R else torch.empty((0, self.vocab), dtype=torch.float32, device=self.device)

    def check_status(self) -> None:
        """Raise if, since the last check, a kernel met a token id outside the vocabulary or gave
        up one of its bounded waits (its output is then zeros, so the step's logits are not to be
        used).  One small copy; synchronises."""
        words = self.status.tolist()
        if any(words):
            self.status.zero_()
            problems = []
            if words[0]:
                problems.append("a kernel met a token id outside the vocabulary")
            problems += [ops.describe_wait(i, words[i]) for i in (1, 2) if words[i]]
            raise StepError("; ".join(problems))

    def memory_report(self) -> dict:
        return {"weights": self.model.weight_bytes(), "cache": self.cache_storage.bytes(),
                "workspace": self.workspace.bytes(),
                "pages": [self.cache.group_spec(g).num_pages for g in range(self.cache.num_groups)]}
