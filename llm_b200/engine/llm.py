"""The Python entry point: LLM, in the manner of the reference's runtime/LLM.h.

The reference's LLM owns the model, runs one step per scheduled batch (`inference`,
runtime/LLM.h:205-219) and serves requests through two callbacks (`server`,
:221-263), taking text through its tokenizer.  This one takes and returns token
ids.  Option names are the reference's where it has them: max_num_seqs,
max_num_batched_tokens, eos_token_id (runtime/Scheduler.h:60-64), max_seq_len and
max_new_tokens (model/llm/tiny_llama.cpp:19-20).
"""
from __future__ import annotations

import time
from typing import Callable, Dict, List, Optional, Sequence

import torch

from ..config.engine_options import EngineOptions
from ..sampling.sampler import Sampler, uniform_for
from .engine import Engine, StepEntry
from .scheduler import PENDING_TOKEN, Request, ScheduledBatch, Scheduler, SchedulerConfig


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", max_num_seqs: int = 8,
                 max_num_batched_tokens: int = 512, max_seq_len: Optional[int] = None,
                 eos_token_id: Optional[int] = None, kv_block_size: int = 16,
                 num_kv_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.9,
                 use_cuda_graphs: bool = True, device: str = "cuda:0", random_config: Optional[dict] = None,
                 random_seed: int = 0, lookahead: bool = True, random_on_device: bool = False, tensors=None):
        """model: a folder with config.json and model.safetensors, or None together with
        random_config (a config.json's contents) for seeded random weights (random_on_device:
        drawn by the GPU's generator instead of the CPU's, for models of many billions of weights;
        other values than the folder that write_random_model writes)."""
        options = EngineOptions(dtype=dtype, kv_block_size=kv_block_size, max_num_seqs=max_num_seqs,
                                max_num_batched_tokens=max_num_batched_tokens, max_seq_len=max_seq_len,
                                num_kv_blocks=num_kv_blocks, gpu_memory_utilization=gpu_memory_utilization,
                                max_logit_rows=max_num_seqs, use_cuda_graphs=use_cuda_graphs, device=device)
        self.engine = Engine(model, options, random_config=random_config, random_seed=random_seed,
                             random_on_device=random_on_device, tensors=tensors)
        if eos_token_id is None:
            eos_token_id = self.engine.spec.eos_token_id
        self.eos_token_id = eos_token_id
        self.scheduler_config = SchedulerConfig(max_num_seqs, max_num_batched_tokens, eos_token_id)
        self.sampler = Sampler(max_num_seqs, self.engine.device)
        self.lookahead = lookahead     # launch decode steps before the previous step's tokens are read

    # ---- one scheduled batch through the model: tokens in, next tokens out ----
    def launch(self, scheduler: Scheduler, batch: ScheduledBatch, previous=None):
        """Start a step and the sampling of its tokens without waiting for either.  Tokens that
        are still pending in the scheduler (sampled by `previous`, a launch() result that the
        host has not read yet) are taken from the previous step's sampler output on the device.
        Returns (rows, handle): the entries that sample and the handle of their tokens."""
        entries, rows = [], []
        feed_rows = {e.request_id: i for i, e in enumerate(previous[0])} if previous is not None else {}
        for e in batch.entries:
            want = [len(e.tokens) - 1] if e.samples else []
            if len(e.tokens) == 1 and e.tokens[0] == PENDING_TOKEN:
                entries.append(StepEntry(e.request_id, [0], want, feed=feed_rows[e.request_id]))
            else:
                entries.append(StepEntry(e.request_id, e.tokens, want))
            if e.samples:
                rows.append(e)
        logits = self.engine.step(entries, feed_source=previous[1].device if feed_rows else None)
        temps, unis = [], []
        for e in rows:
            sp = scheduler.sampling_of(e.request_id)
            temps.append(sp.temperature)
            unis.append(uniform_for(sp.seed, e.request_id, e.start + len(e.tokens)) if sp.temperature > 0 else 0.0)
        return rows, self.sampler.sample_async(logits, temps, unis)

    def inference(self, scheduler: Scheduler, batch: ScheduledBatch) -> Dict[int, int]:
        """One step, waited for: the next token of every entry that samples."""
        rows, handle = self.launch(scheduler, batch)
        return {e.request_id: t for e, t in zip(rows, handle.result())}

    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256, temperature: float = 0.0,
                 seed: int = 0, ignore_eos: bool = False) -> List[List[int]]:
        """Generated token ids for every prompt (lists of token ids), in the prompts' order."""
        scheduler = Scheduler(self.engine.cache, self.scheduler_config)
        ids = []
        for i, p in enumerate(prompts):
            rid = scheduler.add_request(list(p), max_new_tokens, temperature, seed, ignore_eos)
            if rid < 0:
                raise ValueError(f"prompt {i} cannot run: empty, or {len(p)} + {max_new_tokens} tokens exceed "
                                 f"max_seq_len {self.engine.max_seq_len} or the cache pool")
            ids.append(rid)
        results: Dict[int, List[int]] = {}
        self._run_to_idle(scheduler, lambda r: results.__setitem__(r.id, r.generated))
        self.last_num_preemptions = scheduler.num_preemptions
        return [results[rid] for rid in ids]

    def _run_to_idle(self, scheduler: Scheduler, on_finished: Callable[[Request], None],
                     poll: Optional[Callable[[], None]] = None) -> None:
        """Steps until no request is left; poll(), if given, is called before every step is
        scheduled and may add requests.

        While requests only decode, a step is launched before the tokens of the step before it
        have reached the host: its input tokens are fed on the device from the sampler's output,
        and the host reads the earlier tokens (to store them and to look for the end of a request)
        while the GPU is already busy.  A request that turns out to have ended runs one step too
        far; that step's token is dropped.  Whenever the next batch could depend on the tokens
        (a request at its last token, prompts waiting, pages short) the step is waited for first.
        Host-side times of the steps that only decode are kept in last_stats, as the reference's
        driver keeps sched/wait/update times per step (runtime/Driver.h:16,74-83)."""
        stats = {"steps": 0, "decode_steps": 0, "decode_tokens": 0, "decode_seconds": 0.0, "lookahead_steps": 0,
                 "prompt_steps": 0, "prompt_step_tokens": 0, "prompt_seconds": 0.0,
                 "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                 # host seconds over all steps: choosing the batch, launching it, waiting for tokens, accounting for them
                 "sched_seconds": 0.0, "launch_seconds": 0.0, "wait_seconds": 0.0, "update_seconds": 0.0}
        previous = None              # (batch, rows, handle) of a launched step whose tokens are not read yet
        clock = time.perf_counter
        t_mark = clock()
        while scheduler.num_requests():
            if poll is not None:
                poll()
            t0 = clock()
            batch = scheduler.schedule()
            if batch.empty():
                raise RuntimeError("the scheduler has requests but nothing can run: the cache pool is too "
                                   "small for the request at the head of the queue")
            t1 = clock()
            rows, handle = self.launch(scheduler, batch, (previous[1], previous[2]) if previous else None)
            t2 = clock()
            waited = 0.0
            if previous is not None:         # the GPU is busy with `batch`: now read the step before it
                p_batch, p_rows, p_handle = previous
                got = p_handle.result()
                waited = clock() - t2
                scheduler.resolve(p_batch, {e.request_id: t for e, t in zip(p_rows, got)})
                previous = None
            decode_only = all(len(e.tokens) == 1 for e in batch.entries)
            if self.lookahead and decode_only and scheduler.can_look_ahead(batch):
                scheduler.update_pending(batch)
                previous = (batch, rows, handle)
                stats["lookahead_steps"] += 1
            else:
                t3 = clock()
                got = handle.result()
                waited += clock() - t3
                tokens = {e.request_id: t for e, t in zip(rows, got)}
                for r in scheduler.update(batch, tokens):
                    on_finished(r)
            stats["steps"] += 1
            now = clock()
            stats["sched_seconds"] += t1 - t0
            stats["launch_seconds"] += t2 - t1
            stats["wait_seconds"] += waited
            stats["update_seconds"] += now - t2 - waited
            if decode_only:
                stats["decode_steps"] += 1
                stats["decode_tokens"] += len(batch.entries)
                stats["decode_seconds"] += now - t_mark
                stats["d2h_bytes_per_step"] = max(stats["d2h_bytes_per_step"], 4 * len(rows))
                stats["h2d_bytes_per_step"] = max(stats["h2d_bytes_per_step"], self.engine.last_h2d_bytes)
            else:                        # a step that brings at least one prompt portion (decoded tokens may ride along)
                stats["prompt_steps"] += 1
                stats["prompt_step_tokens"] += sum(len(e.tokens) for e in batch.entries)
                stats["prompt_seconds"] += now - t_mark
            t_mark = now
        assert previous is None
        stats["preemptions"] = scheduler.num_preemptions
        self.last_stats = stats
        self.engine.check_status()

    def server(self, receive: Callable[[bool], Optional[List[int]]], emit: Callable[[int, List[int]], None],
               max_new_tokens: int = 256, temperature: float = 0.0, seed: int = 0) -> None:
        """Serve until `receive(True)` returns None.  receive(wait) yields the next prompt
        (token ids) or None; with wait=False it must not block.  emit(request_id, tokens)
        gets every finished request (runtime/LLM.h:221-263)."""
        scheduler = Scheduler(self.engine.cache, self.scheduler_config)

        def submit(prompt):
            rid = scheduler.add_request(list(prompt), max_new_tokens, temperature, seed)
            if rid < 0:
                emit(-1, [])

        def poll():
            while True:
                more = receive(False)
                if more is None:
                    return
                submit(more)

        def finished(r: Request):
            self.engine.check_status()           # tokens leave only after the kernels that made them reported no failure
            emit(r.id, r.generated)

        while True:
            prompt = receive(True)
            if prompt is None:
                break
            submit(prompt)
            # the same loop as generate(): decode steps are launched one ahead of the host
            self._run_to_idle(scheduler, finished, poll)
