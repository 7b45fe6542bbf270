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
from .scheduler import Request, ScheduledBatch, Scheduler, SchedulerConfig


class LLM:
    def __init__(self, model: str, dtype: str = "bfloat16", max_num_seqs: int = 8,
                 max_num_batched_tokens: int = 512, max_seq_len: Optional[int] = None,
                 eos_token_id: Optional[int] = None, kv_block_size: int = 16,
                 num_kv_blocks: Optional[int] = None, gpu_memory_utilization: float = 0.9,
                 use_cuda_graphs: bool = True, device: str = "cuda:0", random_config: Optional[dict] = None,
                 random_seed: int = 0):
        """model: a folder with config.json and model.safetensors, or None together with
        random_config (a config.json's contents) for seeded random weights."""
        options = EngineOptions(dtype=dtype, kv_block_size=kv_block_size, max_num_seqs=max_num_seqs,
                                max_num_batched_tokens=max_num_batched_tokens, max_seq_len=max_seq_len,
                                num_kv_blocks=num_kv_blocks, gpu_memory_utilization=gpu_memory_utilization,
                                max_logit_rows=max_num_seqs, use_cuda_graphs=use_cuda_graphs, device=device)
        self.engine = Engine(model, options, random_config=random_config, random_seed=random_seed)
        if eos_token_id is None:
            eos_token_id = self.engine.spec.eos_token_id
        self.eos_token_id = eos_token_id
        self.scheduler_config = SchedulerConfig(max_num_seqs, max_num_batched_tokens, eos_token_id)
        self.sampler = Sampler(max_num_seqs, self.engine.device)

    # ---- one scheduled batch through the model: tokens in, next tokens out ----
    def inference(self, scheduler: Scheduler, batch: ScheduledBatch) -> Dict[int, int]:
        entries, rows = [], []
        for e in batch.entries:
            entries.append(StepEntry(e.request_id, e.tokens, [len(e.tokens) - 1] if e.samples else []))
            if e.samples:
                rows.append(e)
        logits = self.engine.step(entries)
        temps, unis = [], []
        for e in rows:
            r = scheduler.requests[e.request_id]
            temps.append(r.temperature)
            unis.append(uniform_for(r.seed, r.id, e.start + len(e.tokens)) if r.temperature > 0 else 0.0)
        tokens = self.sampler.sample(logits, temps, unis)
        return {e.request_id: t for e, t in zip(rows, tokens)}

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

    def _run_to_idle(self, scheduler: Scheduler, on_finished: Callable[[Request], None]) -> None:
        """Steps until no request is left.  Host-side times of the steps that only decode
        (schedule, copy in, run, sample, copy out, update) are kept in last_stats, as the
        reference's driver keeps sched/wait/update times per step (runtime/Driver.h:16,74-83)."""
        stats = {"steps": 0, "decode_steps": 0, "decode_tokens": 0, "decode_seconds": 0.0,
                 "h2d_bytes_per_step": self.engine.layout.total * 4, "d2h_bytes_per_step": 0}
        while scheduler.num_requests():
            t0 = time.perf_counter()
            batch = scheduler.schedule()
            if batch.empty():
                raise RuntimeError("the scheduler has requests but nothing can run: the cache pool is too "
                                   "small for the request at the head of the queue")
            tokens = self.inference(scheduler, batch)       # ends with the device-to-host copy of the tokens
            for r in scheduler.update(batch, tokens):
                on_finished(r)
            stats["steps"] += 1
            if all(len(e.tokens) == 1 for e in batch.entries):
                stats["decode_steps"] += 1
                stats["decode_tokens"] += len(batch.entries)
                stats["decode_seconds"] += time.perf_counter() - t0
                stats["d2h_bytes_per_step"] = max(stats["d2h_bytes_per_step"], 4 * len(tokens))
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

        while True:
            prompt = receive(True)
            if prompt is None:
                break
            submit(prompt)
            while scheduler.num_requests():
                while True:
                    more = receive(False)
                    if more is None:
                        break
                    submit(more)
                batch = scheduler.schedule()
                if batch.empty():
                    raise RuntimeError("the scheduler has requests but nothing can run")
                for r in scheduler.update(batch, self.inference(scheduler, batch)):
                    emit(r.id, r.generated)
