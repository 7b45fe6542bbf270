"""Options of the engine that config.json does not hold.

Names follow the reference where it has them: max_num_seqs,
max_num_batched_tokens, eos_token_id (runtime/Scheduler.h:60-64), max_seq_len
and max_new_tokens (model/llm/tiny_llama.cpp:19-20), the 16-token KV block
(kv/KV_Layout.h:2) and the 0.9 share of free memory that the cache pool takes
(tensor/Arena.h:49).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

DTYPES = ("bfloat16", "float32")


@dataclass
class EngineOptions:
    dtype: str = "bfloat16"
    kv_block_size: int = 16
    max_num_seqs: int = 8
    max_num_batched_tokens: int = 512
    max_seq_len: Optional[int] = None          # default: max_position_embeddings
    num_kv_blocks: Optional[int] = None        # pages per cache group; default from memory
    gpu_memory_utilization: float = 0.9
    max_logit_rows: Optional[int] = None       # most rows of logits one step returns
    use_cuda_graphs: bool = True
    device: str = "cuda:0"
    poison_freed_pages: bool = False           # debug: pages that go back to the pool are overwritten with a huge value

    def validate(self) -> None:
        if self.dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {DTYPES}, got {self.dtype!r}")
        if self.kv_block_size not in (8, 16, 32, 64):
            raise ValueError(f"kv_block_size must be 8, 16, 32 or 64, got {self.kv_block_size}")
        if self.max_num_seqs <= 0 or self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_seqs and max_num_batched_tokens must be positive")
        if self.max_num_seqs > self.max_num_batched_tokens:
            raise ValueError("max_num_seqs must not exceed max_num_batched_tokens")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
