"""Next-token choice above the step function.

Greedy argmax with ties to the lowest id is what the reference has
(kernel/sampling/Argmax.h:20-43).  Temperature sampling is added: softmax of
logits / temperature in float32 and an inverse-CDF draw.  The uniform number of a
draw is a function of (seed, request id, position of the new token) only, three
rounds of the splitmix64 finaliser, so that what a request samples does not depend
on what else is in the batch or on how its prompt was cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..csrc import ops

_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_for(seed: int, request_id: int, position: int) -> float:
    """A number in [0, 1) with 24 random bits."""
    z = _mix64(seed & _M64)
    z = _mix64(z ^ (request_id & _M64))
    z = _mix64(z ^ (position & _M64))
    return (z >> 40) / float(1 << 24)


@dataclass
class SamplingParams:
    temperature: float = 0.0          # 0 = greedy
    seed: int = 0
    max_new_tokens: int = 256
    eos_token_id: Optional[int] = None   # None: the model's; -1: never stop at a token
    ignore_eos: bool = False


class Sampler:
    def __init__(self, max_rows: int, device: torch.device):
        self.device = device
        self.max_rows = max_rows
        self._host = torch.zeros((2, max_rows), dtype=torch.float32).pin_memory()
        self._dev = torch.zeros((2, max_rows), dtype=torch.float32, device=device)
        self._out = torch.zeros(max_rows, dtype=torch.int32, device=device)
        self._out_host = torch.zeros(max_rows, dtype=torch.int32).pin_memory()

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> List[int]:
        """One token per row of logits [R, V] (float32, device); returns host ints."""
        rows = logits.shape[0]
        if rows == 0:
            return []
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the sampler's limit {self.max_rows}")
        if any(t > 0.0 for t in temperatures):
            self._host[0, :rows] = torch.tensor(list(temperatures), dtype=torch.float32)
            self._host[1, :rows] = torch.tensor(list(uniforms), dtype=torch.float32)
            self._dev.copy_(self._host, non_blocking=True)
            ops.sample_rows(self._out, logits, rows, self._dev[0], self._dev[1])
        else:
            ops.sample_rows(self._out, logits, rows)
        self._out_host.copy_(self._out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self._out_host[:rows].tolist()
