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


class SampleHandle:
    """Tokens that are being sampled: `device` holds them on the GPU (for feeding the next
    step), result() waits for the copy to the host and returns them as ints."""

    def __init__(self, device: torch.Tensor, host: torch.Tensor, rows: int, event):
        self.device, self._host, self.rows, self._event = device, host, rows, event

    def result(self) -> List[int]:
        if self.rows == 0:
            return []
        self._event.synchronize()
        return self._host[:self.rows].tolist()


class Sampler:
    """Two sets of buffers, used in turn, so that the tokens of one step can still be read (by
    the host, and by the next step on the device) while the following step is sampled."""

    def __init__(self, max_rows: int, device: torch.device):
        self.device = device
        self.max_rows = max_rows
        self._host = [torch.zeros((2, max_rows), dtype=torch.float32).pin_memory() for _ in range(2)]
        self._dev = [torch.zeros((2, max_rows), dtype=torch.float32, device=device) for _ in range(2)]
        self._out = [torch.zeros(max_rows, dtype=torch.int32, device=device) for _ in range(2)]
        self._out_host = [torch.zeros(max_rows, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._turn = 0

    def sample_async(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> SampleHandle:
        """One token per row of logits [R, V] (float32, device), without waiting for them."""
        rows = logits.shape[0]
        if rows > self.max_rows:
            raise ValueError(f"{rows} rows exceed the sampler's limit {self.max_rows}")
        k = self._turn
        self._turn ^= 1
        out = self._out[k]
        if rows == 0:
            return SampleHandle(out, self._out_host[k], 0, None)
        if any(t > 0.0 for t in temperatures):
            h = self._host[k]
            h[0, :rows] = torch.tensor(list(temperatures), dtype=torch.float32)
            h[1, :rows] = torch.tensor(list(uniforms), dtype=torch.float32)
            self._dev[k].copy_(h, non_blocking=True)
            ops.sample_rows(out, logits, rows, self._dev[k][0], self._dev[k][1])
        else:
            ops.sample_rows(out, logits, rows)
        self._out_host[k].copy_(out, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return SampleHandle(out, self._out_host[k], rows, event)

    def sample(self, logits: torch.Tensor, temperatures: Sequence[float], uniforms: Sequence[float]) -> List[int]:
        """One token per row of logits [R, V]; returns host ints."""
        return self.sample_async(logits, temperatures, uniforms).result()
