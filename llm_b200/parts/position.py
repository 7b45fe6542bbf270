"""Rotary position encoding (rotate-half).

Tables as the reference builds them (kernel/embedding/RoPECache.h:15-20):
inv_i = theta^(-2i/HS), angle = pos * inv_i formed in float32, cos and sin of that
angle, for pos < max_position and i < HS/2.  The power and the cos/sin are evaluated
in float64 on the host and rounded once, so the table holds the correctly rounded
values of the 32-bit angle.
"""
from __future__ import annotations

import numpy as np
import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    role = "position"

    def __init__(self, head_dim: int, theta: float, max_position: int, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        if head_dim % 2:
            raise ValueError(f"rope: head_dim {head_dim} must be even")
        self.head_dim, self.theta, self.max_position = head_dim, float(theta), int(max_position)
        self._tables = None

    def host_tables(self):
        half = self.head_dim // 2
        i = np.arange(half, dtype=np.float64)
        inv = np.power(np.float64(self.theta), -2.0 * i / self.head_dim).astype(np.float32)
        pos = np.arange(self.max_position, dtype=np.float32)
        ang = (pos[:, None] * inv[None, :]).astype(np.float32)        # one float32 product
        ang64 = ang.astype(np.float64)
        return np.cos(ang64).astype(np.float32), np.sin(ang64).astype(np.float32)

    def tables(self):
        """(cos, sin), float32 [max_position, head_dim/2] on the device."""
        if self._tables is None:
            key = (self.head_dim, self.theta, self.max_position, str(self.device))
            if key not in _TABLE_CACHE:      # layers with the same constants share one table
                c, s = self.host_tables()
                _TABLE_CACHE[key] = (torch.from_numpy(c).to(self.device).contiguous(),
                                     torch.from_numpy(s).to(self.device).contiguous())
            self._tables = _TABLE_CACHE[key]
        return self._tables


_TABLE_CACHE = {}


register_part("position", "rope", RotaryEmbedding)
