"""RMSNorm on the residual stream.

y = x * rsqrt(mean(x^2) + eps) * gain with the sum, the root and the scaling in
float32 (kernel/LayerNorm/RMSNorm.h:13-30,40-42 of the reference).  The stream's
pending term is added to the residual in the same pass
(kernel/residual/Residual.h:17-19 is a separate kernel there).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, ResidualStream, register_part


class RMSNorm(Part):
    role = "norm"

    def __init__(self, size: int, eps: float, prefix: str, dtype, device):
        super().__init__(prefix, dtype, device)
        self.size = size
        self.eps = float(eps)
        self.gain = None

    def parameters(self):
        return {self.name("weight"): ParamInfo((self.size,), kind="gain", init="ones_normal")}

    def bind(self, tensors):
        self.gain = tensors[self.name("weight")]

    def forward(self, stream: ResidualStream, ctx, tag: str = "normed") -> torch.Tensor:
        out = ctx.workspace.get(tag, stream.rows, self.size, self.dtype)
        ops.add_rmsnorm(stream.resid, stream.pending, self.gain, out, stream.rows, self.eps)
        stream.pending = None
        return out

    def forward_rows(self, rows_f32: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        """Norm of float32 rows that are not a stream (the gathered rows before the head)."""
        ops.add_rmsnorm(rows_f32, None, self.gain, out, n_rows, self.eps)
        return out


register_part("norm", "rmsnorm", RMSNorm)
