"""SwiGLU feed-forward: down( silu(gate(x)) * up(x) ).

The reference runs gate and up as two products and the activation as a third kernel
(model/modules/MLP.h:10-13, kernel/activation/SwiGLU.h:31-33); here gate and up are
one product over a stacked weight, and with many rows (prompts) the product's epilogue applies
the activation itself, so that the stacked product never reaches memory.
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, register_part
from .linear import FUSE_PARTIALS, linear, linear_swiglu


class SwiGLU(Part):
    role = "ffn"

    def __init__(self, hidden_size: int, intermediate_size: int, bias: bool = False, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        self.hidden_size, self.intermediate_size = hidden_size, intermediate_size
        self.bias = bool(bias)        # the three projections carry bias vectors (model/modules/MLP.h:9-13)
        self.w_gate_up = None
        self.w_down = None
        self.b_gate_up = None
        self.b_down = None

    def parameters(self):
        p = {
            self.name("gate_proj.weight"): ParamInfo((self.intermediate_size, self.hidden_size)),
            self.name("up_proj.weight"): ParamInfo((self.intermediate_size, self.hidden_size)),
            self.name("down_proj.weight"): ParamInfo((self.hidden_size, self.intermediate_size)),
        }
        if self.bias:
            p[self.name("gate_proj.bias")] = ParamInfo((self.intermediate_size,), kind="gain", init="normal")
            p[self.name("up_proj.bias")] = ParamInfo((self.intermediate_size,), kind="gain", init="normal")
            p[self.name("down_proj.bias")] = ParamInfo((self.hidden_size,), kind="gain", init="normal")
        return p

    def bind(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.name("gate_proj.weight")],
                                    tensors[self.name("up_proj.weight")]], dim=0).contiguous()
        self.w_down = tensors[self.name("down_proj.weight")].contiguous()
        if self.bias:
            self.b_gate_up = torch.cat([tensors[self.name("gate_proj.bias")], tensors[self.name("up_proj.bias")]]).contiguous()
            self.b_down = tensors[self.name("down_proj.bias")].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        T, ws = ctx.n_tokens, ctx.workspace
        act = ws.get("ffn_act", T, self.intermediate_size, self.dtype)
        if self.bias or not linear_swiglu(x, self.w_gate_up, act, T):
            gate_up = linear(x, self.w_gate_up, ws.get("gate_up", T, 2 * self.intermediate_size, self.dtype), T,
                             allow_partial=FUSE_PARTIALS, bias=self.b_gate_up)
            ops.silu_mul(act, gate_up, T)
        return linear(act, self.w_down, ws.get("ffn_out", T, self.hidden_size, self.dtype), T, allow_partial=FUSE_PARTIALS,
                      bias=self.b_down)


register_part("ffn", "swiglu", SwiGLU)
