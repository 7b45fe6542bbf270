"""How a layer's parts are arranged on the residual stream.

"prenorm": x += mixer(norm1(x)); x += ffn(norm2(x)), the arrangement of the
reference's block (model/llm/tiny_llama.cpp:29-34).  Each sum is left pending on
the stream and folded in by the next norm.
"""
from __future__ import annotations

from .base import ResidualStream, build_part, register_part


class PreNormBlock:
    role = "block"
    roles = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "ffn": "ffn"}

    def __init__(self, part_specs, dtype, device):
        missing = [r for r in self.roles if r not in part_specs]
        if missing:
            raise ValueError(f"prenorm block lacks parts {missing}")
        self.parts = {r: build_part(self.roles[r], part_specs[r], dtype, device) for r in self.roles}
        self.norm1, self.mixer = self.parts["norm1"], self.parts["mixer"]
        self.norm2, self.ffn = self.parts["norm2"], self.parts["ffn"]

    def forward(self, stream: ResidualStream, ctx, view) -> None:
        stream.pending = self.mixer.forward(self.norm1.forward(stream, ctx), ctx, view)
        stream.pending = self.ffn.forward(self.norm2.forward(stream, ctx), ctx)


register_part("block", "prenorm", PreNormBlock)
