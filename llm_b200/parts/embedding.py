"""Token embedding in, logits out.

Embedding: a row copy without scaling (kernel/embedding/TokenEmbedding.h:12-17),
written straight into the float32 residual stream.  Head: logits = rows W^T in
float32 at the rows that were asked for; untied unless the spec ties it to the
embedding table (model/modules/LMHead.h:5-13 is always untied and runs every row).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import ParamInfo, Part, ResidualStream, register_part
from .linear import linear


class TokenEmbedding(Part):
    role = "embedding"

    def __init__(self, vocab_size: int, hidden_size: int, prefix: str = "", dtype=None, device=None):
        super().__init__(prefix, dtype, device)
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.table = None

    def parameters(self):
        return {self.name("weight"): ParamInfo((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        self.table = tensors[self.name("weight")].contiguous()

    def forward(self, ctx, stream: ResidualStream) -> None:
        ops.embedding(stream.resid, self.table, ctx.token_ids, ctx.n_tokens, ctx.status)
        stream.pending = None


class LMHead(Part):
    role = "head"

    def __init__(self, hidden_size: int, vocab_size: int, tied_to=None, prefix: str = "", dtype=None,
                 device=None):
        super().__init__(prefix, dtype, device)
        self.hidden_size, self.vocab_size, self.tied_to = hidden_size, vocab_size, tied_to
        self.weight = None

    def parameters(self):
        if self.tied_to:
            return {}
        return {self.name("weight"): ParamInfo((self.vocab_size, self.hidden_size))}

    def bind(self, tensors):
        self.weight = tensors[self.tied_to if self.tied_to else self.name("weight")].contiguous()

    def forward(self, rows: torch.Tensor, n_rows: int, out: torch.Tensor) -> torch.Tensor:
        return linear(rows, self.weight, out, n_rows)

    def logits(self, stream: ResidualStream, ctx, final_norm, buffers) -> torch.Tensor:
        """Everything after the last layer: the wanted rows of the stream (with its pending term)
        are gathered, normalised by final_norm (None: the model has none) and projected.  buffers:
        (float32 rows, rows in the compute dtype, float32 logits), each with room for
        ctx.n_logit_rows rows, at addresses that stay fixed between steps."""
        rows, normed, out = buffers
        R = ctx.n_logit_rows
        ops.gather_rows(rows, stream.resid, stream.pending, ctx.logit_rows, R)
        if final_norm is not None:
            final_norm.forward_rows(rows, R, normed)
        else:
            ops.cast_rows(normed, rows, R)
        return linear(normed, self.weight, out, R)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
