"""What every part is, and the registries that map a kind to its class.

A part is built from its own parameters (sizes and constants) plus the compute
dtype and the device; it names its tensors, receives them once, and runs on the
rows it is given.  No part knows which model it is in: the ModelSpec chooses parts
layer by layer through these registries, and a new kind is added by registering a
class here (tests register toy kinds without touching the package).

Roles and what each must provide, beyond Part:

  norm       forward(stream, ctx) -> rows [T, H] in the compute dtype; folds the
             stream's pending term into the residual first.
  mixer      cache_need() / state_need(); forward(x, ctx, view) -> [T, H].
  ffn        forward(x, ctx) -> [T, H].
  position   either tables() -> (cos, sin) float32 [max_position, head_dim/2] for the kernels that
             rotate half a head against the other (fused with the cache store), or apply(q, k,
             ctx): its own in-place transform of the step's queries [T, heads, head_dim] and new
             keys [T, kv_heads, head_dim] (views of one buffer), run by the mixer between the
             projection and the cache store.  A part with neither leaves q and k as they are.
  block      forward(stream, ctx, view): arranges norm / mixer / ffn on the stream.
  embedding  forward(ctx, stream): fills the residual stream from token ids.
  head       logits(stream, ctx, final_norm, buffers) -> float32 logits [R, V] at ctx.logit_rows:
             everything after the last layer (row gather, final norm, projection, and whatever
             else a model does to its logits) belongs to this role.

A part whose launches are sized from host-side data of the step (ctx.host_*), so that a captured
CUDA graph of one step would be wrong for another, says so with is_graph_safe(ctx) -> False; the
engine then runs that step without capture or replay.  children() names the parts a part is
built from (the position part inside a mixer), so that the engine can ask them too.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch


@dataclass(frozen=True)
class ParamInfo:
    """One tensor a part expects from the checkpoint.

    kind: "matrix" is kept in the compute dtype; "gain" is a small vector kept in
    float32; "int_table" is kept as int32.  init names the random-weights rule:
    "normal" N(0, 0.02), "ones_normal" 1 + N(0, 0.01), "zeros"."""

    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values a mixer keeps per token: every past token ("full") or only the
    last `window` of them ("window")."""

    kind: str
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self):
        return (self.kind, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one tensor of this shape per live request,
    zeroed when the request is admitted."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


class Part:
    role = "part"

    def __init__(self, prefix: str, dtype: torch.dtype, device: torch.device):
        self.prefix = prefix
        self.dtype = dtype
        self.device = device

    def name(self, local: str) -> str:
        return f"{self.prefix}.{local}" if self.prefix else local

    def parameters(self) -> Dict[str, ParamInfo]:
        """Checkpoint name -> what is expected there."""
        return {}

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by parameters(), already on the device and in the
        dtype their kind asks for.  Called once."""

    def children(self):
        """Parts that this part is built from."""
        return []

    def is_graph_safe(self, ctx) -> bool:
        """Whether this step's launches of the part depend only on the step's numbers of entries,
        tokens and wanted rows (and the key bucket), so that a captured graph may be replayed."""
        return True


_REGISTRIES: Dict[str, Dict[str, Callable]] = {
    role: {} for role in ("norm", "mixer", "ffn", "position", "block", "embedding", "head")
}


def register_part(role: str, kind: str, cls: Callable) -> None:
    if role not in _REGISTRIES:
        raise KeyError(f"unknown role '{role}'; roles: {sorted(_REGISTRIES)}")
    _REGISTRIES[role][kind] = cls


def part_class(role: str, kind: str) -> Callable:
    try:
        return _REGISTRIES[role][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRIES.get(role, {}))) or "(none)"
        raise KeyError(f"no {role} of kind '{kind}' is registered; known: {known}") from None


def build_part(role: str, spec, dtype: torch.dtype, device: torch.device):
    """spec: a PartSpec (kind, params, prefix)."""
    return part_class(role, spec.kind)(**spec.params, prefix=spec.prefix, dtype=dtype, device=device)


class ResidualStream:
    """The hidden state between parts: a float32 residual plus, possibly, a term that
    is still to be added to it.  Keeping the last part's output pending lets the next
    norm add it and normalise in one pass over the row."""

    def __init__(self, resid: torch.Tensor, rows: int):
        self.resid = resid            # [max_rows, H] float32
        self.rows = rows
        self.pending: Optional[torch.Tensor] = None   # [rows, H] compute dtype
