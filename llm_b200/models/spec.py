"""A model as data: which parts each layer is made of, with their sizes and
constants, and the order in which layers run.  Architectures produce a ModelSpec
from their typed config; the engine builds parts from it through the registries
of llm_b200.parts and knows nothing of any architecture by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: its kind (a registry key), its constructor parameters, and the
    prefix of its tensors' names in the checkpoint."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement and the parts it arranges, by role.

    cache_of: index of the layer whose cache this layer's mixer reads instead of
    keeping one of its own (None = its own)."""

    block: str
    parts: Dict[str, PartSpec]
    cache_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_position: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[int, ...]            # indices into layers, in execution order; may repeat
    final_norm: Optional[PartSpec]    # None: the head takes the stream as it is
    head: PartSpec
    eos_token_id: Optional[int] = None

    def validate(self) -> None:
        n = len(self.layers)
        for i in self.order:
            if not (0 <= i < n):
                raise ValueError(f"order names layer {i}, but there are {n} layers")
        for i, layer in enumerate(self.layers):
            if layer.cache_of is not None:
                if not (0 <= layer.cache_of < n) or layer.cache_of == i:
                    raise ValueError(f"layer {i}: cache_of={layer.cache_of} is not another layer")
                if self.layers[layer.cache_of].cache_of is not None:
                    raise ValueError(f"layer {i}: cache_of={layer.cache_of} itself borrows a cache")
