"""A ModelSpec turned into parts, and the plan of caches and states that its layer
order implies.

The order is a list of layer indices.  Every occurrence of a layer in it that keeps
keys and values gets a cache instance of its own (a layer that runs twice must not
overwrite what its first run stored); a layer with `cache_of` reads the instance of
the latest earlier occurrence of that other layer.  Instances with the same need
(every key, or a window of w) form one group and share page ids and block tables.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..cache.storage import CacheInstance
from ..config.model_config import parse_config
from ..models.spec import ModelSpec
from ..parts.base import CacheNeed, ParamInfo, ResidualStream, StateNeed, build_part, part_class


@dataclass
class Occurrence:
    layer: int
    cache_instance: Optional[int]     # index into Model.cache_instances
    owns_cache: bool
    state_instance: Optional[int]


class Model:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device):
        spec.validate()
        self.spec, self.dtype, self.device = spec, dtype, device
        self.embedding = build_part("embedding", spec.embedding, dtype, device)
        self.blocks = [part_class("block", layer.block)(layer.parts, dtype, device) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, dtype, device) if spec.final_norm is not None else None
        self.head = build_part("head", spec.head, dtype, device)

        self._graph_askers = None
        self.group_keys: List[tuple] = []            # (kind, window) per group
        self.cache_instances: List[CacheInstance] = []
        self.state_needs: List[StateNeed] = []
        self.occurrences: List[Occurrence] = []
        latest: Dict[int, int] = {}                  # layer -> cache instance of its latest occurrence
        for layer_idx in spec.order:
            layer = spec.layers[layer_idx]
            mixer = self.blocks[layer_idx].mixer
            need: Optional[CacheNeed] = mixer.cache_need()
            state: Optional[StateNeed] = mixer.state_need()
            inst, owns = None, True
            if layer.cache_of is not None:
                if need is not None:
                    raise ValueError(f"layer {layer_idx} borrows the cache of layer {layer.cache_of} but its "
                                     f"mixer asks for one of its own")
                if layer.cache_of not in latest:
                    raise ValueError(f"layer {layer_idx} reads the cache of layer {layer.cache_of}, which has "
                                     f"not run before it in the order")
                inst, owns = latest[layer.cache_of], False
            elif need is not None:
                key = need.group_key()
                if key not in self.group_keys:
                    self.group_keys.append(key)
                inst = len(self.cache_instances)
                self.cache_instances.append(CacheInstance(self.group_keys.index(key), need.num_kv_heads, need.head_dim))
                latest[layer_idx] = inst
            st = None
            if state is not None:
                st = len(self.state_needs)
                self.state_needs.append(state)
            self.occurrences.append(Occurrence(layer_idx, inst, owns, st))

    def parts(self):
        """Every part of the model, the parts that parts are built from included."""
        def walk(part):
            yield part
            for child in getattr(part, "children", lambda: [])():
                yield from walk(child)
        yield from walk(self.embedding)
        for block in self.blocks:
            for part in block.parts.values():
                yield from walk(part)
        if self.final_norm is not None:
            yield from walk(self.final_norm)
        yield from walk(self.head)

    def is_graph_safe(self, ctx) -> bool:
        """Whether every part says that this step may be captured in, or replayed from, a CUDA graph.
        Only parts that bring an answer of their own are asked (found once)."""
        if self._graph_askers is None:
            from ..parts.base import Part
            self._graph_askers = [p for p in self.parts() if hasattr(p, "is_graph_safe")
                                  and getattr(type(p), "is_graph_safe", None) is not Part.is_graph_safe]
        return all(p.is_graph_safe(ctx) for p in self._graph_askers)

    def parameters(self) -> Dict[str, ParamInfo]:
        out: Dict[str, ParamInfo] = {}
        for part in self.parts():
            for name, info in part.parameters().items():
                if name in out and out[name] != info:
                    raise ValueError(f"tensor '{name}' is declared twice with different shapes")
                out[name] = info
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.bind(tensors)

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for part in self.parts():
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    def forward(self, ctx, stream: ResidualStream, views) -> None:
        """Embedding and every layer occurrence in order; leaves the last term pending."""
        self.embedding.forward(ctx, stream)
        for occ, view in zip(self.occurrences, views):
            self.blocks[occ.layer].forward(stream, ctx, view)


def collect_parameters(config_dict: dict) -> Dict[str, ParamInfo]:
    """Names and shapes that a model of this config.json expects (no device needed)."""
    arch, cfg = parse_config(config_dict)
    return Model(arch.build_spec(cfg), torch.bfloat16, torch.device("cpu")).parameters()
