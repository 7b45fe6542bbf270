"""Device side of the cache: the pages' memory and the state slots' memory.

Per cache instance (one per layer occurrence that keeps keys and values) two tensors
[pages, kv_heads, page_size, head_dim], keys and values, so that one (page, head) is
a contiguous [page_size, head_dim] tile.  The reference keeps
[block][16][kv_heads][head_dim] (kv/KV_pool.h:17-18,76-79); putting the head outside
the token makes a page of one head a single contiguous tile for bulk copies.  A page
id is valid in every instance of its group, as a block id is valid in every layer of
the reference (kv/KV_pool.h:71-73).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class CacheInstance:
    group: int
    num_kv_heads: int
    head_dim: int


def element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


def bytes_per_page(instances: List[CacheInstance], group: int, page_size: int, dtype: torch.dtype) -> int:
    """Bytes that one more page of this group costs over all its instances (K and V)."""
    return sum(2 * page_size * i.num_kv_heads * i.head_dim * element_size(dtype)
               for i in instances if i.group == group)


POISON = 1e30


class CacheStorage:
    def __init__(self, instances: List[CacheInstance], pages_per_group: List[int], page_size: int,
                 dtype: torch.dtype, device: torch.device):
        self.instances = instances
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        for inst in instances:
            shape = (pages_per_group[inst.group], inst.num_kv_heads, page_size, inst.head_dim)
            self.k.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v.append(torch.zeros(shape, dtype=dtype, device=device))

    def pages(self, instance: int) -> Tuple[torch.Tensor, torch.Tensor]:
        return self.k[instance], self.v[instance]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k + self.v)

    def poison(self, group: int, pages: List[int]) -> None:
        """Debug aid: fill these pages of every instance of the group with POISON, so that a kernel
        that reads a key or value its request no longer (or not yet) holds gives logits that are far
        off instead of nearly right.  The value is huge but finite, not NaN: a kernel may load a
        whole tile and give the keys beyond a request's length weight zero, which is sound for any
        finite leftover."""
        if not pages:
            return
        idx = torch.tensor(sorted(set(pages)), dtype=torch.long, device=self.k[0].device if self.k else None)
        for inst, k, v in zip(self.instances, self.k, self.v):
            if inst.group == group:
                k.index_fill_(0, idx, POISON)
                v.index_fill_(0, idx, POISON)


class StateStorage:
    """One tensor [slots, *shape] per state instance; a slot is zeroed when a request
    takes it."""

    def __init__(self, needs, max_requests: int, device: torch.device):
        self.tensors = [torch.zeros((max_requests, *n.shape), dtype=n.dtype, device=device) for n in needs]

    def zero_slots(self, slots: List[int]) -> None:
        if not slots or not self.tensors:
            return
        for t in self.tensors:
            for s in slots:
                t[s].zero_()

    def tensor(self, instance: int) -> torch.Tensor:
        return self.tensors[instance]
