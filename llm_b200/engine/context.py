"""What a step hands to the parts: the batch's metadata on the device, the cache
and state views of the layer that is running, and scratch buffers.

The metadata is what the reference's Engine::prepare builds per step
(runtime/Engine.h:52-71): per entry the token offsets, per token its position and
its place in the cache, and the entries' block tables.  Here it also carries which
batch entry a token belongs to (so that prompt portions and decoded tokens share
one batch), the rows whose logits are wanted, and one table and slot map per cache
group.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch


class Workspace:
    """Scratch buffers by tag, sized for the most rows a step may bring, allocated at
    first use and kept: their addresses stay fixed, which CUDA-graph replay needs."""

    def __init__(self, max_rows: int, device: torch.device):
        self.max_rows = max_rows
        self.device = device
        self._buffers: Dict[Tuple[str, int, torch.dtype], torch.Tensor] = {}

    def get(self, tag: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        if rows > self.max_rows:
            raise ValueError(f"workspace '{tag}': {rows} rows exceed the step limit {self.max_rows}")
        key = (tag, cols, dtype)
        buf = self._buffers.get(key)
        if buf is None:
            buf = torch.empty((self.max_rows, cols), dtype=dtype, device=self.device)
            self._buffers[key] = buf
        return buf[:rows]

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class GroupView:
    """One cache group as a step sees it."""

    page_size: int
    block_table: torch.Tensor      # int32 [entries, table_width] on the device
    slot_map: torch.Tensor         # int32 [tokens]: page * page_size + offset of each new token
    kind: str = "full"
    window: Optional[int] = None


@dataclass
class LayerView:
    """Cache and state of the layer occurrence that is running."""

    group: Optional[GroupView] = None
    k_pages: Optional[torch.Tensor] = None     # [pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    owns_cache: bool = True                    # False: reads another layer's pages, writes none
    state: Optional[torch.Tensor] = None       # [slots, *shape]


@dataclass
class StepContext:
    n_tokens: int
    n_entries: int
    n_logit_rows: int
    # device, int32
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_entry: torch.Tensor
    cu_tokens: torch.Tensor        # [entries + 1]
    kv_lens: torch.Tensor          # [entries]: tokens held after this step
    state_slots: torch.Tensor      # [entries]
    logit_rows: torch.Tensor       # [rows]
    status: torch.Tensor           # [4]: word 0 is set by kernels that meet bad input, 1 and 2 by tensor-core kernels whose wait gave up
    # host copies for planning (not read by kernels)
    host_entry_tokens: np.ndarray = None      # [entries] tokens per entry
    host_entry_start: np.ndarray = None       # [entries] first position of each entry
    host_state_slots: np.ndarray = None       # [entries] state slot of each entry's request
    groups: Dict[int, GroupView] = field(default_factory=dict)
    workspace: Workspace = None
    capturing: bool = False
    kv_bucket: int = 0                         # longest request of the step, rounded up to 256 keys
    layer_views: List[LayerView] = None        # cache and state of every layer occurrence, over this step's metadata

    @property
    def max_entry_tokens(self) -> int:
        return int(self.host_entry_tokens.max()) if self.n_entries else 0

    @property
    def decode_only(self) -> bool:
        return self.n_entries > 0 and self.max_entry_tokens == 1
