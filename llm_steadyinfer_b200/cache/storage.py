"""Device tensors behind the cache manager: per group one key and one value tensor
``[layers_in_group, num_pages, kv_heads, page_size, head_dim]`` and, for mixers with
fixed-size state, one tensor ``[slots, *shape]`` per layer. The reference keeps
``[L, num_blocks, block_size, kv_dim]`` in fp32 (src/source/scheduler/kv_manager.cpp:41-53);
here a page holds each head's rows contiguously and has the compute dtype.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from .manager import CacheLayout, CacheManager


@dataclass
class LayerCache:
    """What one layer's mixer sees of the cache during a step."""
    k: Optional[torch.Tensor]              # [num_pages, kv_heads, page_size, head_dim]
    v: Optional[torch.Tensor]
    block_table: Optional[torch.Tensor]    # int32 [num_seqs, table_width] of the layer's group, this step
    page_size: int
    writes: bool                           # False for a layer that reads another layer's cache
    state: Optional[torch.Tensor]          # [slots, *shape] or None
    group: Optional[int]


class CacheStorage:
    def __init__(self, layout: CacheLayout, manager: CacheManager, dtype: torch.dtype, device):
        self.layout = layout
        self.manager = manager
        self.dtype = dtype
        self.device = torch.device(device)
        self.keys: List[torch.Tensor] = []
        self.values: List[torch.Tensor] = []
        ps = manager.page_size
        for g, grp in enumerate(manager.groups):
            shape = (len(grp.layers), grp.pool.num_pages, grp.need.num_kv_heads, ps, grp.need.head_dim)
            self.keys.append(torch.zeros(shape, dtype=dtype, device=self.device))
            self.values.append(torch.zeros(shape, dtype=dtype, device=self.device))
        self.states: List[Optional[torch.Tensor]] = []
        for s in layout.states:
            self.states.append(None if s is None else torch.zeros(
                (manager.slots.num_slots, *s.shape), dtype=s.dtype, device=self.device))

    def bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for t in self.keys + self.values)
        return n + sum(t.numel() * t.element_size() for t in self.states if t is not None)

    def zero_new_slots(self) -> None:
        """State of requests admitted (or reset) since the last call starts at zero."""
        slots = self.manager.new_slots
        if slots and any(t is not None for t in self.states):
            idx = torch.tensor(sorted(set(slots)), dtype=torch.long, device=self.device)
            for t in self.states:
                if t is not None:
                    t.index_fill_(0, idx, 0)
        slots.clear()

    def layer_views(self, tables: List[Optional[torch.Tensor]]) -> List[LayerCache]:
        """``tables[g]``: this step's device block table of group g."""
        views = []
        ps = self.manager.page_size
        for i in range(len(self.layout.needs)):
            g = self.layout.layer_group[i]
            if g is None:
                views.append(LayerCache(None, None, None, ps, False, self.states[i], None))
                continue
            j = self.layout.layer_index_in_group[i]
            views.append(LayerCache(self.keys[g][j], self.values[g][j], tables[g], ps,
                                    self.layout.cache_from[i] is None, self.states[i], g))
        return views
