"""Device memory behind the cache manager's bookkeeping.

Per layer with a paged need: one tensor ``[pages, kv_heads, page_size, head_dim]``
for each entry of the need (keys and values for attention; whatever a mixer names),
indexed by the page ids of the layer's group (the reference's per-layer views are
``[P, B, kv_heads, hd]``, include/inferx/core/kv_cache.h:40-150; heads are moved
outward here so that one head's part of a page is contiguous).  Per state need of a
mixer: one tensor ``[slots, *shape]``.  Everything starts from zero; a slot is zeroed again when it
is handed to a new request.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..parts.base import LayerCache, PagedKvNeed, StateNeed
from .manager import CacheManager, is_paged_need


class CacheStorage:
    def __init__(self, cache_needs_per_layer, manager: CacheManager, dtype: torch.dtype, device):
        self.manager = manager
        self.device = torch.device(device)
        self.paged: Dict[int, Dict[str, torch.Tensor]] = {}
        self.group_of_layer: Dict[int, int] = {}
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        window_to_group = {g.window: i for i, g in enumerate(manager.groups)}
        for layer, needs in enumerate(cache_needs_per_layer):
            for need in needs:
                if is_paged_need(need):
                    g = window_to_group[int(need.window)]
                    if self.group_of_layer.setdefault(layer, g) != g:
                        raise TypeError(f"layer {layer}: paged needs with different windows; "
                                        "one block table addresses a layer's pages")
                    pages = manager.pools[g].num_pages
                    shape = (pages, need.kv_heads, manager.page_size, need.head_dim)
                    per = self.paged.setdefault(layer, {})
                    for name in getattr(need, "entries", ("k", "v")):
                        if name in per:
                            raise TypeError(f"layer {layer}: paged entry {name!r} named twice")
                        per[name] = torch.zeros(shape, dtype=getattr(need, "dtype", None) or dtype,
                                                device=self.device)
                elif isinstance(need, StateNeed) or hasattr(need, "shape"):
                    self.state.setdefault(layer, {})[need.name] = torch.zeros(
                        (manager.max_slots,) + tuple(need.shape), dtype=need.dtype,
                        device=self.device)
                else:
                    raise TypeError(f"layer {layer}: unknown cache need {need!r}")

    def bytes(self) -> int:
        n = 0
        for per in self.paged.values():
            n += sum(t.numel() * t.element_size() for t in per.values())
        for per in self.state.values():
            n += sum(t.numel() * t.element_size() for t in per.values())
        return n

    def layer_caches(self, schedule) -> List[LayerCache]:
        """One ``LayerCache`` per schedule entry."""
        out = []
        for e in schedule:
            src = e.cache_layer
            out.append(LayerCache(
                group=self.group_of_layer.get(src, -1), pages=self.paged.get(src, {}),
                writes=e.writes_cache, state=self.state.get(src, {})))
        return out

    def zero_slots(self, slots) -> None:
        if not slots:
            return
        idx = torch.tensor(list(slots), dtype=torch.long, device=self.device)
        for per in self.state.values():
            for t in per.values():
                t.index_fill_(0, idx, 0)
