"""The device side of the cache: pools of pages per group of layers, and state slots.

Layers (runs of the schedule that own a cache) are grouped by what their mixers ask for:
paged keys and values with the same window, number of KV heads and head size share a group,
hence a page pool, a free list and block tables (``return_b200/cache/manager.py``).  The pool of
a group is one tensor ``[layers, 2, num_pages, Hkv, page_size, D]`` in the activation dtype
(index 0 of the second axis: keys, 1: values), so one page id addresses a slab in every layer of
the group, as in the reference (rollout/cache.py:19-24), and one (page, kv head) tile is
contiguous.  A mixer whose cache is one vector a token (``LatentCacheNeed``: a latent that is key and value for all
heads) gets a group of its own kind by (window, width) and one tensor ``[layers, num_pages, page_size, width]``.
A mixer that asks for state of fixed size gets ``[max_reside + 1, *shape]``, one row per
request slot and a last one that belongs to no request (the padding rows of a captured decode step
point at it) (after rollout/cache.py:340-360).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..parts.base import BuildEnv, CompositeNeed, KVCacheNeed, KVView, LatentCacheNeed, LayerContext, StateNeed
from .manager import CacheManager, GroupSpec


class CacheStorage:
    def __init__(self, needs: List[object], page_size: int, num_pages: int, max_reside: int, env: BuildEnv,
                 longest_append: Optional[int] = None):
        """``num_pages``: pages of a group that keeps every key (the pool's capacity in tokens / page size).
        A group that keeps a window gets only what ``max_reside`` requests can hold of it at a time: the
        window plus the longest run of tokens one step may append (``longest_append``; None: unknown, the
        group then gets ``num_pages`` too), in pages, plus one for the ragged ends."""
        self.env = env
        self.page_size = page_size
        self.max_reside = max_reside
        signature_to_group: Dict[Tuple, int] = {}
        self.group_specs: List[GroupSpec] = []
        self._group_layers: List[int] = []
        self._group_shape: List[Tuple[int, int]] = []
        self.entry_place: Dict[Tuple, Tuple[int, int]] = {}    # key of a need -> (group, layer in group)
        self._state_needs: Dict[Tuple, StateNeed] = {}
        self._composite: Dict[Tuple, Tuple[str, ...]] = {}     # key of a composite need -> its children's names

        def register(key: Tuple, need) -> None:
            """``key``: (schedule index,) for a run's own need, (schedule index, child, ...) below a composite one."""
            if need is None:
                return
            if isinstance(need, CompositeNeed):
                self._composite[key] = tuple(name for name, _ in need.children)
                for name, child in need.children:
                    register(key + (name,), child)
            elif isinstance(need, (KVCacheNeed, LatentCacheNeed)):
                latent = isinstance(need, LatentCacheNeed)
                # a latent is one vector a token: stored as "0 heads" of its width, one tensor instead of keys and values
                sig = (need.window, 0, need.width) if latent else (need.window, need.num_kv_heads, need.head_dim)
                if sig not in signature_to_group:
                    signature_to_group[sig] = len(self.group_specs)
                    name = "full" if need.window is None else f"window{need.window}"
                    pages = num_pages
                    if need.window is not None and longest_append is not None:
                        per_request = (need.window + longest_append + page_size - 1) // page_size + 1
                        pages = max(1, min(num_pages, max_reside * per_request))
                    self.group_specs.append(GroupSpec(f"{name}_latent{need.width}" if latent else
                                                      f"{name}_h{need.num_kv_heads}_d{need.head_dim}",
                                                      page_size, pages, need.window))
                    self._group_layers.append(0)
                    self._group_shape.append(sig[1:])
                g = signature_to_group[sig]
                self.entry_place[key] = (g, self._group_layers[g])
                self._group_layers[g] += 1
            elif isinstance(need, StateNeed):
                self._state_needs[key] = need
            else:
                raise TypeError(f"schedule entry {key[0]}: unknown cache need {need!r}")

        for index, need in enumerate(needs):
            register((index,), need)
        if not self.group_specs:
            # a model without paged layers still counts tokens per request
            self.group_specs.append(GroupSpec("none", page_size, num_pages, None))
            self._group_layers.append(0)
            self._group_shape.append((0, 0))
        self.pools: List[Optional[torch.Tensor]] = []
        self._layer_views: Dict[Tuple[int, int], Tuple[torch.Tensor, torch.Tensor]] = {}
        self.states: Dict[Tuple, torch.Tensor] = {}

    def make_manager(self) -> CacheManager:
        manager = CacheManager(self.group_specs, self.max_reside)
        manager.on_slot_taken.append(self.reset_slot)
        manager.truncatable = not self._state_needs
        return manager

    def allocate(self) -> None:
        dev, dt = self.env.device, self.env.act_dtype
        self.pools = []
        self._layer_views = {}
        for spec, layers, (hkv, d) in zip(self.group_specs, self._group_layers, self._group_shape):
            if layers == 0:
                self.pools.append(None)
                continue
            if hkv == 0:                     # latents: [layers, pages, page_size, width]
                self.pools.append(torch.zeros((layers, spec.num_pages, spec.page_size, d), dtype=dt, device=dev))
                continue
            self.pools.append(torch.zeros((layers, 2, spec.num_pages, hkv, spec.page_size, d), dtype=dt, device=dev))
        self.states = {i: torch.zeros((self.max_reside + 1,) + tuple(n.shape), dtype=n.dtype, device=dev)
                       for i, n in self._state_needs.items()}

    def bytes_per_token(self) -> int:
        total = 0
        for layers, (hkv, d) in zip(self._group_layers, self._group_shape):
            total += layers * (2 * hkv if hkv else 1) * d * torch.empty((), dtype=self.env.act_dtype).element_size()
        return total

    def poison(self) -> None:
        """Fills every page with NaN, so that a read of a slot nobody wrote shows in the logits."""
        for p in self.pools:
            if p is not None:
                p.fill_(float("nan"))

    def reset_slot(self, slot: int) -> None:
        """A request that takes a slot starts from zero state."""
        for t in self.states.values():
            t[slot].zero_()                  # in stream order: after the last step of whoever held the slot before

    def layer_context(self, owner_index: int, batch, write: bool) -> LayerContext:
        return self._context((owner_index,), batch, write)

    def _context(self, key: Tuple, batch, write: bool) -> LayerContext:
        ctx = LayerContext(batch=batch, write_cache=write)
        place = self.entry_place.get(key)
        if place is not None:
            g, layer = place
            views = self._layer_views.get(place)
            if views is None:                # the views of a layer's keys and values are made once
                pool = self.pools[g]
                views = self._layer_views[place] = ((pool[layer], None) if self._group_shape[g][0] == 0 else
                                                    (pool[layer, 0], pool[layer, 1]))
            ctx.kv = KVView(k=views[0], v=views[1], block_table=batch.block_tables[g],
                            page_size=self.group_specs[g].page_size, group=g)
        if key in self.states:
            ctx.state = self.states[key]
        names = self._composite.get(key)
        if names is not None:
            ctx.children = {name: self._context(key + (name,), batch, write) for name in names}
        return ctx
