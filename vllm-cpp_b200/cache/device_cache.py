"""Device side of the cache: which caches share a group, and the tensors pages and slots index.

The host runtime (csrc/runtime/cache_manager.*) hands out page ids per *group*
and one slot per request; this module decides the groups from what the model's
mixers keep, and owns the tensors:

* a "kv" group -- all caches whose mixers keep keys and values of the same shape
  and the same window -- is one tensor
  ``[caches in group, num_pages, 2 (K,V), kv_heads, page_size, head_dim]``: a page id
  means the same page in every cache of the group (as a page of the reference
  covers every layer, src/kv_cache_manager.cpp:15-29), head-major inside a page so
  the keys of one KV head are contiguous runs of page_size * head_dim;
* a "state" group is ``[caches in group, num_slots, *shape]``: per-request state
  of fixed size, addressed by the request's slot.  It is zeroed for a request
  whose first tokens arrive (start position 0).

The reference has one pool for all layers and no per-request state
(src/kv_cache_manager.h:50-147).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import CacheSpec

_TORCH_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "int32": torch.int32}


@dataclass
class CacheGroup:
    spec: CacheSpec
    cache_ids: list          # caches of the model that live in this group, in tensor order
    paged: bool
    runtime_index: int = -1  # index of the group in the host CacheManager (paged groups only)


@dataclass
class KVCacheView:
    group: int               # index into the step context's groups
    pages: torch.Tensor      # [num_pages, 2, kv_heads, page_size, head_dim] of one cache


@dataclass
class StateCacheView:
    group: int
    state: torch.Tensor      # [num_slots, *shape] of one cache


class CacheLayout:
    """Groups of a model's caches; paged groups come first and map one-to-one to host pools."""

    def __init__(self, cache_specs: dict[int, CacheSpec]):
        self.groups: list[CacheGroup] = []
        by_spec: dict[CacheSpec, CacheGroup] = {}
        for cid in sorted(cache_specs):
            spec = cache_specs[cid]
            if spec not in by_spec:
                by_spec[spec] = CacheGroup(spec, [], paged=(spec.kind == "kv"))
                self.groups.append(by_spec[spec])
            by_spec[spec].cache_ids.append(cid)
        self.groups.sort(key=lambda g: not g.paged)
        self.paged = [g for g in self.groups if g.paged]
        for i, g in enumerate(self.paged):
            g.runtime_index = i
        self.where = {cid: (gi, g.cache_ids.index(cid)) for gi, g in enumerate(self.groups) for cid in g.cache_ids}

    def page_size_of(self, group: CacheGroup, page_size: int) -> int:
        """Tokens per page of a paged group: what its caches asked for, else the engine's ``page_size``."""
        return group.spec.page_size or page_size

    def num_pages_of(self, group: CacheGroup, page_size: int, num_pages: int) -> int:
        """Every paged group gets a pool for as many tokens as ``num_pages`` pages of the engine's size hold."""
        return num_pages * page_size // self.page_size_of(group, page_size)

    def runtime_groups(self, runtime, page_size: int, num_pages: int):
        """GroupSpec list for the host CacheManager, one pool per paged group."""
        return [runtime.GroupSpec(self.page_size_of(g, page_size), self.num_pages_of(g, page_size, num_pages), g.spec.window)
                for g in self.paged]

    def bytes_per_token(self, elem_size: int) -> int:
        return sum(len(g.cache_ids) * 2 * g.spec.num_kv_heads * g.spec.head_dim * elem_size for g in self.paged)


class DeviceCache:
    def __init__(self, layout: CacheLayout, page_size: int, num_pages: int, num_slots: int, dtype: torch.dtype, device):
        self.layout = layout
        self.page_size, self.num_pages, self.num_slots = page_size, num_pages, num_slots
        self.tensors: list[torch.Tensor] = []
        for g in layout.groups:
            n = len(g.cache_ids)
            if g.paged:
                shape = (n, layout.num_pages_of(g, page_size, num_pages), 2, g.spec.num_kv_heads,
                         layout.page_size_of(g, page_size), g.spec.head_dim)
                self.tensors.append(torch.zeros(shape, dtype=dtype, device=device))
            else:
                sdt = _TORCH_DTYPES[g.spec.dtype]
                self.tensors.append(torch.full((n, num_slots) + tuple(g.spec.shape), g.spec.initial_value, dtype=sdt, device=device))
        self.views = {}
        for cid, (gi, li) in layout.where.items():
            t = self.tensors[gi][li]
            self.views[cid] = KVCacheView(gi, t) if layout.groups[gi].paged else StateCacheView(gi, t)

    def reset_state(self, ctx) -> None:
        """Sets the fixed-size state of the requests whose entries start at position 0 to its initial value: a
        kernel that reads the step's own integers, so that a captured step does it as well."""
        from .. import ops
        for g, t in zip(self.layout.groups, self.tensors):
            if not g.paged:
                ops.state_reset(t, ctx.slots, ctx.q_len, ctx.ctx_len, ctx.E, g.spec.initial_value, ctx.status)

    def poison(self, value: float = float("nan")) -> None:
        """Fills every page with a value that shows if anything reads what it should not."""
        for g, t in zip(self.layout.groups, self.tensors):
            if g.paged:
                t.fill_(value)

    def poison_pages(self, runtime_group: int, pages: list[int], value: float = float("nan")) -> None:
        """The same for the pages a request gives back: whoever gets them next must write before it reads."""
        pages = [p for p in pages if p >= 0]
        if not pages:
            return
        for g, t in zip(self.layout.groups, self.tensors):
            if g.paged and g.runtime_index == runtime_group:
                t[:, torch.tensor(pages, dtype=torch.long, device=t.device)] = value
