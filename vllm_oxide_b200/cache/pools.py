"""Device memory of the cache and its host-side bookkeeping, laid out from a model's parts.

Every call of the model's run order that writes a cache gets pages of its own: the tensors
its mixer's `CacheSpec` names (by default K and V), each [num_pages, heads, page_size, width]
in the compute dtype or the one the spec gives (inside a page the layout is head-major, so one
(page, head) is one contiguous page_size x width tile; the reference's pool is
[slot, kv_heads, head_dim], crates/engine/src/backend/paged.rs:25-27, and leaves the layout to
the backend, crates/engine/src/backend/mod.rs:10-12). Calls whose mixers ask for the same kind
of cache (all keys, or a window of w) with the same tensors form a group: one page pool and one block table per request serve all of them, a page number being
valid in every layer of its group. Mixers with fixed-size state get a tensor
[max_seqs, *shape] indexed by the request's state slot. The page bookkeeping itself is the
native `CacheManager`.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..csrc.build import runtime_module
from ..errors import CapacityError, ConfigError
from ..parts.base import CacheSpec, LayerCache, ModelSpec


class CachePools:
    def __init__(self, spec: ModelSpec, page_size: int, max_seqs: int, dtype: torch.dtype, device: str,
                 num_pages: Optional[int] = None, pool_bytes: Optional[int] = None):
        rt = runtime_module()
        self.page_size, self.dtype, self.device = page_size, dtype, device
        # cache number -> spec, from the calls that write it
        cache_specs: Dict[int, CacheSpec] = {}
        for call in spec.schedule:
            mixer = spec.blocks[call.layer].mixer
            cs = mixer.cache_spec()
            if call.cache is None:
                continue
            if cs is None:
                raise ConfigError(f"layer {call.layer} is scheduled with cache {call.cache} but its mixer keeps none")
            if call.write:
                if call.cache in cache_specs and cache_specs[call.cache] != cs:
                    raise ConfigError(f"cache {call.cache} is written by mixers with different needs")
                cache_specs[call.cache] = cs
        for call in spec.schedule:
            if call.cache is not None and call.cache not in cache_specs:
                raise ConfigError(f"cache {call.cache} is read by layer {call.layer} but no call writes it")
            if call.cache is not None and not call.write:
                if spec.blocks[call.layer].mixer.cache_spec() != cache_specs[call.cache]:
                    raise ConfigError(f"layer {call.layer} reads cache {call.cache} whose shape differs from its own")
        self.cache_specs = cache_specs
        group_keys: List[tuple] = []
        self.cache_group: Dict[int, int] = {}
        for c in sorted(cache_specs):
            key = cache_specs[c].group_key()
            if key not in group_keys:
                group_keys.append(key)
            self.cache_group[c] = group_keys.index(key)
        self.group_keys = group_keys
        # bytes one page costs in each group (over all caches of the group)
        self.page_bytes = [0] * len(group_keys)
        for c, cs in cache_specs.items():
            for t in cs.paged_tensors():
                if t.heads <= 0 or t.width <= 0:
                    raise ConfigError(f"cache {c}: a paged tensor needs positive heads and width, got {t}")
                es = torch.empty((), dtype=t.dtype or dtype).element_size()
                self.page_bytes[self.cache_group[c]] += t.heads * t.width * page_size * es
        if num_pages is None:
            total = sum(self.page_bytes)
            if not total:
                num_pages = 1
            else:
                if pool_bytes is None:
                    raise ConfigError("either num_pages or a cache budget in bytes is needed")
                # the reference's sizing (crates/engine/src/model.rs:202-212): budget / bytes per page
                num_pages = int(pool_bytes // total)
                if num_pages < 1:
                    raise CapacityError("cache budget (pages)", 1, num_pages)
        self.num_pages = int(num_pages)
        groups = []
        for key in group_keys:
            kind, window = key[0], key[1]
            if kind not in ("full", "window"):
                raise ConfigError(f"cache kind {kind!r} is not known (full or window)")
            groups.append(rt.GroupSpec(rt.WINDOW if kind == "window" else rt.FULL, int(window), self.num_pages))
        self.manager = rt.CacheManager(page_size, groups, max_seqs)
        # cache number -> its tensors, in the order of the spec (K, V by default)
        self.kv: Dict[int, tuple] = {}
        for c, cs in cache_specs.items():
            self.kv[c] = tuple(torch.zeros((self.num_pages, t.heads, page_size, t.width), dtype=t.dtype or dtype, device=device)
                               for t in cs.paged_tensors())
        # fixed-size per-request state, one tensor per call whose mixer asks for it
        self.state: Dict[int, torch.Tensor] = {}
        for idx, call in enumerate(spec.schedule):
            ss = spec.blocks[call.layer].mixer.state_spec()
            if ss is not None:
                self.state[idx] = torch.zeros((max_seqs,) + tuple(ss.shape), dtype=ss.dtype, device=device)

    @property
    def num_groups(self) -> int:
        return len(self.group_keys)

    def layer_cache(self, cache: Optional[int], write: bool) -> Optional[LayerCache]:
        if cache is None:
            return None
        return LayerCache(tensors=self.kv[cache], group=self.cache_group[cache], write=write)

    def reset_slot(self, slot: int) -> None:
        """A request was admitted to this slot: its state starts from zero."""
        for t in self.state.values():
            t[slot].zero_()

    def bytes_per_token(self) -> int:
        return sum(self.page_bytes) // self.page_size

