"""The cache manager: device planes of keys and values, block tables, state slots.

It is built from the needs that the model's schedule entries declare
(:class:`cajeta_llm_b200.parts.base.KvNeed`, :class:`...StateNeed`):

* entries whose mixers cache keys and values are sorted into groups by
  (kv heads, head size, window); a group owns one K and one V tensor
  ``[planes, pages, kv_heads, page_tokens, head_dim]`` with one plane per entry, and one
  pool of page ids (:mod:`cajeta_llm_b200.cache.pages`);
* entries whose mixers keep per-request state of fixed size get a tensor
  ``[max_seqs, *shape]`` indexed by the request's slot, zeroed when a slot is admitted.
  (The reference has no recurrent state; its fixed-size per-slot things are scratch and
  histograms, model/DeviceKv.cajeta:44-48, model/MoeFfn.cajeta:2830-2836.)

All bookkeeping is on the host, in native code (:mod:`cajeta_llm_b200.cache.pages`); the
block-table rows of the requests in a step are uploaded with the step's other metadata.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..parts.base import KvNeed, StateNeed
from .pages import CacheBooks, CacheError, GroupSpec


class CacheManager:
    def __init__(self, kv_needs: Sequence[Optional[KvNeed]], state_needs: Sequence[Optional[StateNeed]],
                 cache_from: Sequence[Optional[int]], page_tokens: int, max_seqs: int, max_tokens_per_seq: int,
                 num_pages, cache_dtype: torch.dtype, device: torch.device | str | None):
        """``kv_needs[i]`` / ``state_needs[i]`` belong to schedule entry ``i``;
        ``cache_from[i]`` names the entry whose plane entry ``i`` reads instead of owning
        one.  ``num_pages`` is the pool size of every group, or a function
        ``GroupSpec -> pages`` that sizes each group by its own need (a windowed group holds
        far fewer pages a request than one that keeps every key).  ``device=None`` keeps only
        the books (no tensors), for tests of the bookkeeping."""
        n = len(kv_needs)
        self.page_tokens = page_tokens
        self.max_seqs = max_seqs
        self.device = torch.device(device) if device is not None else None
        self.cache_dtype = cache_dtype
        specs: List[GroupSpec] = []
        self.entry_group: List[Optional[int]] = [None] * n
        self.entry_plane: List[Optional[int]] = [None] * n
        plane_count: List[int] = []
        for i in range(n):
            need = kv_needs[i]
            if need is None or cache_from[i] is not None:
                continue
            spec = GroupSpec(need.kv_heads, need.head_dim, need.window)
            if spec not in specs:
                specs.append(spec)
                plane_count.append(0)
            g = specs.index(spec)
            self.entry_group[i] = g
            self.entry_plane[i] = plane_count[g]
            plane_count[g] += 1
        for i in range(n):
            src = cache_from[i]
            if src is None:
                continue
            if self.entry_group[src] is None:
                raise CacheError(f"schedule entry {i} reads the cache of entry {src}, which caches nothing")
            a, b = kv_needs[i], kv_needs[src]
            if a is None or (a.kv_heads, a.head_dim) != (b.kv_heads, b.head_dim):
                raise CacheError(f"schedule entry {i} cannot read the cache of entry {src}: head layout differs")
            if b.window > 0 and (a.window == 0 or a.window > b.window):
                raise CacheError(f"schedule entry {i} (window {a.window}) cannot read the cache of entry {src}, "
                                 f"which keeps only a window of {b.window}")
            self.entry_group[i] = self.entry_group[src]
            self.entry_plane[i] = self.entry_plane[src]
        self.group_specs = specs
        counts = [int(num_pages(spec)) if callable(num_pages) else int(num_pages) for spec in specs]
        self.group_pages = counts
        self.books = CacheBooks(specs, counts, page_tokens, max_seqs, max_tokens_per_seq)
        self.k: List[torch.Tensor] = []
        self.v: List[torch.Tensor] = []
        self.state: Dict[int, torch.Tensor] = {}
        if self.device is not None:
            for spec, planes, pages in zip(specs, plane_count, counts):
                shape = (planes, pages, spec.kv_heads, page_tokens, spec.head_dim)
                self.k.append(torch.zeros(shape, dtype=cache_dtype, device=self.device))
                self.v.append(torch.zeros(shape, dtype=cache_dtype, device=self.device))
            for i, need in enumerate(state_needs):
                if need is not None:
                    self.state[i] = torch.zeros((max_seqs,) + tuple(need.shape), dtype=need.dtype, device=self.device)

    # -- requests --------------------------------------------------------------------
    def admit(self) -> Optional[int]:
        slot = self.books.admit()
        if slot is not None:
            for t in self.state.values():
                t[slot].zero_()
        return slot

    def release(self, slot: int) -> None:
        self.books.release(slot)

    def length(self, slot: int) -> int:
        return int(self.books.length[slot])

    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        return self.books.pages_needed(slot, n_new)

    def pages_to_hold(self, slot: int, n_new: int, step_tokens: int = 0) -> List[int]:
        return self.books.pages_to_hold(slot, n_new, step_tokens)

    def free_pages(self) -> List[int]:
        return self.books.free_pages()

    def reserve(self, slot: int, n_new: int) -> bool:
        return self.books.reserve(slot, n_new)

    def commit(self, slot: int, n_new: int) -> None:
        self.books.commit(slot, n_new)

    # -- what a step needs -----------------------------------------------------------
    @property
    def num_groups(self) -> int:
        return len(self.group_specs)

    def table_rows(self, group: int, slots: Sequence[int], width: Optional[int] = None) -> np.ndarray:
        """Block-table rows of ``slots`` in ``group`` (int32 ``[len(slots), width]``)."""
        t = self.books.groups[group].table
        w = t.shape[1] if width is None else width
        return t[list(slots), :w]

    def table_width(self, slots: Sequence[int]) -> int:
        """Columns that cover every page the given slots have ever been given."""
        return self.books.table_width(slots)

    def plane(self, entry: int) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor], Optional[int]]:
        g = self.entry_group[entry]
        if g is None:
            return None, None, None
        p = self.entry_plane[entry]
        return self.k[g][p], self.v[g][p], g

    def bytes_per_token(self) -> int:
        """Cache bytes one token occupies over all planes."""
        size = torch.empty((), dtype=self.cache_dtype).element_size()
        total = 0
        for g, spec in enumerate(self.group_specs):
            planes = sum(1 for e, gg in enumerate(self.entry_group) if gg == g and self.entry_plane[e] is not None
                         and self._owns(e))
            total += 2 * planes * spec.kv_heads * spec.head_dim * size
        return total

    def _owns(self, entry: int) -> bool:
        g, p = self.entry_group[entry], self.entry_plane[entry]
        for e in range(entry):
            if self.entry_group[e] == g and self.entry_plane[e] == p:
                return False
        return True
