"""The books of the cache manager restated plainly in Python: pages, block tables, request
slots.  The engine's books are native code (``cajeta_llm_b200/csrc/host_books.cpp``); the tests
drive both with the same random orders of requests and compare every table, length and free
list after every call (``test_cache_books.py``).  Shares no code with the product path.

Keys and values live in pages of ``page_tokens`` positions.  Layers with the same
needs (kv heads, head size, window) form a *group*: the group has its own pool of
pages and its own free list, and a page id is shared by all layers of the group (each
layer has its own plane).  The reference's device pool does the same with its
"kinds" (model/KvPool.cajeta:11-17,170-210, model/KvFreeList.cajeta:4-60); its host
cache draws per (sequence, layer) instead (model/PagedKvCache.cajeta:54-127,284-309).

A request holds a *slot*: the row of its block table in every group and the index of
its fixed-size state.  Position ``p`` of a request lies in page
``table[slot][p // page_tokens]`` at ``p % page_tokens`` (model/KvPage.cajeta:15-19).

Pages are given back
* when the request is released (finish, cancel, preemption): all of them
  (model/PagedKvCache.cajeta:639-661, model/KvPool.cajeta:348-367);
* for a windowed group, as soon as every position of a page lies behind the window of
  the request's next token: with length ``L`` and window ``w`` the next token reads
  keys ``[L + 1 - w, L]`` (model/PagedKvCache.cajeta:382-388), so page ``j`` is given
  back when ``(j + 1) * page_tokens <= L + 1 - w``.
Reservation is all-or-nothing across groups and returns False when pages run out,
leaving the books unchanged (model/PagedKvCache.cajeta:200-207,
model/KvPool.cajeta:234-255).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np


class CacheError(RuntimeError):
    """A misuse of the cache books (double free, unknown slot, table overflow)."""


class PageAllocator:
    """Free list of one group's pages (LIFO, like the reference's free-list stack)."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise CacheError(f"num_pages must be >= 0, found {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._held = np.zeros(num_pages, dtype=bool)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) when fewer are free."""
        if n < 0:
            raise CacheError(f"cannot take {n} pages")
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            if self._held[p]:
                raise CacheError(f"page {p} handed out twice")
            self._held[p] = True
        return out

    def give_back(self, pages: Sequence[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise CacheError(f"page {p} does not exist")
            if not self._held[p]:
                raise CacheError(f"page {p} freed twice")
            self._held[p] = False
            self._free.append(p)

    def check(self) -> None:
        """No page lost, held twice or free twice."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in range(self.num_pages):
            if self._held[p] == (p in free):
                raise CacheError(f"page {p} is {'both held and free' if self._held[p] else 'neither held nor free'}")


@dataclass(frozen=True)
class GroupSpec:
    """Needs shared by the cache planes of one group."""

    kv_heads: int
    head_dim: int
    window: int      # 0: every key is kept


class GroupBook:
    """Block tables and page ownership of one group."""

    def __init__(self, spec: GroupSpec, num_pages: int, page_tokens: int, max_seqs: int, max_pages_per_seq: int):
        self.spec = spec
        self.page_tokens = page_tokens
        self.allocator = PageAllocator(num_pages)
        self.table = np.full((max_seqs, max_pages_per_seq), -1, dtype=np.int32)
        self.first_live = np.zeros(max_seqs, dtype=np.int64)   # lowest logical page still held
        self.next_page = np.zeros(max_seqs, dtype=np.int64)    # logical pages ever given (held: [first_live, next_page))

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_tokens)

    def pages_needed(self, slot: int, length: int, n_new: int) -> int:
        return max(0, self.pages_for(length + n_new) - int(self.next_page[slot]))

    def grow(self, slot: int, length: int, n_new: int, pages: List[int]) -> None:
        start = int(self.next_page[slot])
        if start + len(pages) > self.table.shape[1]:
            raise CacheError(f"request in slot {slot} needs {start + len(pages)} pages; a table row holds {self.table.shape[1]}")
        for i, p in enumerate(pages):
            self.table[slot, start + i] = p
        self.next_page[slot] = start + len(pages)

    def trim_window(self, slot: int, length: int) -> int:
        """Give back the pages that lie wholly behind the window of the next token."""
        w = self.spec.window
        if w <= 0:
            return 0
        dead_below = length + 1 - w                       # positions < dead_below are never read again
        if dead_below <= 0:
            return 0
        last_dead = min(dead_below // self.page_tokens, int(self.next_page[slot]))   # pages [first_live, last_dead) are dead
        first = int(self.first_live[slot])
        if last_dead <= first:
            return 0
        pages = [int(self.table[slot, j]) for j in range(first, last_dead)]
        self.allocator.give_back(pages)
        self.table[slot, first:last_dead] = -1
        self.first_live[slot] = last_dead
        return len(pages)

    def release(self, slot: int) -> int:
        first, nxt = int(self.first_live[slot]), int(self.next_page[slot])
        pages = [int(self.table[slot, j]) for j in range(first, nxt)]
        self.allocator.give_back(pages)
        self.table[slot, :nxt] = -1
        self.first_live[slot] = 0
        self.next_page[slot] = 0
        return len(pages)

    def held_pages(self, slot: int) -> List[int]:
        return [int(self.table[slot, j]) for j in range(int(self.first_live[slot]), int(self.next_page[slot]))]


class CacheBooks:
    """Slots, lengths and the per-group books of every live request."""

    def __init__(self, groups: Sequence[GroupSpec], num_pages: Sequence[int], page_tokens: int, max_seqs: int,
                 max_tokens_per_seq: int):
        if page_tokens < 1:
            raise CacheError(f"page_tokens must be >= 1, found {page_tokens}")
        if len(groups) != len(num_pages):
            raise CacheError("one page count per group is needed")
        self.page_tokens = page_tokens
        self.max_seqs = max_seqs
        self.max_tokens_per_seq = max_tokens_per_seq
        self.max_pages_per_seq = -(-max_tokens_per_seq // page_tokens)
        self.groups = [GroupBook(g, n, page_tokens, max_seqs, self.max_pages_per_seq) for g, n in zip(groups, num_pages)]
        self.length = np.zeros(max_seqs, dtype=np.int64)
        self.live = np.zeros(max_seqs, dtype=bool)
        self._free_slots: List[int] = list(range(max_seqs - 1, -1, -1))

    # -- slots -----------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return len(self._free_slots)

    def admit(self) -> Optional[int]:
        """A free slot for a new request (length 0), or None when all are taken."""
        if not self._free_slots:
            return None
        s = self._free_slots.pop()
        self.live[s] = True
        self.length[s] = 0
        return s

    def _need_live(self, slot: int) -> None:
        if not (0 <= slot < self.max_seqs) or not self.live[slot]:
            raise CacheError(f"slot {slot} holds no request")

    # -- pages -----------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """New pages per group that appending ``n_new`` tokens would draw."""
        self._need_live(slot)
        L = int(self.length[slot])
        return [g.pages_needed(slot, L, n_new) for g in self.groups]

    def free_pages(self) -> List[int]:
        return [g.allocator.free_count for g in self.groups]

    def fits(self, needs: Sequence[Sequence[int]]) -> bool:
        """Whether the summed per-group needs of several requests fit the free pages."""
        for gi, g in enumerate(self.groups):
            if sum(n[gi] for n in needs) > g.allocator.free_count:
                return False
        return True

    def reserve(self, slot: int, n_new: int) -> bool:
        """Make sure pages exist for positions ``[length, length + n_new)``; all or nothing."""
        self._need_live(slot)
        L = int(self.length[slot])
        if L + n_new > self.max_tokens_per_seq:
            raise CacheError(f"request in slot {slot} would reach {L + n_new} tokens; the limit is {self.max_tokens_per_seq}")
        needs = [g.pages_needed(slot, L, n_new) for g in self.groups]
        if any(n > g.allocator.free_count for n, g in zip(needs, self.groups)):
            return False
        for n, g in zip(needs, self.groups):
            pages = g.allocator.take(n)
            assert pages is not None
            g.grow(slot, L, n_new, pages)
        return True

    # -- one token for each of several requests (a decode step), the books' hot path -------------
    def reserve_one_each(self, slots: Sequence[int]) -> Optional[np.ndarray]:
        """``reserve(slot, 1)`` for every slot, all or nothing over the whole list.  Returns the
        requests' lengths (before the new token) or None when the pages are not there."""
        idx = np.asarray(slots, dtype=np.int64)
        if idx.size == 0:
            return np.zeros(0, dtype=np.int64)
        if idx.min() < 0 or idx.max() >= self.max_seqs or not self.live[idx].all():
            bad = [int(s) for s in idx if not (0 <= s < self.max_seqs) or not self.live[s]]
            raise CacheError(f"slot {bad[0]} holds no request")
        L = self.length[idx]
        if int(L.max()) + 1 > self.max_tokens_per_seq:
            s = int(idx[int(L.argmax())])
            raise CacheError(f"request in slot {s} would reach {int(L.max()) + 1} tokens; the limit is {self.max_tokens_per_seq}")
        wanting = []
        for g in self.groups:
            short = np.nonzero(-(-(L + 1) // self.page_tokens) > g.next_page[idx])[0]
            if short.size > g.allocator.free_count:
                return None
            wanting.append(short)
        for g, short in zip(self.groups, wanting):
            for i in short:
                pages = g.allocator.take(1)
                assert pages is not None
                g.grow(int(idx[i]), int(L[i]), 1, pages)
        return L

    def commit_one_each(self, slots: Sequence[int]) -> None:
        """``commit(slot, 1)`` for every slot."""
        idx = np.asarray(slots, dtype=np.int64)
        if idx.size == 0:
            return
        self.length[idx] += 1
        L = self.length[idx]
        for g in self.groups:
            if (-(-L // self.page_tokens) > g.next_page[idx]).any():
                raise CacheError("a token was committed without reserved pages")
            if g.spec.window > 0:
                for s, n in zip(idx, L):
                    g.trim_window(int(s), int(n))

    def commit(self, slot: int, n_new: int) -> None:
        """The step that wrote ``n_new`` tokens is launched: advance the length and give
        back pages that have passed behind a window."""
        self._need_live(slot)
        self.length[slot] += n_new
        L = int(self.length[slot])
        for g in self.groups:
            if g.pages_for(L) > int(g.next_page[slot]):
                raise CacheError(f"slot {slot}: committed {L} tokens without reserved pages")
            g.trim_window(slot, L)

    def release(self, slot: int) -> None:
        """Give back everything the request holds; the slot is free again."""
        self._need_live(slot)
        for g in self.groups:
            g.release(slot)
        self.length[slot] = 0
        self.live[slot] = False
        self._free_slots.append(slot)

    def check(self) -> None:
        """Invariants: no page lost, held twice or freed twice; tables agree with owners."""
        for g in self.groups:
            g.allocator.check()
            owners: Dict[int, int] = {}
            for s in range(self.max_seqs):
                held = g.held_pages(s)
                if not self.live[s] and held:
                    raise CacheError(f"free slot {s} still holds pages {held}")
                for p in held:
                    if p < 0:
                        raise CacheError(f"slot {s} has a hole in its live pages")
                    if p in owners:
                        raise CacheError(f"page {p} is held by slots {owners[p]} and {s}")
                    owners[p] = s
                row = g.table[s]
                live_range = set(range(int(g.first_live[s]), int(g.next_page[s])))
                for j in range(row.shape[0]):
                    if (row[j] >= 0) != (j in live_range):
                        raise CacheError(f"slot {s}: table entry {j} disagrees with the live range")
            if len(owners) != g.allocator.used_count:
                raise CacheError(f"{g.allocator.used_count} pages are out, {len(owners)} are in tables")
