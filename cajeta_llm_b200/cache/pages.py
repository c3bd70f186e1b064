"""The books of the cache manager: pages, block tables, request slots.

The bookkeeping itself is native code (``csrc/host_books.cpp``, compiled with the host
compiler and loaded through ctypes: no GPU and no CUDA toolkit is needed for it); this
module is its Python face.  Block tables, lengths and live ranges are numpy views of the
native arrays, not copies.

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

import ctypes
from dataclasses import dataclass
from typing import List, Optional, Sequence

import numpy as np

from ..csrc import build as _build


class CacheError(RuntimeError):
    """A misuse of the cache books (double free, unknown slot, table overflow)."""


_lib: Optional[ctypes.CDLL] = None
_P = ctypes.c_void_p
_IP = ctypes.POINTER(ctypes.c_int)


def _native() -> ctypes.CDLL:
    """The native books, compiled at first use."""
    global _lib
    if _lib is None:
        lib = ctypes.CDLL(_build.build("host_books"))
        c_int, c_ll = ctypes.c_int, ctypes.c_longlong
        sigs = {
            "cj_pages_create": (_P, [c_int]), "cj_pages_destroy": (None, [_P]), "cj_pages_error": (ctypes.c_char_p, [_P]),
            "cj_pages_free_count": (c_int, [_P]), "cj_pages_take": (c_int, [_P, c_int, _IP]),
            "cj_pages_give_back": (c_int, [_P, _IP, c_int]), "cj_pages_check": (c_int, [_P]),
            "cj_books_create": (_P, [c_int, _IP, _IP, c_int, c_int, c_int]), "cj_books_destroy": (None, [_P]),
            "cj_books_error": (ctypes.c_char_p, [_P]),
            "cj_books_length": (_P, [_P]), "cj_books_live": (_P, [_P]), "cj_books_table": (_P, [_P, c_int]),
            "cj_books_first_live": (_P, [_P, c_int]), "cj_books_next_page": (_P, [_P, c_int]),
            "cj_books_width": (c_int, [_P]), "cj_books_free_slots": (c_int, [_P]), "cj_books_free_count": (c_int, [_P, c_int]),
            "cj_books_admit": (c_int, [_P]), "cj_books_release": (c_int, [_P, c_int]),
            "cj_books_pages_needed": (c_int, [_P, c_int, c_int, _IP]), "cj_books_reserve": (c_int, [_P, c_int, c_int]),
            "cj_books_reserve_step": (c_int, [_P, _IP, _IP, c_int, _IP]), "cj_books_commit": (c_int, [_P, c_int, c_int]),
            "cj_books_reserve_one_each": (c_int, [_P, _IP, c_int, _P]), "cj_books_commit_one_each": (c_int, [_P, _IP, c_int]),
            "cj_books_table_width": (c_int, [_P, _IP, c_int]),
            "cj_books_layout_step": (c_ll, [_P, c_int, _IP, _IP, _IP, _IP, _IP, c_int, c_int, c_int, _P, c_ll]),
            "cj_books_check": (c_int, [_P]),
        }
        for name, (res, args) in sigs.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib


def _ints(values: Sequence[int]) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


def _ip(a: np.ndarray):
    return a.ctypes.data_as(_IP)


def _view(ptr: int, shape, dtype) -> np.ndarray:
    n = int(np.prod(shape))
    if n == 0 or not ptr:
        return np.zeros(shape, dtype=dtype)
    buf = (ctypes.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype).reshape(shape)


class PageAllocator:
    """Free list of one group's pages (a stack, like the reference's free list)."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise CacheError(f"num_pages must be >= 0, found {num_pages}")
        self._lib = _native()
        self._h = self._lib.cj_pages_create(num_pages)
        self.num_pages = num_pages

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.cj_pages_destroy(h)

    def _fail(self):
        raise CacheError(self._lib.cj_pages_error(self._h).decode())

    @property
    def free_count(self) -> int:
        return self._lib.cj_pages_free_count(self._h)

    @property
    def used_count(self) -> int:
        return self.num_pages - self.free_count

    def take(self, n: int) -> Optional[List[int]]:
        """``n`` pages, or None (and nothing taken) when fewer are free."""
        out = np.empty(max(n, 1), dtype=np.int32)
        st = self._lib.cj_pages_take(self._h, n, _ip(out))
        if st < 0:
            self._fail()
        return out[:n].tolist() if st else None

    def give_back(self, pages: Sequence[int]) -> None:
        a = _ints(pages)
        if self._lib.cj_pages_give_back(self._h, _ip(a), a.size) < 0:
            self._fail()

    def check(self) -> None:
        """No page lost, held twice or free twice."""
        if self._lib.cj_pages_check(self._h) < 0:
            self._fail()


@dataclass(frozen=True)
class GroupSpec:
    """Needs shared by the cache planes of one group."""

    kv_heads: int
    head_dim: int
    window: int      # 0: every key is kept


class _GroupPages:
    """Page counts of one group of the books."""

    def __init__(self, books: "CacheBooks", index: int, num_pages: int):
        self._books, self._index, self.num_pages = books, index, num_pages

    @property
    def free_count(self) -> int:
        return self._books._lib.cj_books_free_count(self._books._h, self._index)

    @property
    def used_count(self) -> int:
        return self.num_pages - self.free_count


class GroupBook:
    """Block tables and page ownership of one group, as views of the native books."""

    def __init__(self, books: "CacheBooks", index: int, spec: GroupSpec, num_pages: int):
        lib, h = books._lib, books._h
        self.spec = spec
        self.page_tokens = books.page_tokens
        self.allocator = _GroupPages(books, index, num_pages)
        self.table = _view(lib.cj_books_table(h, index), (books.max_seqs, books.max_pages_per_seq), np.int32)
        self.first_live = _view(lib.cj_books_first_live(h, index), (books.max_seqs,), np.int64)   # lowest logical page still held
        self.next_page = _view(lib.cj_books_next_page(h, index), (books.max_seqs,), np.int64)     # logical pages ever given

    def pages_for(self, length: int) -> int:
        return -(-length // self.page_tokens)

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
        self._lib = _native()
        self.page_tokens = page_tokens
        self.max_seqs = max_seqs
        self.max_tokens_per_seq = max_tokens_per_seq
        self.max_pages_per_seq = -(-max_tokens_per_seq // page_tokens)
        windows, counts = _ints([g.window for g in groups]), _ints(list(num_pages))
        self._h = self._lib.cj_books_create(len(groups), _ip(windows), _ip(counts), page_tokens, max_seqs, max_tokens_per_seq)
        if not self._h:
            raise CacheError(f"the books cannot be made for {len(groups)} groups of {list(num_pages)} pages, "
                             f"{max_seqs} requests of {max_tokens_per_seq} tokens")
        self.groups = [GroupBook(self, i, g, n) for i, (g, n) in enumerate(zip(groups, num_pages))]
        self.length = _view(self._lib.cj_books_length(self._h), (max_seqs,), np.int64)
        self.live = _view(self._lib.cj_books_live(self._h), (max_seqs,), np.bool_)
        self._needs = np.zeros(max(1, len(groups)), dtype=np.int32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            # the views must not outlive the arrays they look at
            self.groups, self.length, self.live = [], None, None
            self._lib.cj_books_destroy(h)

    def _fail(self):
        raise CacheError(self._lib.cj_books_error(self._h).decode())

    # -- slots -----------------------------------------------------------------------
    @property
    def free_slots(self) -> int:
        return self._lib.cj_books_free_slots(self._h)

    def admit(self) -> Optional[int]:
        """A free slot for a new request (length 0), or None when all are taken."""
        s = self._lib.cj_books_admit(self._h)
        return s if s >= 0 else None

    # -- pages -----------------------------------------------------------------------
    def pages_needed(self, slot: int, n_new: int) -> List[int]:
        """New pages per group that appending ``n_new`` tokens would draw."""
        if self._lib.cj_books_pages_needed(self._h, slot, n_new, _ip(self._needs)) < 0:
            self._fail()
        return self._needs[:len(self.groups)].tolist()

    def pages_to_hold(self, slot: int, n_new: int, step_tokens: int = 0) -> List[int]:
        """Pages per group that the request in ``slot`` will hold at most, beyond those it holds
        now, while its next ``n_new`` tokens are fed in steps of at most ``step_tokens`` each
        (0: in one step).  A group that keeps every key needs them all; a windowed group gives
        pages back as it goes and never holds more than its window plus one step's tokens span,
        ``ceil((window + step_tokens) / page_tokens) + 1``.  What admission counts with."""
        raw = self.pages_needed(slot, n_new)
        if step_tokens <= 0:
            return raw
        out = []
        for g, need in zip(self.groups, raw):
            if g.spec.window > 0:
                most = -(-(g.spec.window + step_tokens) // self.page_tokens) + 1
                held = int(g.next_page[slot]) - int(g.first_live[slot])
                need = min(need, max(0, most - held))
            out.append(need)
        return out

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
        st = self._lib.cj_books_reserve(self._h, slot, n_new)
        if st < 0:
            self._fail()
        return bool(st)

    def reserve_step(self, slots: Sequence[int], n_new: Sequence[int]) -> Optional[List[int]]:
        """``reserve`` for every request of a step, all or nothing over the whole step.  Returns
        None when the pages were reserved, else (nothing changed) the new pages per group that
        the step wants."""
        s, n = _ints(slots), _ints(n_new)
        st = self._lib.cj_books_reserve_step(self._h, _ip(s), _ip(n), s.size, _ip(self._needs))
        if st < 0:
            self._fail()
        return None if st else self._needs[:len(self.groups)].tolist()

    # -- one token for each of several requests (a decode step), the books' hot path -------------
    def reserve_one_each(self, slots: Sequence[int]) -> Optional[np.ndarray]:
        """``reserve(slot, 1)`` for every slot, all or nothing over the whole list.  Returns the
        requests' lengths (before the new token) or None when the pages are not there."""
        s = _ints(slots)
        prior = np.empty(s.size, dtype=np.int64)
        st = self._lib.cj_books_reserve_one_each(self._h, _ip(s), s.size, prior.ctypes.data)
        if st < 0:
            self._fail()
        return prior if st else None

    def commit_one_each(self, slots: Sequence[int]) -> None:
        """``commit(slot, 1)`` for every slot."""
        s = _ints(slots)
        if self._lib.cj_books_commit_one_each(self._h, _ip(s), s.size) < 0:
            self._fail()

    def commit(self, slot: int, n_new: int) -> None:
        """The step that wrote ``n_new`` tokens is launched: advance the length and give
        back pages that have passed behind a window."""
        if self._lib.cj_books_commit(self._h, slot, n_new) < 0:
            self._fail()

    def release(self, slot: int) -> None:
        """Give back everything the request holds; the slot is free again."""
        if self._lib.cj_books_release(self._h, slot) < 0:
            self._fail()

    # -- what a step takes to the device -------------------------------------------------------
    def table_width(self, slots: Sequence[int]) -> int:
        """Columns that cover every page the given slots have ever been given."""
        s = _ints(slots)
        return self._lib.cj_books_table_width(self._h, _ip(s), s.size)

    def layout_step(self, slots: np.ndarray, n_tokens: np.ndarray, tokens: np.ndarray, n_want: np.ndarray,
                    wants: np.ndarray, width: int, out: np.ndarray, pad_requests: int = 0, pad_wanted: int = 0) -> int:
        """Lays a step's metadata into ``out`` (int32): tokens | positions | row -> request |
        request starts | prior lengths | slots | wanted rows | one slab ``[requests, width]`` of
        block-table rows per group.  ``pad_requests`` / ``pad_wanted`` lay the per-request arrays
        and the wanted rows out for at least that many (requests without rows, wanted row 0), so
        that steps of one number of rows share one shape.  All arguments are contiguous int32
        arrays; returns the number of values written."""
        n = self._lib.cj_books_layout_step(self._h, slots.size, _ip(slots), _ip(n_tokens), _ip(tokens), _ip(n_want),
                                           _ip(wants), width, pad_requests, pad_wanted, out.ctypes.data, out.size)
        if n < 0:
            self._fail()
        return int(n)

    def check(self) -> None:
        """Invariants: no page lost, held twice or freed twice; tables agree with owners."""
        if self._lib.cj_books_check(self._h) < 0:
            self._fail()
