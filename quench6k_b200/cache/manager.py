"""The cache manager: keys and values in fixed-size pages with a block table per request, one
pool of pages per group of layers with the same needs, and slots for fixed-size per-request state.

The reference keeps contiguous per-sequence buffers (crates/engine/src/flint.rs:436-478) and, for
its sliding layers, a ring of 8192 rows (:26-28, :855-859); its only paging is virtual-memory
growth in the other model's path (crates/cuda/kernels/vmm.cu:31-70).  Here:

* a group is "full" (a request holds pages for every position) or "sliding" with a window W (a
  request holds pages only for positions a later query can still see: after a step that leaves
  the request at length n, blocks that lie wholly below n - W + 1 go back to the pool);
* each group has its own pool and its own block table per request; a table lists the page of
  every logical block (position // page_size), -1 where none is held;
* pools are LIFO, so a page that was just given back is the next one handed out;
* a request also holds one state slot for mixers with fixed-size state of their own.

All of this is host bookkeeping; the device sees only the block tables the step function uploads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np


class OutOfPages(RuntimeError):
    """A pool cannot supply the pages a step needs.  Nothing was allocated."""


class OutOfSlots(RuntimeError):
    """Every request slot is taken."""


@dataclass(frozen=True)
class GroupSpec:
    kind: str                      # "full" | "sliding"
    window: Optional[int] = None   # sliding: number of visible keys including the query's own position

    def __post_init__(self):
        if self.kind not in ("full", "sliding"):
            raise ValueError(f"unknown cache group kind {self.kind!r}")
        if self.kind == "sliding" and not (isinstance(self.window, int) and self.window > 0):
            raise ValueError("a sliding group needs a positive window")


class PagePool:
    """Page ids 0..n-1 of one group; LIFO free list; every page is free or has exactly one owner."""

    def __init__(self, num_pages: int):
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))     # pop() hands out 0 first
        self._owner: List[Optional[Hashable]] = [None] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self, owner: Hashable) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        assert self._owner[page] is None, f"page {page} handed out twice"
        self._owner[page] = owner
        return page

    def give_back(self, page: int, owner: Hashable) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} outside the pool")
        if self._owner[page] is None:
            raise RuntimeError(f"page {page} freed twice")
        if self._owner[page] != owner:
            raise RuntimeError(f"page {page} belongs to {self._owner[page]!r}, not {owner!r}")
        self._owner[page] = None
        self._free.append(page)

    def owner_of(self, page: int) -> Optional[Hashable]:
        return self._owner[page]


class SlotPool:
    """Fixed-size per-request state lives in slot `s` of per-layer tensors [max_requests, ...]."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._used = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} request slots are in use")
        s = self._free.pop()
        self._used.add(s)
        return s

    def give_back(self, slot: int) -> None:
        if slot not in self._used:
            raise RuntimeError(f"slot {slot} freed twice")
        self._used.remove(slot)
        self._free.append(slot)


class BlockTable:
    """Pages of one request in one group by logical block: a growable int32 array.  Blocks
    [0, first_held) were given back (-1); blocks [first_held, len) hold a page each."""

    __slots__ = ("buf", "n", "first_held")

    def __init__(self):
        self.buf = np.full(16, -1, dtype=np.int32)
        self.n = 0
        self.first_held = 0

    def __len__(self) -> int:
        return self.n

    def append(self, page: int) -> None:
        if self.n == len(self.buf):
            grown = np.full(2 * len(self.buf), -1, dtype=np.int32)
            grown[:self.n] = self.buf[:self.n]
            self.buf = grown
        self.buf[self.n] = page
        self.n += 1

    def array(self) -> np.ndarray:
        return self.buf[:self.n]

    def tolist(self) -> List[int]:
        return self.buf[:self.n].tolist()


@dataclass
class _Request:
    slot: int
    length: int                         # tokens whose keys are in the cache
    tables: List[BlockTable]            # per group
    reserved: int = 0                   # tokens of the step in flight (pages held, not yet counted in length)


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, num_pages: Sequence[int], max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if len(num_pages) != len(groups):
            raise ValueError("one page count per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(n) for n in num_pages]
        self.slots = SlotPool(max_requests)
        self.requests: Dict[Hashable, _Request] = {}

    # ------------------------------------------------------------------ requests
    def add(self, rid: Hashable) -> int:
        """Register a request; returns its state slot."""
        if rid in self.requests:
            raise KeyError(f"request {rid!r} is already live")
        slot = self.slots.take()
        self.requests[rid] = _Request(slot, 0, [BlockTable() for _ in self.groups])
        return slot

    def remove(self, rid: Hashable) -> None:
        """The request ended (finished, aborted or preempted): every page and the slot go back."""
        req = self.requests.pop(rid)
        for g, table in enumerate(req.tables):
            for page in reversed(table.tolist()[table.first_held:]):
                self.pools[g].give_back(page, rid)
        self.slots.give_back(req.slot)

    def length(self, rid: Hashable) -> int:
        return self.requests[rid].length

    def slot(self, rid: Hashable) -> int:
        return self.requests[rid].slot

    def table(self, rid: Hashable, group: int) -> List[int]:
        """Pages by logical block as a list (-1 where none is held)."""
        return self.requests[rid].tables[group].tolist()

    def table_array(self, rid: Hashable, group: int) -> np.ndarray:
        """The same as an int32 array view (valid until the request's next reserve)."""
        return self.requests[rid].tables[group].array()

    def table_len(self, rid: Hashable, group: int) -> int:
        return len(self.requests[rid].tables[group])

    # ------------------------------------------------------------------ pages for a step
    def _first_needed_block(self, g: int, start: int) -> int:
        """First logical block a step whose first new position is `start` reads in group g."""
        spec = self.groups[g]
        if spec.kind == "full":
            return 0
        return max(0, start - spec.window + 1) // self.page_size

    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        """Pages each group's pool must supply so that the request can run n_new more tokens.
        A table holds a page for every block from the first one the next step reads up to its
        end (full groups never give pages back early; a sliding group gives back exactly the
        blocks below the next step's first block), so the need is the blocks past the table's end."""
        req = self.requests[rid]
        end = req.length + n_new
        last = (end - 1) // self.page_size if end > 0 else -1
        out = []
        for g in range(len(self.groups)):
            table = req.tables[g]
            assert self._first_needed_block(g, req.length) >= table.first_held, "a block the next step reads was given back"
            out.append(max(0, last + 1 - len(table)))
        return out

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        total = [0] * len(self.groups)
        for rid, n in wants:
            for g, c in enumerate(self.pages_needed(rid, n)):
                total[g] += c
        return all(total[g] <= self.pools[g].num_free for g in range(len(self.groups)))

    def reserve(self, rid: Hashable, n_new: int) -> None:
        """Hold pages for the next n_new positions of the request (all groups, or none: raises
        OutOfPages without changing anything)."""
        req = self.requests[rid]
        if req.reserved:
            raise RuntimeError(f"request {rid!r} already has a step in flight")
        need = self.pages_needed(rid, n_new)
        for g, c in enumerate(need):
            if c > self.pools[g].num_free:
                raise OutOfPages(f"group {g} ({self.groups[g].kind}) needs {c} pages for request {rid!r}, "
                                 f"{self.pools[g].num_free} are free")
        end = req.length + n_new
        last = (end - 1) // self.page_size if end > 0 else -1
        for g in range(len(self.groups)):
            table = req.tables[g]
            while len(table) <= last:
                table.append(self.pools[g].take(rid))
        req.reserved = n_new

    def commit(self, rid: Hashable) -> None:
        """The step in flight is done: its tokens count, and pages a window has passed go back."""
        req = self.requests[rid]
        req.length += req.reserved
        req.reserved = 0
        for g, spec in enumerate(self.groups):
            if spec.kind != "sliding":
                continue
            # the next query sits at position `length` and sees keys > length - window
            dead = max(0, req.length - spec.window + 1) // self.page_size     # blocks [0, dead) lie wholly below
            table = req.tables[g]
            for b in range(table.first_held, min(dead, len(table))):
                self.pools[g].give_back(int(table.buf[b]), rid)
                table.buf[b] = -1
            table.first_held = max(table.first_held, min(dead, len(table)))

    def cancel(self, rid: Hashable) -> None:
        """The step in flight did not run: pages taken for it stay with the request (they are
        reused by its next step or returned by remove)."""
        self.requests[rid].reserved = 0

    # ------------------------------------------------------------------ the step's description
    def pack_step(self, rids: Sequence[Hashable], tokens: Sequence[Sequence[int]], want: Sequence[Sequence[int]],
                  widths: Sequence[int], vocab_size: int, out: np.ndarray, feed_limit: int = 0, pad: int = 0,
                  pad_pages: Sequence[int] = (), pad_slot: int = 0) -> Tuple[int, int, int, int, int]:
        """Write the step's int32 block into `out`:
        [tokens T | positions T | request of token T | q_start R+1 | pos_start R | slot R | logit rows |
        one R x widths[g] block table per group].  Returns (ints written, T, wanted rows, longest
        context, longest entry).  pad > 0 appends that many filler entries (counted in R, T and the
        wanted rows): token 0 at position 0, its logits wanted, slot pad_slot and the single page
        pad_pages[g] in group g."""
        if pad < 0 or (pad and len(pad_pages) != len(widths)):
            raise ValueError("one filler page per cache group is needed")
        real = len(rids)
        R = real + pad
        q_lens = [len(t) for t in tokens]
        T, W = sum(q_lens) + pad, sum(len(w) for w in want) + pad
        total = 3 * T + (R + 1) + 2 * R + W + sum(R * w for w in widths)
        if total > out.size:
            raise ValueError(f"the step needs {total} ints, the block holds {out.size}")
        o = 0

        def take(n):
            nonlocal o
            v = out[o:o + n]
            o += n
            return v

        tok, pos, rot = take(T), take(T), take(T)
        qs, psv, sl, lr = take(R + 1), take(R), take(R), take(W)
        t = w = 0
        qs[0] = 0
        max_ctx = max_q = 0
        for r, rid in enumerate(rids):
            req = self.requests[rid]
            n = q_lens[r]
            arr = np.asarray(tokens[r], dtype=np.int64)
            if n and (arr.min() < -feed_limit or arr.max() >= vocab_size):      # -1 .. -feed_limit: tokens still on the device
                raise ValueError(f"request {rid!r}: token id outside 0..{vocab_size - 1}")
            tok[t:t + n] = arr
            pos[t:t + n] = np.arange(req.length, req.length + n)
            rot[t:t + n] = r
            for i in want[r]:
                if not 0 <= i < n:
                    raise ValueError(f"request {rid!r}: wanted place {i} outside its {n} tokens")
                lr[w] = t + i
                w += 1
            t += n
            qs[r + 1] = t
            psv[r] = req.length
            sl[r] = req.slot
            max_ctx, max_q = max(max_ctx, req.length + n), max(max_q, n)
        for r in range(real, R):
            tok[t], pos[t], rot[t], lr[w] = 0, 0, r, t
            t, w = t + 1, w + 1
            qs[r + 1], psv[r], sl[r] = t, 0, pad_slot
            max_ctx, max_q = max(max_ctx, 1), max(max_q, 1)
        for g, wd in enumerate(widths):
            tb = take(R * wd).reshape(R, wd)
            tb[:] = -1
            if pad:
                tb[real:, 0] = pad_pages[g]
            for r, rid in enumerate(rids):
                row = self.requests[rid].tables[g].array()
                if len(row) > wd:
                    raise ValueError(f"request {rid!r} holds {len(row)} blocks in group {g}, the table is {wd} wide")
                tb[r, :len(row)] = row
        return total, T, W, max_ctx, max_q

    # ------------------------------------------------------------------ invariants (tests)
    def check(self) -> None:
        for g, pool in enumerate(self.pools):
            held = {}
            for rid, req in self.requests.items():
                tab = req.tables[g]
                for b, page in enumerate(tab.tolist()):
                    assert (page < 0) == (b < tab.first_held), f"group {g}: request {rid!r} block {b} page {page} first_held {tab.first_held}"
                    if page < 0:
                        continue
                    assert page not in held, f"group {g}: page {page} held by {held[page]} and {(rid, b)}"
                    held[page] = (rid, b)
                    assert pool.owner_of(page) == rid, f"group {g}: page {page} owner {pool.owner_of(page)!r} != {rid!r}"
            free = list(pool._free)
            assert len(set(free)) == len(free), f"group {g}: a page is twice in the free list"
            assert not (set(free) & set(held)), f"group {g}: a page is both free and held"
            assert len(free) + len(held) == pool.num_pages, f"group {g}: {pool.num_pages - len(free) - len(held)} pages lost"
        slots = [r.slot for r in self.requests.values()]
        assert len(set(slots)) == len(slots), "a state slot is held twice"
        assert len(slots) + self.slots.num_free == self.slots.num_slots, "a state slot is lost"
