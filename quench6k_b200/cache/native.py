"""The cache manager of the C++ host library (csrc/host/host.cpp) behind the interface of the
Python one in manager.py: same rules, same errors, and a packed step description written by C++.

Request ids of any hashable kind are mapped to 64-bit numbers that are never used twice.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Hashable, Iterator, List, Sequence, Tuple

import numpy as np

from .manager import GroupSpec, OutOfPages, OutOfSlots

_i32p = ctypes.POINTER(ctypes.c_int32)
_i64p = ctypes.POINTER(ctypes.c_int64)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_lib = None


def host_lib():
    """The loaded library with its argument types declared."""
    global _lib
    if _lib is not None:
        return _lib
    from ..ops.build import host_library
    lib = host_library()
    vp, i, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    sig = {
        "q6k_host_last_error": (ctypes.c_char_p, []),
        "q6k_host_abi_version": (i, []),
        "q6k_cm_create": (vp, [i, _i32p, _i32p, i, _i32p, i]),
        "q6k_cm_destroy": (None, [vp]),
        "q6k_cm_add": (i, [vp, i64, _i32p]),
        "q6k_cm_remove": (i, [vp, i64]),
        "q6k_cm_info": (i, [vp, i64, _i64p, _i32p]),
        "q6k_cm_pages_needed": (i, [vp, i64, i, _i32p]),
        "q6k_cm_can_reserve": (i, [vp, _i64p, _i32p, i, _i32p]),
        "q6k_cm_reserve": (i, [vp, i64, i]),
        "q6k_cm_commit": (i, [vp, i64]),
        "q6k_cm_cancel": (i, [vp, i64]),
        "q6k_cm_check": (i, [vp]),
        "q6k_cm_num_free": (i, [vp, i]),
        "q6k_cm_slots_free": (i, [vp]),
        "q6k_cm_num_live": (i, [vp]),
        "q6k_cm_table": (i, [vp, i64, i, ctypes.POINTER(_i32p), _i32p]),
        "q6k_cm_fill_step": (i, [vp, i, _i64p, _i32p, _i32p, _i32p, _i32p, _i32p, i, i, i, _i32p, i, _i32p, i64, _i64p]),
        "q6k_sched_create": (vp, [vp, i, i]),
        "q6k_sched_destroy": (None, [vp]),
        "q6k_sched_add": (i, [vp, i64, _i32p, i, i, _i32p, i]),
        "q6k_sched_adopt": (i, [vp, i64, _i32p, i, ctypes.c_int32, i, _i32p, i]),
        "q6k_sched_abort": (i, [vp, i64, _i32p]),
        "q6k_sched_counts": (i, [vp, _i32p, _i32p]),
        "q6k_sched_queue": (i, [vp, i, _i64p, i, _i32p]),
        "q6k_sched_request": (i, [vp, i64, _i64p, _i32p, _i32p, _i32p]),
        "q6k_sched_schedule": (i, [vp, i, _i64p, _i64p, _i32p, _i32p, _i32p, _i64p, _i32p, _i64p, _i32p, _i64p, _i32p, _i32p]),
        "q6k_sched_tokens": (i, [vp, i64, i64, i, _i32p]),
        "q6k_sched_update": (i, [vp, _i32p, i, i, _i64p, _i32p, _i32p]),
        "q6k_sched_set_output_token": (i, [vp, i64, i, ctypes.c_int32]),
        "q6k_sched_stop": (i, [vp, i64, i]),
        "q6k_st_open": (i, [ctypes.c_char_p, ctypes.POINTER(vp)]),
        "q6k_st_close": (None, [vp]),
        "q6k_st_count": (i, [vp]),
        "q6k_st_entry": (i, [vp, i, ctypes.c_char_p, i, ctypes.c_char_p, _i64p, _i32p, _i64p, _i64p]),
        "q6k_st_read": (i, [vp, i, vp, i64]),
        "q6k_st_read_range": (i, [vp, i, i64, vp, i64]),
        "q6k_fill_normal_host": (i, [vp, i, i64, i64, ctypes.c_uint64, ctypes.c_float, ctypes.c_float, i]),
        "q6k_sample_rows": (i, [i, i, _i32p, _f32p, _i32p, _f32p, _i32p, _f32p, _f32p, _f32p, _f32p, _i32p, _i64p, _f64p, _i32p]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if lib.q6k_host_abi_version() != 5:
        raise RuntimeError("the host library does not match this package")
    _lib = lib
    return lib


def raise_for(rc: int) -> None:
    """Turn an error kind of the host library into the exception the Python twin raises."""
    if rc == 0:
        return
    msg = host_lib().q6k_host_last_error().decode()
    if rc == 2:
        raise OutOfPages(msg)
    if rc == 3:
        raise OutOfSlots(msg)
    if rc == 4:
        raise KeyError(msg)
    if rc == 5:
        raise ValueError(msg)
    raise RuntimeError(msg)


def i32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.int32)


def ptr32(a: np.ndarray):
    return a.ctypes.data_as(_i32p)


def ptr64(a: np.ndarray):
    return a.ctypes.data_as(_i64p)


class _PoolView:
    def __init__(self, mgr: "NativeCacheManager", group: int, num_pages: int):
        self._mgr, self._group, self.num_pages = mgr, group, num_pages

    @property
    def num_free(self) -> int:
        return host_lib().q6k_cm_num_free(self._mgr._h, self._group)


class _SlotView:
    def __init__(self, mgr: "NativeCacheManager", num_slots: int):
        self._mgr, self.num_slots = mgr, num_slots

    @property
    def num_free(self) -> int:
        return host_lib().q6k_cm_slots_free(self._mgr._h)


class _LiveView:
    """`rid in manager.requests`, `len(...)`, truth value and iteration over the live requests."""

    def __init__(self, mgr: "NativeCacheManager"):
        self._mgr = mgr

    def __contains__(self, rid: Hashable) -> bool:
        return self._mgr._live(rid)

    def __len__(self) -> int:
        return host_lib().q6k_cm_num_live(self._mgr._h)

    def __iter__(self) -> Iterator[Hashable]:
        return iter([rid for rid in list(self._mgr._nid) if self._mgr._live(rid)])


class NativeCacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, num_pages: Sequence[int], max_requests: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        if len(num_pages) != len(groups):
            raise ValueError("one page count per group is needed")
        self.groups = list(groups)
        self.page_size = page_size
        lib = host_lib()
        sliding = i32([g.kind == "sliding" for g in groups])
        windows = i32([g.window or 0 for g in groups])
        pages = i32(list(num_pages))
        self._h = lib.q6k_cm_create(len(groups), ptr32(sliding), ptr32(windows), page_size, ptr32(pages), max_requests)
        if not self._h:
            raise ValueError(lib.q6k_host_last_error().decode())
        self.pools = [_PoolView(self, g, int(n)) for g, n in enumerate(num_pages)]
        self.slots = _SlotView(self, max_requests)
        self.requests = _LiveView(self)
        self._nid: Dict[Hashable, int] = {}
        self._rid: Dict[int, Hashable] = {}
        self._held = set()                   # ids a scheduler keeps although the request holds no cache now
        self._next = 1

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.q6k_cm_destroy(h)

    # ------------------------------------------------------------------ ids
    def intern(self, rid: Hashable) -> int:
        nid = self._nid.get(rid)
        if nid is None:
            nid = self._next
            self._next += 1
            self._nid[rid] = nid
            self._rid[nid] = rid
        return nid

    def forget(self, rid: Hashable) -> None:
        nid = self._nid.pop(rid, None)
        if nid is not None:
            self._rid.pop(nid, None)
        self._held.discard(rid)

    def rid_of(self, nid: int) -> Hashable:
        return self._rid[nid]

    def _known(self, rid: Hashable) -> int:
        nid = self._nid.get(rid)
        if nid is None:
            raise KeyError(rid)
        return nid

    def _live(self, rid: Hashable) -> bool:
        nid = self._nid.get(rid)
        if nid is None:
            return False
        length, slot = ctypes.c_int64(), ctypes.c_int32()
        return host_lib().q6k_cm_info(self._h, nid, ctypes.byref(length), ctypes.byref(slot)) == 0

    # ------------------------------------------------------------------ requests
    def add(self, rid: Hashable) -> int:
        if self._live(rid):
            raise KeyError(f"request {rid!r} is already live")
        fresh = rid not in self._nid
        slot = ctypes.c_int32()
        rc = host_lib().q6k_cm_add(self._h, self.intern(rid), ctypes.byref(slot))
        if rc and fresh:
            self.forget(rid)
        raise_for(rc)
        return slot.value

    def remove(self, rid: Hashable) -> None:
        raise_for(host_lib().q6k_cm_remove(self._h, self._known(rid)))
        if rid not in self._held:
            self.forget(rid)

    def _info(self, rid: Hashable) -> Tuple[int, int]:
        length, slot = ctypes.c_int64(), ctypes.c_int32()
        raise_for(host_lib().q6k_cm_info(self._h, self._known(rid), ctypes.byref(length), ctypes.byref(slot)))
        return length.value, slot.value

    def length(self, rid: Hashable) -> int:
        return self._info(rid)[0]

    def slot(self, rid: Hashable) -> int:
        return self._info(rid)[1]

    def table_array(self, rid: Hashable, group: int) -> np.ndarray:
        """A copy of the request's pages by logical block (-1 where none is held)."""
        p, n = _i32p(), ctypes.c_int32()
        raise_for(host_lib().q6k_cm_table(self._h, self._known(rid), group, ctypes.byref(p), ctypes.byref(n)))
        return np.ctypeslib.as_array(p, shape=(n.value,)).copy() if n.value else np.zeros(0, dtype=np.int32)

    def table(self, rid: Hashable, group: int) -> List[int]:
        return self.table_array(rid, group).tolist()

    def table_len(self, rid: Hashable, group: int) -> int:
        p, n = _i32p(), ctypes.c_int32()
        raise_for(host_lib().q6k_cm_table(self._h, self._known(rid), group, ctypes.byref(p), ctypes.byref(n)))
        return n.value

    # ------------------------------------------------------------------ pages for a step
    def pages_needed(self, rid: Hashable, n_new: int) -> List[int]:
        out = np.zeros(max(1, len(self.groups)), dtype=np.int32)
        raise_for(host_lib().q6k_cm_pages_needed(self._h, self._known(rid), n_new, ptr32(out)))
        return out[:len(self.groups)].tolist()

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]]) -> bool:
        ids = np.array([self._known(rid) for rid, _ in wants], dtype=np.int64)
        ns = i32([n for _, n in wants])
        yes = ctypes.c_int32()
        raise_for(host_lib().q6k_cm_can_reserve(self._h, ptr64(ids), ptr32(ns), len(wants), ctypes.byref(yes)))
        return bool(yes.value)

    def reserve(self, rid: Hashable, n_new: int) -> None:
        raise_for(host_lib().q6k_cm_reserve(self._h, self._known(rid), n_new))

    def commit(self, rid: Hashable) -> None:
        raise_for(host_lib().q6k_cm_commit(self._h, self._known(rid)))

    def cancel(self, rid: Hashable) -> None:
        raise_for(host_lib().q6k_cm_cancel(self._h, self._known(rid)))

    def check(self) -> None:
        rc = host_lib().q6k_cm_check(self._h)
        if rc:
            raise AssertionError(host_lib().q6k_host_last_error().decode())

    # ------------------------------------------------------------------ the step's description
    def pack_step(self, rids: Sequence[Hashable], tokens: Sequence[Sequence[int]], want: Sequence[Sequence[int]],
                  widths: Sequence[int], vocab_size: int, out: np.ndarray, feed_limit: int = 0, pad: int = 0,
                  pad_pages: Sequence[int] = (), pad_slot: int = 0) -> Tuple[int, int, int, int, int]:
        """Write the step's int32 block into `out`:
        [tokens T | positions T | request of token T | q_start R+1 | pos_start R | slot R | logit rows |
        one R x widths[g] block table per group].  Returns (ints written, T, wanted rows, longest
        context, longest entry).  feed_limit > 0 admits token ids -1 .. -feed_limit, which stand for
        tokens the step before has sampled and which are resolved on the device.  pad > 0 appends
        that many filler entries (counted in R, T and the wanted rows): token 0 at position 0, its
        logits wanted, slot pad_slot and the single page pad_pages[g] in group g."""
        R = len(rids)
        ids = np.array([self._known(r) for r in rids], dtype=np.int64)
        q_lens = i32([len(t) for t in tokens])
        flat = np.concatenate([np.asarray(t, dtype=np.int64) for t in tokens]) if R else np.zeros(0, dtype=np.int64)
        if flat.size and (flat.min() < -feed_limit or flat.max() >= vocab_size):
            bad = next(r for r, t in zip(rids, tokens) if len(t) and (min(t) < -feed_limit or max(t) >= vocab_size))
            raise ValueError(f"request {bad!r}: token id outside 0..{vocab_size - 1}")
        flat = i32(flat)
        wc = i32([len(w) for w in want])
        wflat = i32([i for w in want for i in w])
        wd = i32(list(widths) or [0])
        meta = np.zeros(5, dtype=np.int64)
        pp = i32(list(pad_pages) or [0])
        if pad and len(pad_pages) != len(widths):
            raise ValueError("one filler page per cache group is needed")
        rc = host_lib().q6k_cm_fill_step(self._h, R, ptr64(ids), ptr32(q_lens), ptr32(flat), ptr32(wflat), ptr32(wc), ptr32(wd),
                                         vocab_size, feed_limit, pad, ptr32(pp), pad_slot, ptr32(out), out.size, ptr64(meta))
        if rc == 5 and "wanted place" in host_lib().q6k_host_last_error().decode():
            for r, t, w in zip(rids, tokens, want):
                for i in w:
                    if not 0 <= i < len(t):
                        raise ValueError(f"request {r!r}: wanted place {i} outside its {len(t)} tokens")
        raise_for(rc)
        return tuple(int(v) for v in meta)
