"""Continuous batching above the step function.

Each call to `schedule()` builds one step under a token budget:

1. every running request whose prompt is in the cache decodes one token;
2. what is left of the budget goes to prompt portions, first of running requests that are still
   prefilling (in admission order), then of waiting requests, admitted first-come first-served
   while a slot, budget and pages for the portion are there.  A portion may be cut anywhere; if the
   pools cannot hold all of it, it shrinks to what they can hold, down to nothing (the request waits).

When pages run out for the decode tokens, the most recently admitted running request is preempted:
its pages and slot go back, and it returns to the front of the waiting queue to be recomputed from
its prompt and the tokens it has produced.  A request running alone that cannot get a page ends
with reason "length" (the cache is its context).  A prompt that could never fit is refused when
it is added.

The reference serves Flint one request at a time (crates/cli/src/serve.rs:981-1168) and, for its
other model, admits a request only if its memory plan fits and fails requests when memory is held
by running ones (crates/engine/src/session.rs:824-904); finish reasons are its Stop, Length and
Cancelled (crates/engine/src/session.rs:162-169).  This scheduler is host logic only and runs
against the cache manager without a GPU.

`Scheduler` is the C++ one (csrc/host/host.cpp, wrapped by NativeScheduler below) when the cache
manager is the C++ one, else PyScheduler, its Python twin with the same rules; the tests run both.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, Hashable, List, Optional, Sequence

import ctypes

import numpy as np

from ..cache import NativeCacheManager
from ..cache.native import host_lib, i32, ptr32, ptr64, raise_for
from ..sampling.params import SamplingParams
from ..sampling.sampler import SplitMix64
from .batch import StepEntry

FINISH_STOP, FINISH_LENGTH, FINISH_CANCELLED = "stop", "length", "cancelled"


@dataclass
class Request:
    rid: Hashable
    prompt: List[int]
    params: SamplingParams
    output: List[int] = field(default_factory=list)
    finish_reason: Optional[str] = None
    num_computed: int = 0                 # tokens of prompt + output whose keys are in the cache
    preemptions: int = 0
    rng: Optional[SplitMix64] = None

    @property
    def tokens(self) -> List[int]:
        return self.prompt + self.output

    @property
    def num_tokens(self) -> int:
        return len(self.prompt) + len(self.output)

    def token_slice(self, start: int, count: int) -> List[int]:
        """tokens[start:start+count] without building the whole list."""
        n = len(self.prompt)
        if start >= n:
            return self.output[start - n:start - n + count]
        if start + count <= n:
            return self.prompt[start:start + count]
        return self.prompt[start:] + self.output[:start + count - n]

    @property
    def finished(self) -> bool:
        return self.finish_reason is not None


@dataclass
class ScheduledEntry:
    request: Request
    start: int                            # index into request.tokens of the first token run
    count: int
    samples: bool                         # the last token of this entry yields the request's next token


@dataclass
class ScheduledStep:
    entries: List[ScheduledEntry]
    preempted: List[Request] = field(default_factory=list)
    finished: List[Request] = field(default_factory=list)      # ended while scheduling (cache exhausted)

    def step_entries(self) -> List[StepEntry]:
        out = []
        for e in self.entries:
            toks = e.request.token_slice(e.start, e.count)
            out.append(StepEntry(e.request.rid, toks, [e.count - 1] if e.samples else []))
        return out

    @property
    def num_tokens(self) -> int:
        return sum(e.count for e in self.entries)


def capacity_tokens(manager) -> int:
    """Most tokens one request can ever hold: the smallest pool of a group that keeps every key
    bounds it.  A sliding group holds a window's worth of pages whatever the length, so its
    (possibly much smaller) pool bounds nothing."""
    full = [p.num_pages for p, g in zip(manager.pools, manager.groups) if g.kind != "sliding"]
    return min(full) * manager.page_size if full else 1 << 60


def check_pools(manager) -> None:
    """A sliding group must hold its window and one more token wherever they lie on the pages,
    or no request could ever advance."""
    for i, (p, g) in enumerate(zip(manager.pools, manager.groups)):
        if g.kind == "sliding":
            need = -(-g.window // manager.page_size) + 1
            if p.num_pages < need:
                raise ValueError(f"cache group {i}: {p.num_pages} pages cannot hold a window of {g.window} keys and the next token "
                                 f"({need} pages of {manager.page_size})")


class PyScheduler:
    """`on_admit(slot)` is called for every request admitted by `schedule()`, before it returns, so
    that the caller can clear the per-request state in that slot."""

    def __init__(self, manager, max_batch_tokens: int = 2048, max_running: Optional[int] = None,
                 on_admit: Optional[Callable[[int], None]] = None):
        if max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be at least 1")
        self.manager = manager
        check_pools(manager)
        self.max_batch_tokens = max_batch_tokens
        self.max_running = max_running if max_running is not None else manager.slots.num_slots
        self._admit = manager.add
        self._release = manager.remove
        self._on_admit = on_admit
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []          # admission order
        self.by_id: Dict[Hashable, Request] = {}

    # ------------------------------------------------------------------ queue
    def capacity_tokens(self) -> int:
        return capacity_tokens(self.manager)

    def add(self, req: Request) -> None:
        if req.rid in self.by_id:
            raise KeyError(f"request {req.rid!r} already exists")
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        req.params.validate()
        if len(req.prompt) + 1 > self.capacity_tokens():
            raise ValueError(f"prompt of {len(req.prompt)} tokens exceeds the cache capacity of {self.capacity_tokens()} tokens")
        self.by_id[req.rid] = req
        self.waiting.append(req)

    def adopt(self, req: Request) -> None:
        """Take a request that is live in the cache manager with its whole prompt counted as cached
        and its first output token given: it decodes from the next step on."""
        if req.rid in self.by_id:
            raise KeyError(f"request {req.rid!r} already exists")
        req.params.validate()
        req.num_computed = len(req.prompt)
        self.by_id[req.rid] = req
        self.running.append(req)

    def abort(self, rid: Hashable) -> Optional[Request]:
        req = self.by_id.get(rid)
        if req is None or req.finished:
            return None
        self._finish(req, FINISH_CANCELLED)
        return req

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def set_output_token(self, req: Request, index: int, token: int) -> None:
        """A token that was entered as a placeholder (the step that samples it was still running) gets its value."""
        req.output[index] = int(token)

    def stop_at(self, req: Request, n_keep: int) -> None:
        """The request turns out to have ended with its n_keep-th output token (a stop token that
        was still a placeholder when later steps were planned): what came after is dropped."""
        del req.output[n_keep:]
        if req.rid in self.by_id and not req.finished:
            self._finish(req, FINISH_STOP)
        req.finish_reason = FINISH_STOP

    def _finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        if req in self.running:
            self.running.remove(req)
            self._release(req.rid)
        elif req in self.waiting:
            self.waiting.remove(req)
        self.by_id.pop(req.rid, None)

    def _preempt(self, req: Request) -> None:
        self.running.remove(req)
        self._release(req.rid)
        req.num_computed = 0
        req.preemptions += 1
        self.waiting.appendleft(req)

    # ------------------------------------------------------------------ one step
    def _fit(self, chosen: List, rid: Hashable, want: int) -> int:
        """Largest n <= want such that the pools hold `chosen` plus n tokens of rid."""
        if want <= 0:
            return 0
        if self.manager.can_reserve(chosen + [(rid, want)]):
            return want
        lo, hi = 0, want                   # can_reserve is monotone in n
        while lo < hi:
            mid = (lo + hi + 1) // 2
            if self.manager.can_reserve(chosen + [(rid, mid)]):
                lo = mid
            else:
                hi = mid - 1
        return lo

    def schedule(self) -> ScheduledStep:
        step = ScheduledStep([])
        budget = self.max_batch_tokens
        # 1. decode tokens; preempt from the back until they fit
        while True:
            decoding = [r for r in self.running if r.num_computed == r.num_tokens - 1 and r.output]
            decoding = decoding[:budget]
            wants = [(r.rid, 1) for r in decoding]
            if self.manager.can_reserve(wants):
                break
            if len(self.running) == 1:
                lone = self.running[0]
                self._finish(lone, FINISH_LENGTH)
                step.finished.append(lone)
                continue
            victim = self.running[-1]
            self._preempt(victim)
            step.preempted.append(victim)
        chosen = list(wants)
        for r in decoding:
            step.entries.append(ScheduledEntry(r, r.num_computed, 1, True))
        budget -= len(decoding)
        in_step = {r.rid for r in decoding}
        # 2. prompt portions of running requests still prefilling
        for r in self.running:
            if budget <= 0:
                break
            if r.rid in in_step:
                continue
            left = r.num_tokens - r.num_computed
            n = self._fit(chosen, r.rid, min(left, budget))
            if n <= 0:
                continue
            step.entries.append(ScheduledEntry(r, r.num_computed, n, n == left))
            chosen.append((r.rid, n))
            in_step.add(r.rid)
            budget -= n
        # 3. admit waiting requests, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_running and self.manager.slots.num_free > 0:
            r = self.waiting[0]
            slot = self._admit(r.rid)
            left = r.num_tokens
            n = self._fit(chosen, r.rid, min(left, budget))
            if n <= 0:
                self._release(r.rid)
                break                      # the head of the queue waits; nobody overtakes it
            self.waiting.popleft()
            self.running.append(r)
            if self._on_admit is not None:
                self._on_admit(slot)
            step.entries.append(ScheduledEntry(r, 0, n, n == left))
            chosen.append((r.rid, n))
            budget -= n
        if not step.entries and not step.finished and self.running:
            # every running request is mid-prefill and no page is free: make room from the back
            if len(self.running) > 1:
                victim = self.running[-1]
                self._preempt(victim)
                step.preempted.append(victim)
                more = self.schedule()
                more.preempted = step.preempted + more.preempted
                return more
            lone = self.running[0]
            self._finish(lone, FINISH_LENGTH)
            step.finished.append(lone)
        return step

    def update(self, step: ScheduledStep, sampled: Sequence[int]) -> List[Request]:
        """Account for a finished step.  `sampled` holds one token for every entry with
        samples=True, in order.  Returns the requests that ended."""
        done: List[Request] = []
        it = iter(sampled)
        for e in step.entries:
            r = e.request
            if r.finished:                 # aborted while the step ran
                if e.samples:
                    next(it)
                continue
            r.num_computed += e.count
            if not e.samples:
                continue
            tok = int(next(it))
            r.output.append(tok)
            if tok in r.params.stop_tokens:
                self._finish(r, FINISH_STOP)
            elif len(r.output) >= r.params.max_tokens:
                self._finish(r, FINISH_LENGTH)
            elif r.num_tokens + 1 > self.capacity_tokens():
                self._finish(r, FINISH_LENGTH)
            if r.finished:
                done.append(r)
        return done


_REASONS = {1: FINISH_STOP, 2: FINISH_LENGTH, 3: FINISH_CANCELLED}


class NativeScheduler:
    """The C++ scheduler behind PyScheduler's interface.  Queues, token lists and decisions live in
    C++; the `Request` objects here mirror what the caller reads (output, counts, finish reason)
    and carry what only Python needs (sampling parameters, the random stream)."""

    def __init__(self, manager: NativeCacheManager, max_batch_tokens: int = 2048, max_running: Optional[int] = None,
                 on_admit: Optional[Callable[[int], None]] = None):
        if max_batch_tokens < 1:
            raise ValueError("max_batch_tokens must be at least 1")
        self.manager = manager
        self.max_batch_tokens = max_batch_tokens
        self.max_running = max_running if max_running is not None else manager.slots.num_slots
        self._on_admit = on_admit
        self._lib = host_lib()
        self._h = self._lib.q6k_sched_create(manager._h, max_batch_tokens, self.max_running)
        if not self._h:
            raise ValueError(self._lib.q6k_host_last_error().decode())
        self.by_id: Dict[Hashable, Request] = {}

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.q6k_sched_destroy(h)

    # ------------------------------------------------------------------ queue
    def capacity_tokens(self) -> int:
        return capacity_tokens(self.manager)

    def _queue(self, which: int) -> List[Request]:
        cap = len(self.by_id) + 1
        ids, n = np.zeros(cap, dtype=np.int64), ctypes.c_int32()
        raise_for(self._lib.q6k_sched_queue(self._h, which, ptr64(ids), cap, ctypes.byref(n)))
        return [self.by_id[self.manager.rid_of(int(i))] for i in ids[:n.value]]

    @property
    def waiting(self) -> List[Request]:
        return self._queue(0)

    @property
    def running(self) -> List[Request]:
        return self._queue(1)

    def _drop(self, req: Request) -> None:
        self.by_id.pop(req.rid, None)
        self.manager.forget(req.rid)

    def _register(self, req: Request, call) -> None:
        if req.rid in self.by_id:
            raise KeyError(f"request {req.rid!r} already exists")
        req.params.validate()
        known = req.rid in self.manager._nid
        nid = self.manager.intern(req.rid)
        rc = call(nid, i32(req.prompt), i32(req.params.stop_tokens))
        if rc:
            if not known:
                self.manager.forget(req.rid)
            raise_for(rc)
        self.manager._held.add(req.rid)
        self.by_id[req.rid] = req

    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("a request needs at least one prompt token")
        self._register(req, lambda nid, prompt, stops: self._lib.q6k_sched_add(
            self._h, nid, ptr32(prompt), len(prompt), req.params.max_tokens, ptr32(stops), len(stops)))

    def adopt(self, req: Request) -> None:
        """Take a request that is live in the cache manager with its whole prompt counted as cached
        and its first output token given: it decodes from the next step on."""
        if len(req.output) != 1:
            raise ValueError("an adopted request brings exactly its first output token")
        self._register(req, lambda nid, prompt, stops: self._lib.q6k_sched_adopt(
            self._h, nid, ptr32(prompt), len(prompt), req.output[0], req.params.max_tokens, ptr32(stops), len(stops)))
        req.num_computed = len(req.prompt)

    def abort(self, rid: Hashable) -> Optional[Request]:
        req = self.by_id.get(rid)
        if req is None or req.finished:
            return None
        live = ctypes.c_int32()
        raise_for(self._lib.q6k_sched_abort(self._h, self.manager._nid[rid], ctypes.byref(live)))
        req.finish_reason = FINISH_CANCELLED
        self._drop(req)
        return req

    def has_work(self) -> bool:
        w, r = ctypes.c_int32(), ctypes.c_int32()
        raise_for(self._lib.q6k_sched_counts(self._h, ctypes.byref(w), ctypes.byref(r)))
        return bool(w.value or r.value)

    def set_output_token(self, req: Request, index: int, token: int) -> None:
        """A token that was entered as a placeholder (the step that samples it was still running) gets its value."""
        req.output[index] = int(token)
        if req.rid in self.by_id:
            raise_for(self._lib.q6k_sched_set_output_token(self._h, self.manager._nid[req.rid], index, int(token)))

    def stop_at(self, req: Request, n_keep: int) -> None:
        """The request turns out to have ended with its n_keep-th output token (a stop token that
        was still a placeholder when later steps were planned): what came after is dropped."""
        del req.output[n_keep:]
        if req.rid in self.by_id:
            raise_for(self._lib.q6k_sched_stop(self._h, self.manager._nid[req.rid], n_keep))
            self._drop(req)
        req.finish_reason = FINISH_STOP

    # ------------------------------------------------------------------ one step
    def schedule(self) -> ScheduledStep:
        cap = len(self.by_id) + 1
        ids, starts = np.zeros(cap, dtype=np.int64), np.zeros(cap, dtype=np.int64)
        counts, samples = np.zeros(cap, dtype=np.int32), np.zeros(cap, dtype=np.int32)
        pre, fin, adm = (np.zeros(cap, dtype=np.int64) for _ in range(3))
        adm_slots = np.zeros(cap, dtype=np.int32)
        n, n_pre, n_fin, n_adm = (ctypes.c_int32() for _ in range(4))
        raise_for(self._lib.q6k_sched_schedule(self._h, cap, ptr64(ids), ptr64(starts), ptr32(counts), ptr32(samples), ctypes.byref(n),
                                               ptr64(pre), ctypes.byref(n_pre), ptr64(fin), ctypes.byref(n_fin),
                                               ptr64(adm), ptr32(adm_slots), ctypes.byref(n_adm)))
        rid_of = self.manager.rid_of
        step = ScheduledStep([])
        for i in pre[:n_pre.value]:
            r = self.by_id[rid_of(int(i))]
            r.num_computed = 0
            r.preemptions += 1
            step.preempted.append(r)
        for i in fin[:n_fin.value]:
            r = self.by_id[rid_of(int(i))]
            r.finish_reason = FINISH_LENGTH
            step.finished.append(r)
            self._drop(r)
        if self._on_admit is not None:
            for slot in adm_slots[:n_adm.value]:
                self._on_admit(int(slot))
        for k in range(n.value):
            r = self.by_id[rid_of(int(ids[k]))]
            step.entries.append(ScheduledEntry(r, int(starts[k]), int(counts[k]), bool(samples[k])))
        return step

    def update(self, step: ScheduledStep, sampled: Sequence[int]) -> List[Request]:
        """Account for a finished step.  `sampled` holds one token for every entry with
        samples=True, in order.  Returns the requests that ended."""
        toks = i32([int(t) for t in sampled])
        cap = len(step.entries) + 1
        done_ids, reasons, n_done = np.zeros(cap, dtype=np.int64), np.zeros(cap, dtype=np.int32), ctypes.c_int32()
        raise_for(self._lib.q6k_sched_update(self._h, ptr32(toks), len(toks), cap, ptr64(done_ids), ptr32(reasons), ctypes.byref(n_done)))
        it = iter(toks.tolist())
        for e in step.entries:
            r = e.request
            if r.finished:                 # aborted while the step ran
                if e.samples:
                    next(it)
                continue
            r.num_computed += e.count
            if e.samples:
                r.output.append(next(it))
        done: List[Request] = []
        for i, why in zip(done_ids[:n_done.value], reasons[:n_done.value]):
            r = self.by_id[self.manager.rid_of(int(i))]
            r.finish_reason = _REASONS[int(why)]
            done.append(r)
            self._drop(r)
        return done


def Scheduler(manager, max_batch_tokens: int = 2048, max_running: Optional[int] = None,
              on_admit: Optional[Callable[[int], None]] = None):
    """The scheduler that matches the cache manager: C++ for the C++ manager, Python for the Python one."""
    cls = NativeScheduler if isinstance(manager, NativeCacheManager) else PyScheduler
    return cls(manager, max_batch_tokens, max_running, on_admit)
