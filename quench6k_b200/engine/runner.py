"""The model on the device, its cache and the one step function.

`step(entries)` takes any mix of (request, next tokens): portions of prompts beside single decoded
tokens, cut anywhere.  It reserves pages, uploads the batch description in one copy, runs only the
given tokens through the model from the cache that earlier steps left, commits the pages and
returns the FP32 logits at the wanted places (reference: one sequence per call,
crates/engine/src/flint.rs:699-771; batches of one-token segments, crates/engine/src/forward.rs:1166-1260).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from .. import ops
from ..cache import CacheManager, GroupSpec, OutOfPages
from ..config.registry import load_config
from ..models.decoder import DecoderModel
from ..parts.base import LayerCache, Runtime
from ..weights import load_folder, random_getter
from .batch import StepContext, StepEntry

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def parse_dtype(d) -> torch.dtype:
    if d not in _DTYPES:
        raise ValueError(f"dtype {d!r} is neither bfloat16 nor float32")
    return _DTYPES[d]


class ModelRunner:
    def __init__(self, model: DecoderModel, rt: Runtime, page_size: int, num_pages: Union[int, Sequence[int]],
                 max_requests: int, cuda_graphs: bool = True):
        if rt.device.type != "cuda":
            raise RuntimeError("the engine runs on a CUDA device only; there is no CPU path")
        self.model, self.rt = model, rt
        self.page_size = page_size
        self.vocab_size = model.spec.vocab_size
        # cache groups: executed positions whose mixers ask for the same kind of cache share one
        reqs = model.cache_requests()
        keys, self.group_of = [], []
        for r in reqs:
            if r is None:
                self.group_of.append(None)
                continue
            if r.key() not in keys:
                keys.append(r.key())
            self.group_of.append(keys.index(r.key()))
        self.group_specs = [GroupSpec(k[0], k[1]) for k in keys]
        n_groups = len(keys)
        pages = [num_pages] * n_groups if isinstance(num_pages, int) else list(num_pages)
        if len(pages) != n_groups:
            raise ValueError(f"{len(pages)} page counts for {n_groups} cache groups")
        self.manager = CacheManager(self.group_specs, page_size, pages, max_requests)
        self.caches: List[Optional[LayerCache]] = []
        for p, r in enumerate(reqs):
            src = model.kv_source[p]
            if src is not None:
                own = self.caches[src]
                if own is None:
                    raise ValueError(f"position {p} borrows the cache of position {src}, which has none")
                self.caches.append(LayerCache(own.group, own.k, own.v, page_size, write=False))
            elif r is None:
                self.caches.append(None)
            else:
                g = self.group_of[p]
                # head-major: a head's pages are contiguous; one page beyond the manager's pool takes what filler entries write
                lead, dt = (r.kv_heads, pages[g] + 1, page_size), r.dtype or rt.dtype
                self.caches.append(LayerCache(g, torch.zeros((*lead, r.head_dim), dtype=dt, device=rt.device),
                                              torch.zeros((*lead, r.v_dim or r.head_dim), dtype=dt, device=rt.device), page_size))

        def state_for(s):
            """One tensor [slots + 1, *shape] per declared state (the extra slot is the filler entries')."""
            if s is None:
                return None
            if isinstance(s, dict):
                return {name: torch.zeros((max_requests + 1, *shape), dtype=dt, device=rt.device) for name, (shape, dt) in s.items()}
            return torch.zeros((max_requests + 1, *s), dtype=torch.float32, device=rt.device)

        self.states = [state_for(s) for s in model.state_shapes()]
        self._pad_pages, self._pad_slot = list(pages), max_requests      # the page and the slot no request ever holds
        # steps whose shape repeats (above all decode steps) replay a CUDA graph per shape; the
        # reference captures one per sequence and token count (crates/engine/src/flint.rs:735-771)
        self.cuda_graphs = cuda_graphs and model.graph_safe()
        self._graphs: "OrderedDict" = OrderedDict()       # least recently replayed first; at most max_graphs are kept
        self._shapes_seen: Dict = {}
        self.max_graphs = 64
        self.graph_max_tokens = 256
        self.graph_replays = 0
        self.graph_captures = 0
        # ids sampled on the device by the step before (greedy decoding that does not wait for the host)
        self.sampled = torch.zeros(max(64, max_requests), dtype=torch.int32, device=rt.device)
        self._feed_limit = 0
        self._pinned: Optional[torch.Tensor] = None
        self._pinned_free: Optional[torch.cuda.Event] = None      # set once the last upload has left the pinned block

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, tensor_cores: bool = True,
                    cuda_graphs: bool = True):
        arch, cfg = load_config(folder)
        model = DecoderModel(arch.build_spec(cfg))
        rt = Runtime(torch.device(device), parse_dtype(dtype), tensor_cores)
        get = load_folder(folder, model.tensors(), model.spec.name_alias, device=rt.device)
        model.bind(get, rt)
        if get.uploader is not None:
            get.uploader.finish()
        ps = page_size or getattr(cfg, "kv_page_size", None) or 16
        return cls(model, rt, ps, num_pages, max_requests, cuda_graphs)

    @classmethod
    def from_random(cls, cfg, seed: int, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, tensor_cores: bool = True,
                    arch=None, cuda_graphs: bool = True):
        """Random weights made on the device from the typed config and a seed (no files)."""
        from ..config.registry import get_architecture
        arch = arch or get_architecture(cfg.architectures[0])
        spec = arch.build_spec(cfg)
        model = DecoderModel(spec)
        rt = Runtime(torch.device(device), parse_dtype(dtype), tensor_cores)
        model.bind(random_getter(model.tensors(), seed, spec.init_std, device=rt.device), rt)
        ps = page_size or getattr(cfg, "kv_page_size", None) or 16
        return cls(model, rt, ps, num_pages, max_requests, cuda_graphs)

    # ------------------------------------------------------------------ requests
    def add_request(self, rid: Hashable) -> None:
        self.reset_slot(self.manager.add(rid))

    def reset_slot(self, slot: int) -> None:
        """Clear the per-request state a new request finds in its slot."""
        for s in self.states:
            for t in (s.values() if isinstance(s, dict) else () if s is None else (s,)):
                t[slot].zero_()

    def end_request(self, rid: Hashable) -> None:
        self.manager.remove(rid)

    def assume_cached(self, rid: Hashable, n_tokens: int) -> None:
        """Take pages for the request's next n_tokens positions and count them as computed without
        running the model: the caller has put (or will put) keys and values into those pages.
        Benchmarks use it to stand at a given context length without a prefill."""
        self.manager.reserve(rid, n_tokens)
        self.manager.commit(rid)

    def has_request(self, rid: Hashable) -> bool:
        return rid in self.manager.requests

    # ------------------------------------------------------------------ the step
    def _context(self, entries: Sequence[StepEntry], widths: Optional[List[int]] = None,
                 static: Optional[torch.Tensor] = None, pad: int = 0) -> StepContext:
        """The step's description: built on the host in one pinned block, uploaded in one copy
        (into `static` when given: a device block a CUDA graph reads).  pad: filler entries after
        the real ones (one token each at position 0 of a page no request holds, logits wanted)."""
        R = len(entries) + pad
        q_lens = [len(e.tokens) for e in entries] + [1] * pad
        if widths is None:
            widths = self._widths(entries)
        n_want = sum(len(e.want) for e in entries) + pad
        total = 3 * sum(q_lens) + (R + 1) + 2 * R + n_want + sum(R * w for w in widths)
        if self._pinned_free is not None:
            self._pinned_free.synchronize()
        if self._pinned is None or self._pinned.numel() < total:
            self._pinned = torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True)
        written, T, n_want, max_context, max_q_len = self.manager.pack_step(
            [e.rid for e in entries], [e.tokens for e in entries], [e.want for e in entries], widths, self.vocab_size,
            self._pinned.numpy(), self._feed_limit, pad, self._pad_pages, self._pad_slot)
        assert written == total
        o = 3 * T
        host = self._pinned.numpy()
        pos_starts = host[o + R + 1:o + 2 * R + 1].tolist()
        slots = host[o + 2 * R + 1:o + 3 * R + 1].tolist()
        dev = static if static is not None else torch.empty(total, dtype=torch.int32, device=self.rt.device)
        if dev.numel() != total:
            raise RuntimeError("the static step block does not match this step's layout")
        dev.copy_(self._pinned[:total], non_blocking=True)
        if self._pinned_free is None:
            self._pinned_free = torch.cuda.Event()
        self._pinned_free.record()
        o = 0

        def view(n):
            nonlocal o
            v = dev[o:o + n]
            o += n
            return v

        d_tok, d_pos, d_rot = view(T), view(T), view(T)
        d_qs, d_ps, d_sl, d_lr = view(R + 1), view(R), view(R), view(n_want)
        d_tabs = [view(R * wd).view(R, wd) for wd in widths]
        return StepContext(T=T, R=R, token_ids=d_tok, positions=d_pos, req_of_token=d_rot, q_start=d_qs, pos_start=d_ps,
                           slot_ids=d_sl, block_tables=d_tabs, logit_rows=d_lr, n_logit_rows=n_want, q_lens=q_lens,
                           pos_starts=pos_starts, slots=slots,
                           max_context=max_context, max_q_len=max_q_len, fed=self.sampled)

    def _widths(self, entries: Sequence[StepEntry]) -> List[int]:
        mgr = self.manager
        return [max(1, max(mgr.table_len(e.rid, g) for e in entries)) for g in range(len(self.group_specs))]

    def _forward(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Eager for steps of a new shape; a step whose shape (tokens and wanted places per entry,
        block-table widths) has been seen before replays a CUDA graph recorded for that shape.
        Decode steps are recorded at once; other shapes when they come a second time.  Steps of
        more than graph_max_tokens tokens always run eagerly: their kernels are long enough to
        hide the launches, and in mixed traffic their shapes seldom repeat often enough to repay
        a recording."""
        if not self.cuda_graphs or sum(len(e.tokens) for e in entries) > self.graph_max_tokens:
            return self.model.forward(self._context(entries), self.caches, self.states)
        widths = [(w + 63) // 64 * 64 for w in self._widths(entries)]
        shape = tuple((len(e.tokens), tuple(e.want)) for e in entries)
        decode = all(len(e.tokens) == 1 for e in entries)
        # decode batches of nearby sizes share one recording: filler entries bring the batch to the next size of a short
        # list, so that a request that ends or arrives seldom means a new recording (their rows are dropped below)
        pad = self.decode_bucket(len(entries)) - len(entries) if decode and all(tuple(e.want) == (0,) for e in entries) else 0
        real_rows = sum(len(e.want) for e in entries)
        shape += ((1, (0,)),) * pad
        key = (shape, tuple(widths))
        slot = self._graphs.get(key)
        if slot is None:
            seen = self._shapes_seen.get(key, 0) + 1
            self._shapes_seen[key] = seen
            if not decode and seen < 2:
                if len(self._shapes_seen) > 4096:
                    self._shapes_seen.clear()
                return self.model.forward(self._context(entries), self.caches, self.states)
            # run the step eagerly from a static block, then record the same launches into a graph
            # (recording executes nothing)
            R, T = len(entries) + pad, sum(len(e.tokens) for e in entries) + pad
            n_want = real_rows + pad
            total = 3 * T + (R + 1) + 2 * R + n_want + sum(R * w for w in widths)
            static = torch.empty(total, dtype=torch.int32, device=self.rt.device)
            ctx = self._context(entries, widths, static, pad)
            ctx.max_context = max(widths) * self.page_size          # launch plans must hold for every replay
            logits = self.model.forward(ctx, self.caches, self.states)
            result = logits[:real_rows].clone() if logits is not None else None
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            before = ops.launch_count
            ctx.made.clear()                        # plans filled on the device are filled again inside the recording
            with torch.cuda.graph(graph):
                out = self.model.forward(ctx, self.caches, self.states)
            self._graphs[key] = (graph, ctx, static, out, ops.launch_count - before)
            self.graph_captures += 1
            while len(self._graphs) > self.max_graphs:              # the graph replayed longest ago goes, with its buffers
                self._graphs.popitem(last=False)
            return result
        self._graphs.move_to_end(key)
        graph, ctx, static, out, launches = slot
        self._context(entries, widths, static, pad)
        graph.replay()
        self.graph_replays += 1
        ops.launch_count += launches
        return out[:real_rows] if out is not None else None

    @staticmethod
    def decode_bucket(n: int) -> int:
        """The batch size a decode step of n requests is recorded at: n up to 8, then the next
        multiple of 4 up to 32, of 8 up to 64, of 16 beyond (at most a third more rows at 9, a quarter beyond 32)."""
        if n <= 8:
            return n
        unit = 4 if n <= 32 else 8 if n <= 64 else 16
        return (n + unit - 1) // unit * unit

    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        return self.manager.can_reserve([(e.rid, len(e.tokens)) for e in entries])

    def step(self, entries: Sequence[StepEntry], feed_limit: int = 0) -> Optional[torch.Tensor]:
        """Run the entries' tokens as one batch; FP32 logits [wanted, vocab] in the order of the
        entries and of their `want` (None if nothing is wanted).  Raises OutOfPages, leaving every
        request as it was, if the pools cannot hold the step.  feed_limit > 0: a token id -(i + 1),
        i < feed_limit, stands for self.sampled[i], an id the step before left on the device."""
        self._feed_limit = feed_limit
        entries = [e for e in entries if len(e.tokens)]
        if not entries:
            return None
        rids = [e.rid for e in entries]
        if len(set(rids)) != len(rids):
            raise ValueError("a request appears twice in one step")
        if not self.can_run(entries):
            raise OutOfPages("the page pools cannot hold this step: " +
                             ", ".join(f"{e.rid!r}+{len(e.tokens)}" for e in entries))
        for e in entries:
            self.manager.reserve(e.rid, len(e.tokens))
        try:
            logits = self._forward(entries)
        except BaseException:
            for e in entries:
                self.manager.cancel(e.rid)
            raise
        for e in entries:
            self.manager.commit(e.rid)
        return logits
