"""The Python entry point: an engine that owns the model, the cache, the scheduler and the sampler.

    eng = Engine.from_folder("model_dir", dtype="bfloat16")
    outs = eng.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=16, temperature=0))

Token ids in, token ids out (the reference's tokenizer and chat template,
crates/cli/src/chat.rs, are outside this engine).  `step()` runs one scheduled batch;
`generate()` runs until every given prompt has finished.

While no live request uses penalties, `step()` does not wait for the tokens of the step it has just
launched: the choice (argmax, or the sampler's arithmetic on the candidate pools with a uniform the
host has drawn from the request's stream) is made on the device and stays there, the next step's
embedding reads it, and the host plans that next step with placeholders, reading the real ids (one
step late) while the GPU already works.  What the host needs a token's value for is the stop test;
a request that turns out to have produced a stop token is ended then, the one token computed
beyond it is dropped, and the tokens it returns are the same as without the look-ahead (the tests
compare both).  A request with penalties is chosen by the host sampler, which needs the tokens it
has generated: while one lives, the engine waits for each step.
"""
from __future__ import annotations

import itertools
import random
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from .. import ops
from ..sampling import Sampler, SamplingParams, SplitMix64
from ..sampling.sampler import ROW_RECORD, device_rows, pool_size
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import FINISH_CANCELLED, Request, ScheduledStep, Scheduler

PENDING = -1          # an output token whose value is still on the device


@dataclass
class RequestOutput:
    rid: Hashable
    prompt: List[int]
    tokens: List[int]
    finish_reason: Optional[str]
    preemptions: int = 0


@dataclass
class _InFlight:
    """A launched step whose sampled ids the host has not read yet."""
    samplers: List[Request]
    index: List[int]                      # where each sampler's placeholder sits in its output
    host: torch.Tensor                    # pinned int32, filled by a copy enqueued behind the step
    ready: "torch.cuda.Event"


class Engine:
    def __init__(self, runner: ModelRunner, max_batch_tokens: int = 2048, max_running: Optional[int] = None,
                 lookahead: bool = True):
        self.runner = runner
        self.scheduler = Scheduler(runner.manager, max_batch_tokens, max_running, on_admit=runner.reset_slot)
        self.sampler = Sampler()
        self._ids = itertools.count()
        self.eos = list(runner.model.spec.eos_token_ids)
        self.stats = {"steps": 0, "tokens": 0, "preemptions": 0, "lookahead_steps": 0}
        self.lookahead = lookahead
        self._inflight: Optional[_InFlight] = None
        self._held: List[Request] = []     # ended, but their last token is still a placeholder
        self._pinned_ids = [None, None]
        self._flip = 0
        self._pinned_rows = [None, None]   # sampling records of the steps in flight (two: one is read while the next is written)
        self._flip_rows = 0
        self._ended_early: List[Request] = []     # ended outside step() (resolved by abort), reported by the next step()

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, max_batch_tokens: int = 2048,
                    tensor_cores: bool = True, lookahead: bool = True) -> "Engine":
        runner = ModelRunner.from_folder(folder, dtype, device, page_size, num_pages, max_requests, tensor_cores)
        return cls(runner, max_batch_tokens, lookahead=lookahead)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, max_batch_tokens: int = 2048,
                    tensor_cores: bool = True, lookahead: bool = True) -> "Engine":
        runner = ModelRunner.from_random(config, seed, dtype, device, page_size, num_pages, max_requests, tensor_cores)
        return cls(runner, max_batch_tokens, lookahead=lookahead)

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, rid: Optional[Hashable] = None) -> Hashable:
        params = params or SamplingParams()
        if rid is None:
            rid = next(self._ids)
        prompt = [int(t) for t in prompt]
        for t in prompt:
            if not 0 <= t < self.runner.vocab_size:
                raise ValueError(f"token id {t} outside 0..{self.runner.vocab_size - 1}")
        if not params.stop_tokens and self.eos:
            params = SamplingParams(**{**params.__dict__, "stop_tokens": list(self.eos)})
        seed = params.seed if params.seed is not None else random.getrandbits(64)
        req = Request(rid, prompt, params, rng=SplitMix64(seed))
        self.scheduler.add(req)
        return rid

    def adopt_request(self, prompt: Sequence[int], first_token: int, params: Optional[SamplingParams] = None,
                      rid: Optional[Hashable] = None) -> Hashable:
        """Add a request whose prompt is taken to be in the cache already, with its first generated
        token given: it decodes from its next step on.  Pages for the prompt are taken here; their
        contents are the caller's business (benchmarks fill the pools with random values)."""
        params = params or SamplingParams()
        params.validate()
        if rid is None:
            rid = next(self._ids)
        seed = params.seed if params.seed is not None else random.getrandbits(64)
        req = Request(rid, [int(t) for t in prompt], params, output=[int(first_token)], rng=SplitMix64(seed))
        self.runner.add_request(rid)
        step = self.scheduler.max_batch_tokens          # pages are taken as portions of a chunked prefill would take them
        for at in range(0, len(req.prompt), step):
            self.runner.assume_cached(rid, min(step, len(req.prompt) - at))
        self.scheduler.adopt(req)
        return rid

    def abort(self, rid: Hashable) -> None:
        """End a live request now (reason "cancelled", the reference's Finish::Cancelled); the next
        step() reports it with the tokens it had produced."""
        self._ended_early += self._resolve()     # every token known before the queue changes
        req = self.scheduler.abort(rid)
        if req is not None:
            self._ended_early.append(req)

    def has_unfinished(self) -> bool:
        """Whether step() still has something to run or to report."""
        return self.scheduler.has_work() or self._inflight is not None or bool(self._held) or bool(self._ended_early)

    # ------------------------------------------------------------------ stepping
    def _device_picks(self) -> bool:
        """Whether every live request's next token can be chosen on the device (greedy, or sampled
        without penalties): then a step need not wait for the one before."""
        return not any(r.params.penalized for r in self.scheduler.by_id.values())

    def _pick_on_device(self, logits: torch.Tensor, samplers: List[Request]) -> torch.Tensor:
        """The step's next tokens into runner.sampled, without a word to the host."""
        vocab = self.runner.vocab_size
        if all(pool_size(r.params, vocab) == 1 for r in samplers):
            return ops.argmax(logits, out=self.runner.sampled)
        n = len(samplers)
        self._flip_rows ^= 1
        host = self._pinned_rows[self._flip_rows]
        if host is None or host.shape[0] < n:
            host = self._pinned_rows[self._flip_rows] = torch.empty((max(64, n), 8), dtype=torch.int32, pin_memory=True)
        k = device_rows([r.params for r in samplers], [r.rng for r in samplers], vocab, host.numpy().view(ROW_RECORD).reshape(-1))
        rows = host[:n].to(logits.device, non_blocking=True)
        ids, vals = ops.topk_pool(logits, k)
        return ops.sample_pool(ids, vals, rows, out=self.runner.sampled)

    def _resolve(self) -> List[Request]:
        """Read the ids of the step in flight (waits for that step only), put them where their
        placeholders stand, end the requests that turn out to have stopped; returns the requests
        that have ended and whose tokens are all known."""
        flight, self._inflight = self._inflight, None
        if flight is not None:
            flight.ready.synchronize()
            toks = flight.host[:len(flight.samplers)].tolist()
            for req, at, tok in zip(flight.samplers, flight.index, toks):
                if at >= len(req.output) or req.finish_reason == FINISH_CANCELLED:
                    continue                   # dropped since: the request had stopped before, or was aborted
                self.scheduler.set_output_token(req, at, tok)
                if tok in req.params.stop_tokens:
                    ended_before = req.finished
                    self.scheduler.stop_at(req, at + 1)       # also outranks a provisional "length" at the same token
                    if not ended_before:
                        self._held.append(req)
        out = [r for r in self._held if PENDING not in r.output]
        self._held = [r for r in self._held if PENDING in r.output]
        return out

    def _entries(self, plan: ScheduledStep) -> List[StepEntry]:
        """The plan's tokens; a placeholder becomes the code of the device id that stands for it."""
        source = {id(r): i for i, r in enumerate(self._inflight.samplers)} if self._inflight is not None else {}
        out = []
        for e in plan.entries:
            toks = e.request.token_slice(e.start, e.count)
            if PENDING in toks:
                toks = [t if t != PENDING else -(source[id(e.request)] + 1) for t in toks]
            out.append(StepEntry(e.request.rid, toks, [e.count - 1] if e.samples else []))
        return out

    def step(self) -> List[RequestOutput]:
        """Schedule and run one batch; returns the requests that ended and whose tokens are all known
        (with the look-ahead, a request is reported one call after the step that ended it)."""
        ended, self._ended_early = self._ended_early, []
        ahead = self.lookahead and self._device_picks()
        if self._inflight is not None and not ahead:
            ended += self._resolve()           # the host samples the next tokens itself: it needs every earlier one
        plan: ScheduledStep = self.scheduler.schedule()
        self.stats["preemptions"] += len(plan.preempted)
        self._held += plan.finished
        before = self._inflight
        if plan.entries:
            entries = self._entries(plan)
            logits = self.runner.step(entries, feed_limit=len(before.samplers) if before is not None else 0)
            samplers = [e.request for e in plan.entries if e.samples]
            if samplers and ahead:
                ids = self._pick_on_device(logits, samplers)               # stays on the device for the next step's embedding
                self._flip ^= 1
                host = self._pinned_ids[self._flip]
                if host is None or host.numel() < len(samplers):
                    host = self._pinned_ids[self._flip] = torch.empty(max(64, len(samplers)), dtype=torch.int32, pin_memory=True)
                host[:len(samplers)].copy_(ids, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record()
                self._held += self.scheduler.update(plan, [PENDING] * len(samplers))      # ends by length are known without the values
                self._inflight = _InFlight(samplers, [len(r.output) - 1 for r in samplers], host, ready)
                self.stats["lookahead_steps"] += 1
            else:
                sampled: List[int] = []
                if samplers:
                    sampled = self.sampler.sample(logits, [r.params for r in samplers], [r.output for r in samplers],
                                                  [r.rng for r in samplers])
                self._held += self.scheduler.update(plan, sampled)
                self._inflight = None
            self.stats["steps"] += 1
            self.stats["tokens"] += plan.num_tokens
        else:
            self._inflight = None
        # the step before: its ids have reached the host while this one was planned and launched
        if before is not None:
            now, self._inflight = self._inflight, before
            ended += self._resolve()
            self._inflight = now
        else:
            ended += [r for r in self._held if PENDING not in r.output]
            self._held = [r for r in self._held if PENDING in r.output]
        return [RequestOutput(r.rid, r.prompt, list(r.output), r.finish_reason, r.preemptions) for r in ended]

    def generate(self, prompts: Sequence[Sequence[int]], params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> List[RequestOutput]:
        """Run the prompts to completion; outputs in the order of the prompts."""
        if params is None or isinstance(params, SamplingParams):
            params = [params or SamplingParams()] * len(prompts)
        if len(params) != len(prompts):
            raise ValueError("one SamplingParams per prompt is needed")
        rids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        results: Dict[Hashable, RequestOutput] = {}
        while len(results) < len(rids):
            if not self.has_unfinished():
                raise RuntimeError("the scheduler has no work left but requests are unfinished")
            for out in self.step():
                results[out.rid] = out
        return [results[r] for r in rids]
