"""The Python entry point: an engine that owns the model, the cache, the scheduler and the sampler.

    eng = Engine.from_folder("model_dir", dtype="bfloat16")
    outs = eng.generate([[1, 2, 3], [4, 5]], SamplingParams(max_tokens=16, temperature=0))

Token ids in, token ids out (the reference's tokenizer and chat template,
crates/cli/src/chat.rs, are outside this engine).  `step()` runs one scheduled batch;
`generate()` runs until every given prompt has finished.
"""
from __future__ import annotations

import itertools
import random
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Union

import torch

from ..sampling import Sampler, SamplingParams, SplitMix64
from .runner import ModelRunner
from .scheduler import Request, ScheduledStep, Scheduler


@dataclass
class RequestOutput:
    rid: Hashable
    prompt: List[int]
    tokens: List[int]
    finish_reason: Optional[str]
    preemptions: int = 0


class Engine:
    def __init__(self, runner: ModelRunner, max_batch_tokens: int = 2048, max_running: Optional[int] = None):
        self.runner = runner
        self.scheduler = Scheduler(runner.manager, max_batch_tokens, max_running, on_admit=runner.reset_slot)
        self.sampler = Sampler()
        self._ids = itertools.count()
        self.eos = list(runner.model.spec.eos_token_ids)
        self.stats = {"steps": 0, "tokens": 0, "preemptions": 0}

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, max_batch_tokens: int = 2048,
                    tensor_cores: bool = True) -> "Engine":
        runner = ModelRunner.from_folder(folder, dtype, device, page_size, num_pages, max_requests, tensor_cores)
        return cls(runner, max_batch_tokens)

    @classmethod
    def from_random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0", page_size: Optional[int] = None,
                    num_pages: Union[int, Sequence[int]] = 256, max_requests: int = 64, max_batch_tokens: int = 2048,
                    tensor_cores: bool = True) -> "Engine":
        runner = ModelRunner.from_random(config, seed, dtype, device, page_size, num_pages, max_requests, tensor_cores)
        return cls(runner, max_batch_tokens)

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
        self.scheduler.abort(rid)

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ------------------------------------------------------------------ stepping
    def step(self) -> List[RequestOutput]:
        """Schedule and run one batch; returns the requests that ended in it."""
        plan: ScheduledStep = self.scheduler.schedule()
        self.stats["preemptions"] += len(plan.preempted)
        ended = list(plan.finished)
        if plan.entries:
            logits = self.runner.step(plan.step_entries())
            samplers = [e.request for e in plan.entries if e.samples]
            sampled: List[int] = []
            if samplers:
                sampled = self.sampler.sample(logits, [r.params for r in samplers], [r.output for r in samplers],
                                              [r.rng for r in samplers])
            ended += self.scheduler.update(plan, sampled)
            self.stats["steps"] += 1
            self.stats["tokens"] += plan.num_tokens
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
            if not self.scheduler.has_work():
                raise RuntimeError("the scheduler has no work left but requests are unfinished")
            for out in self.step():
                results[out.rid] = out
        return [results[r] for r in rids]
