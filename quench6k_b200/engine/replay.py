"""The loop of the trace replay tool: one JSON step in, one logits block out.

A step is {"step": n, "entries": [{"id", "tokens", "want"}], "end": [ids]}.  Entries of unknown
ids start new requests; `end` gives back what the named requests hold after the step.  The loop
calls ModelRunner.step and nothing else: no sampling, no scheduling.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional

import torch

from .batch import StepEntry
from .runner import ModelRunner


def pool_pages(max_tokens: int, page_size: int) -> int:
    """Pages per cache group for `max_tokens` token places, counted in units of 64 tokens (or of
    the page size, if that is larger)."""
    unit = max(64, page_size)
    unit = (unit + page_size - 1) // page_size * page_size
    tokens = (max_tokens + unit - 1) // unit * unit
    return max(1, tokens // page_size)


def replay(runner: ModelRunner, steps: Iterable[Dict], emit: Callable[[int, Optional[torch.Tensor]], None]) -> None:
    """Run the steps in order; `emit(step_number, logits or None)` is called after each."""
    for msg in steps:
        entries = []
        for e in msg.get("entries", []):
            rid = e["id"]
            if not runner.has_request(rid):
                runner.add_request(rid)
            entries.append(StepEntry(rid, e["tokens"], e.get("want", [])))
        logits = runner.step(entries)
        for rid in msg.get("end", []):
            if runner.has_request(rid):
                runner.end_request(rid)
        emit(msg["step"], logits)
