"""Weights by tensor name.

The set of tensors a model needs is declared by its parts (spec.TensorSpec); the loader compares
that declaration with what the files hold and reports, in ONE error, every missing tensor, every
unexpected tensor and every wrong shape or dtype class (the reference checks tensor by tensor:
crates/engine/src/gguf.rs:202-214, crates/engine/src/flint.rs:297-300,316-319,340-343).

Stored dtypes are kept: bfloat16 stays bfloat16, a tensor stored in 32-bit stays 32-bit, integer
tables become int32.  Conversion to what a kernel consumes happens when a part binds its tensors.
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional

import torch

from ..spec import TensorSpec
from .safetensors_io import index_folder

_FLOATS = (torch.bfloat16, torch.float16, torch.float32, torch.float64)
_INTS = (torch.int8, torch.uint8, torch.int16, torch.int32, torch.int64)


class WeightError(ValueError):
    """The checkpoint does not hold what the model declares."""

    def __init__(self, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shape or dtype ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def check_against(declared: List[TensorSpec], found: Dict[str, tuple]) -> None:
    """found: name -> (dtype, shape).  Raises WeightError listing every discrepancy at once."""
    want = {s.name: s for s in declared}
    missing = sorted(n for n in want if n not in found)
    unexpected = sorted(n for n in found if n not in want)
    wrong = []
    for n, s in want.items():
        if n not in found:
            continue
        dt, shape = found[n]
        if tuple(shape) != tuple(s.shape):
            wrong.append(f"{n}: shape {list(shape)}, expected {list(s.shape)}")
        elif s.role == "i32" and dt not in _INTS:
            wrong.append(f"{n}: dtype {dt}, expected an integer type")
        elif s.role != "i32" and dt not in _FLOATS:
            wrong.append(f"{n}: dtype {dt}, expected a floating type")
    if missing or unexpected or wrong:
        raise WeightError(missing, unexpected, wrong)


def _stored(t: torch.Tensor) -> torch.Tensor:
    """What is kept: bfloat16 and float32 as they are; other floats as float32 if wider than 16
    bits else bfloat16; integers as int32."""
    if t.dtype in (torch.bfloat16, torch.float32):
        return t
    if t.dtype == torch.float64:
        return t.to(torch.float32)
    if t.dtype == torch.float16:
        return t.to(torch.bfloat16)
    if t.dtype in _INTS:
        return t.to(torch.int32)
    return t


def load_folder(folder: str, declared: List[TensorSpec],
                alias: Optional[Callable[[str], Optional[str]]] = None) -> Callable[[str], torch.Tensor]:
    """Check the folder's tensors against the declaration; return `get(name) -> CPU tensor`
    that reads one tensor at a time (so that a large model never sits in host memory whole).
    alias: a stored tensor whose name is not declared is looked up under alias(its name) (an
    architecture's table of other naming schemes); such a tensor may also be stored with its leading
    dimensions flattened ([E*I, D] for a declared [E, I, D]) and is reshaped when read."""
    index = index_folder(folder)
    want = {s.name: s for s in declared}
    stored_as: Dict[str, str] = {}                       # declared (or unknown) name -> name in the files
    for n in index:
        target = n
        if n not in want and alias is not None:
            target = alias(n) or n
        if target in stored_as:
            raise WeightError([], [], [f"{target}: stored twice, as {stored_as[target]} and as {n}"])
        stored_as[target] = n
    found = {}
    for target, n in stored_as.items():
        e = index[n][1]
        shape = tuple(e.shape)
        spec = want.get(target)
        if spec is not None and target != n and shape != tuple(spec.shape) and len(shape) >= 1 and len(spec.shape) > len(shape) \
                and shape[-1] == spec.shape[-1] and _count(shape) == _count(spec.shape):
            shape = tuple(spec.shape)                    # leading dimensions flattened in the other scheme
        found[target] = (e.dtype, shape)
    check_against(declared, found)

    def get(name: str) -> torch.Tensor:
        sf, _ = index[stored_as[name]]
        return _stored(sf.read(stored_as[name])).reshape(want[name].shape)

    return get


def _count(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n
