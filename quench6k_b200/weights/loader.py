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


class Uploader:
    """Tensor data from a file to the device through two pinned staging buffers: while one piece
    is on its way to the device the next is read from the file into the other buffer (the
    reference stages through 64 MiB of pinned memory, crates/engine/src/flint.rs:91,136-157, and
    double-buffers on its other path, crates/engine/src/loader.rs:1-9)."""

    def __init__(self, device, piece_bytes: int = 64 << 20):
        self.device = torch.device(device)
        self.piece = piece_bytes
        self.buffers = [torch.empty(piece_bytes, dtype=torch.uint8, pin_memory=True) for _ in range(2)]
        self.sent: List[Optional[torch.cuda.Event]] = [None, None]
        self.flip = 0
        self.bytes = 0

    def into(self, sf, name: str, dst: torch.Tensor) -> None:
        """The stored bytes of tensor `name` of file `sf` into the device tensor dst (contiguous, the stored dtype)."""
        flat = dst.view(-1).view(torch.uint8)
        total = flat.numel()
        with torch.cuda.device(self.device):
            for off in range(0, total, self.piece):
                n = min(self.piece, total - off)
                b = self.flip
                if self.sent[b] is not None:
                    self.sent[b].synchronize()             # the copy that last used this buffer has left it
                sf.read_range(name, off, self.buffers[b][:n])
                flat[off:off + n].copy_(self.buffers[b][:n], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record()
                self.sent[b] = ev
                self.flip ^= 1
        self.bytes += total

    def finish(self) -> None:
        for ev in self.sent:
            if ev is not None:
                ev.synchronize()


def load_folder(folder: str, declared: List[TensorSpec],
                alias: Optional[Callable[[str], object]] = None, device=None) -> Callable[[str], torch.Tensor]:
    """Check the folder's tensors against the declaration; return `get(name) -> tensor` that reads
    one tensor at a time (so that a large model never sits in host memory whole).  With `device`
    (a CUDA device) the tensors come back on it, streamed through two pinned staging buffers;
    else on the CPU.

    alias: a stored tensor whose name is not declared is looked up under alias(its name) (an
    architecture's table of other naming schemes): the declared name, or (declared name, i) for a
    tensor that is slice i along the first axis of the declared one (experts stored one by one are
    stacked as they are read).  A tensor under another name may also be stored with its leading
    dimensions flattened ([E*I, D] for a declared [E, I, D]) and is reshaped when read."""
    index = index_folder(folder)
    want = {s.name: s for s in declared}
    stored_as: Dict[str, str] = {}                       # declared (or unknown) name -> name in the files
    slices: Dict[str, Dict[int, str]] = {}               # declared name -> slice index -> name in the files
    wrong: List[str] = []
    for n in index:
        target = n
        if n not in want and alias is not None:
            target = alias(n) or n
        if isinstance(target, tuple):
            target, i = target
            if target in stored_as or i in slices.get(target, {}):
                raise WeightError([], [], [f"{target}[{i}]: stored twice, the second time as {n}"])
            slices.setdefault(target, {})[int(i)] = n
            continue
        if target in stored_as or target in slices:
            raise WeightError([], [], [f"{target}: stored twice, as {stored_as.get(target, 'slices')} and as {n}"])
        stored_as[target] = n
    found = {}
    missing_slices: List[str] = []
    for target, n in stored_as.items():
        e = index[n][1]
        shape = tuple(e.shape)
        spec = want.get(target)
        if spec is not None and target != n and shape != tuple(spec.shape) and len(shape) >= 1 and len(spec.shape) > len(shape) \
                and shape[-1] == spec.shape[-1] and _count(shape) == _count(spec.shape):
            shape = tuple(spec.shape)                    # leading dimensions flattened in the other scheme
        found[target] = (e.dtype, shape)
    for target, parts in slices.items():
        spec = want.get(target)
        if spec is None:                                 # an alias to a tensor this model does not declare: report the stored names
            for n in parts.values():
                found[n] = (index[n][1].dtype, tuple(index[n][1].shape))
            continue
        some = next(iter(parts.values()))
        for i in range(spec.shape[0]):
            if i not in parts:
                missing_slices.append(f"{target}[{i}] (stored one by one, like {some})")
        for i, n in sorted(parts.items()):
            e = index[n][1]
            if i >= spec.shape[0]:
                found[n] = (e.dtype, tuple(e.shape))     # beyond the declared count: unexpected
            elif tuple(e.shape) != tuple(spec.shape[1:]):
                wrong.append(f"{n}: shape {list(e.shape)}, expected {list(spec.shape[1:])}")
            elif e.dtype != index[some][1].dtype:
                wrong.append(f"{n}: dtype {e.dtype}, the other slices of {target} are {index[some][1].dtype}")
        found[target] = (index[some][1].dtype, tuple(spec.shape))
    try:
        check_against(declared, found)
    except WeightError as err:
        raise WeightError(sorted(err.missing + missing_slices), err.unexpected, err.wrong + wrong) from None
    if missing_slices or wrong:
        raise WeightError(sorted(missing_slices), [], wrong)

    on_device = device is not None and torch.device(device).type == "cuda"
    uploader = Uploader(device) if on_device else None
    direct = (torch.bfloat16, torch.float32, torch.int32)    # stored as they are kept: straight through the staging buffers

    def pieces(name: str):
        """(file, stored name, slice index or None) of everything that makes up the declared tensor."""
        if name in slices:
            return [(index[n][0], n, i) for i, n in sorted(slices[name].items())]
        return [(index[stored_as[name]][0], stored_as[name], None)]

    def get(name: str) -> torch.Tensor:
        shape = tuple(want[name].shape)
        parts = pieces(name)
        dtype = index[parts[0][1]][1].dtype
        if on_device and dtype in direct:
            out = torch.empty(shape, dtype=dtype, device=device)
            for sf, n, i in parts:
                uploader.into(sf, n, out if i is None else out[i])
            return out
        if len(parts) == 1 and parts[0][2] is None:
            t = _stored(parts[0][0].read(parts[0][1])).reshape(shape)
        else:
            t = torch.stack([_stored(sf.read(n)) for sf, n, _ in parts]).reshape(shape)
        return t.to(device) if on_device else t

    get.uploader = uploader
    return get


def _count(shape) -> int:
    n = 1
    for d in shape:
        n *= int(d)
    return n
