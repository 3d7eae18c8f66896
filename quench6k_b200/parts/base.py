"""Interfaces of the parts a layer is put together from, and their registries.

A part gets its sizes and constants as constructor parameters, declares the tensors it needs
(names relative to its own prefix), binds them once, and runs on whatever rows the step hands it.
No part knows which model it is in.

To add a part, subclass the matching base, implement the methods below and register the class
under a name with the matching `register_*`; a spec.PartSpec(kind=name, params=...) then selects it.

  Norm            tensors(); bind(); forward(h_f32 [T, D], rows=None, add=None) -> [R, D] in the operand dtype;
                  with `add` (float32 [T, D], or [slices, T, D] partial sums to be added in order) it
                  first stores h += add (the block's residual add, fused)
  PositionEncoding  tensors(); bind(); rotary_table() -> (inv_freq, rotary_dim, neighbours) for a rotation of pairs
                  of head dimensions (applied inside the q/k kernel), or None and then
                  apply(x_f32 [T, H, hd], positions_i32 [T]) -> None, in place
  Mixer           tensors(); bind(); cache_request() -> CacheRequest | None (kind, window, heads, key and value widths, dtype);
                  state_shape() -> None | shape of one float32 tensor | {name: (shape, dtype)};
                  forward(xn [T, D], ctx: StepContext, cache: LayerCache | None, state: Tensor | None, out_f32 [T, D])
                  adds its result into `out` and returns None, or leaves `out` alone and returns the
                  float32 [T, D] result (or [slices, T, D] partial sums) for the block's next norm to add
  FeedForward     tensors(); bind(); forward(xn [T, D], ctx, out_f32 [T, D]) adds its result into `out`
  Block           built from (norm1, mixer, norm2, ffn); forward(h, ctx, cache, state)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch

from ..spec import PartSpec, TensorSpec


@dataclass
class Runtime:
    """Where and in which precision the parts run."""
    device: torch.device
    dtype: torch.dtype                  # operand, activation and cache dtype: bfloat16, or float32 for the true 32-bit path
    tensor_cores: bool = True           # bfloat16 only: use the tcgen05 kernels where a shape allows

    @property
    def is_fp32(self) -> bool:
        return self.dtype == torch.float32


@dataclass
class CacheRequest:
    """What a mixer needs from the cache manager.  Layers with equal requests share a group
    (one block table per request and group)."""
    kind: str                           # "full": every key; "sliding": the last `window` keys
    window: Optional[int]
    kv_heads: int
    head_dim: int                       # width of a key
    v_dim: Optional[int] = None         # width of a value; None: the key's
    dtype: Optional[torch.dtype] = None  # what the pages hold; None: the runtime's operand dtype

    def key(self) -> Tuple:
        return (self.kind, self.window, self.kv_heads, self.head_dim, self.v_dim or self.head_dim, self.dtype)


@dataclass
class LayerCache:
    """The pages of one executed layer position.  k: [kv_heads, num_pages, page_size, head_dim],
    v: [kv_heads, num_pages, page_size, v_dim] (head-major, so that pages with consecutive numbers
    lie next to each other for one head)."""
    group: int
    k: torch.Tensor
    v: torch.Tensor
    page_size: int
    write: bool = True                  # False: this position reads the pages another position wrote


class Part:
    # True if forward() launches the same kernels with the same arguments whenever the step has
    # the same number of rows and the same block-table widths (everything else read on the device):
    # such steps may be replayed from a CUDA graph.  The token counts (q_lens) are part of a
    # recorded step's identity and may shape the launches; where the requests stand (pos_starts)
    # and their slots are not: a part whose launches depend on them must leave this False (the
    # attention part plans its key splits on the device for that reason; the order of its
    # prompt tiles, which only balances the load, is the one thing it takes from pos_starts).
    graph_safe = False

    def tensors(self) -> List[TensorSpec]:
        return []

    def bind(self, get: Callable[[str], torch.Tensor], rt: Runtime) -> None:
        """`get(name)` returns the stored tensor (on any device, stored dtype) by relative name."""
        self.rt = rt


@dataclass
class WeightedRows:
    """A residual add that has not been made yet: h[t] += sum_s weights[t, s] * y[pair_row[t, s]]
    (pair_row None: row t*S + s).  A feed-forward may return it instead of adding, and the next
    norm (the next block's first, or the model's last) makes the add in the pass that normalises."""
    y: torch.Tensor                       # FP32 [pairs, D]
    weights: torch.Tensor                 # FP32 [T, S]
    pair_row: Optional[torch.Tensor] = None

    def apply(self, h: torch.Tensor) -> None:
        from .. import ops
        ops.combine(self.y, self.pair_row, self.weights, h)


class Tap:
    """A debugging aid: a part that is given a Tap copies small per-row results of every forward
    into it (the routed experts: each row's chosen experts and its router logits), one static
    device buffer per name and executed position, so that the copies are part of a recorded CUDA
    graph and a replayed step fills the same buffers.  Off unless a caller sets it; every copy
    costs a launch."""

    def __init__(self, capacity_rows: int):
        self.capacity = int(capacity_rows)
        self.buffers: Dict[Tuple[str, int], torch.Tensor] = {}

    def record(self, what: str, position: int, rows: torch.Tensor) -> None:
        n = rows.shape[0]
        if n > self.capacity:
            raise ValueError(f"tap: a step of {n} rows exceeds the tap's {self.capacity}")
        buf = self.buffers.get((what, position))
        if buf is None:
            buf = self.buffers[(what, position)] = torch.zeros((self.capacity, *rows.shape[1:]), dtype=rows.dtype, device=rows.device)
        buf[:n].copy_(rows)


class Norm(Part):
    fuses_weighted_rows = False           # forward(..., add=WeightedRows) is understood

    def forward(self, h: torch.Tensor, rows: Optional[torch.Tensor] = None, add=None) -> torch.Tensor:
        """Normalised rows of h in the operand dtype.  `add`: FP32 of h's shape, or [slices, T, D]
        partial sums, or (if fuses_weighted_rows) a WeightedRows: added into h first, in place."""
        raise NotImplementedError


class PositionEncoding(Part):
    is_identity = False                   # True: q and k stay as they are

    def rotary_table(self):
        """(inv_freq float32 [rotary_dim / 2] on the device, rotary_dim, neighbours) of an encoding
        that is a rotation of pairs of head dimensions by position * inv_freq[pair]: the kernel
        that prepares q and k applies it.  None: not such a rotation; `apply` is called instead."""
        return None

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> None:
        """In place on FP32 x [T, heads, head_dim] (q, then k) at int32 positions [T]."""
        raise NotImplementedError


class Mixer(Part):
    def cache_request(self) -> Optional[CacheRequest]:
        return None

    def state_shape(self):
        """This mixer's fixed-size per-request state: None, the shape of one float32 tensor, or
        {name: (shape, dtype)} for several.  forward() gets the tensor [slots, *shape] (or the
        dict of them), indexed by the request's slot; a slot is zeroed when it is handed out."""
        return None

    def forward(self, xn, ctx, cache: Optional[LayerCache], state: Optional[torch.Tensor], out: torch.Tensor) -> Optional[torch.Tensor]:
        raise NotImplementedError


class FeedForward(Part):
    defers_add = False                    # forward(..., defer=True) may return a WeightedRows instead of adding

    def forward(self, xn, ctx, out: torch.Tensor) -> None:
        raise NotImplementedError


class Block:
    def __init__(self, norm1: Norm, mixer: Mixer, norm2: Norm, ffn: FeedForward):
        self.norm1, self.mixer, self.norm2, self.ffn = norm1, mixer, norm2, ffn

    def forward(self, h, ctx, cache, state, pending=None):
        """Runs the block on the stream h in place.  `pending`: an add into h the block before has
        left to this block's first norm; returns the add this block leaves to the next norm, or None."""
        raise NotImplementedError


NORMS: Dict[str, type] = {}
POSITION_ENCODINGS: Dict[str, type] = {}
MIXERS: Dict[str, type] = {}
FEED_FORWARDS: Dict[str, type] = {}
BLOCKS: Dict[str, type] = {}


def _register(table: Dict[str, type], what: str):
    def deco_for(name: str):
        def deco(cls):
            table[name] = cls
            return cls
        return deco
    return deco_for


register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_block = _register(BLOCKS, "block")


def make_part(table: Dict[str, type], what: str, spec: PartSpec, **extra):
    if spec.kind not in table:
        raise KeyError(f"unknown {what} {spec.kind!r}; registered: {', '.join(sorted(table))}")
    return table[spec.kind](**extra, **spec.params)


def to_operand(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    """A stored matrix as the kernels consume it: on the device, in the runtime's operand dtype."""
    return t.to(device=rt.device, dtype=rt.dtype).contiguous()


def to_f32(t: torch.Tensor, rt: Runtime) -> torch.Tensor:
    return t.to(device=rt.device, dtype=torch.float32).contiguous()
