"""Architecture-neutral description of a decoder: what an architecture's builder hands to the engine.

An architecture (config class + builder, see config/registry.py) turns its config.json into a
ModelSpec.  Everything below the builder (weights, parts, cache manager, step function, scheduler)
works from the ModelSpec alone and never asks which architecture it came from.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple


@dataclass
class PartSpec:
    """A part chosen by name from its registry, with its sizes and constants as parameters."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One set of layer weights: the parts and how they are arranged in a block."""
    prefix: str                 # tensor-name prefix, e.g. "model.layers.3."
    mixer: PartSpec
    ffn: PartSpec
    norm: PartSpec              # the kind of both norms of the block
    block: str = "prenorm"      # arrangement, a key of parts.BLOCKS


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    layers: List[LayerSpec]
    order: List[int]                       # executed positions -> index into `layers` (repeats allowed)
    kv_source: List[Optional[int]]         # per executed position: an earlier position whose cache it reads
    final_norm: PartSpec
    embed_name: str = "model.embed_tokens.weight"
    head_name: Optional[str] = "lm_head.weight"    # None: the head is the embedding table (tied)
    final_norm_prefix: str = "model.norm."
    eos_token_ids: Tuple[int, ...] = ()
    init_std: float = 0.02                 # std of the random-weights mode for matrices
    name_alias: Optional[Callable[[str], Optional[str]]] = None   # a stored tensor's other name -> the name declared here (or None)


@dataclass
class TensorSpec:
    """A tensor a part needs.  role: 'matrix' (engine dtype: bfloat16, or float32 in the 32-bit
    path), 'f32' (always float32: norm weights, sinks), 'i32' (integer tables).
    init: ('normal', std) | ('ones',) | ('ones_plus', std) for the random-weights mode."""
    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple = ("normal", None)         # std None -> ModelSpec.init_std
