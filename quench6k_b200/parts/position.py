"""Position encodings.  A rotary one hands the kernel that prepares q and k a table of inverse
frequencies, the number of head dimensions that rotate and how they pair, and the kernel applies
it (reference: crates/cuda/kernels/flint.cu:141-149: rotate-half over the full head with the
literal base 10000); "none" leaves q and k as they are (the reference's per-layer rope flag,
crates/engine/src/flint.rs:254,408).  An encoding that is no rotation implements `apply`."""
from __future__ import annotations

import torch

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class Rotary(PositionEncoding):
    """Pair i of a head turns by position * theta^(-2i / rotary_dim).  rotary_dim: how many leading
    dimensions of the head rotate (default: all; fewer is partial rotary, the rest pass through).
    pairing: "halves" (d with d + rotary_dim/2, the reference's) or "neighbours" (2i with 2i+1).
    The inverse frequencies are computed in double precision and rounded to float32 once; the
    angle is the float32 product of position and inverse frequency, as in the reference."""

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = 0, pairing: str = "halves"):
        self.head_dim, self.theta = head_dim, float(theta)
        self.rotary_dim = int(rotary_dim) or head_dim
        if pairing not in ("halves", "neighbours"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"{self.rotary_dim} rotating dimensions of a head of {head_dim}")
        self.pairing = pairing
        self.inv_freq = None

    def bind(self, get, rt):
        self.rt = rt
        i = torch.arange(self.rotary_dim // 2, dtype=torch.float64)
        self.inv_freq = (self.theta ** (-(2.0 * i) / self.rotary_dim)).to(torch.float32).to(rt.device)

    def rotary_table(self):
        return self.inv_freq, self.rotary_dim, self.pairing == "neighbours"


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    is_identity = True

    def apply(self, x, positions):
        return None
