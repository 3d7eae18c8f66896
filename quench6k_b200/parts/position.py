"""Position encodings.  The rotary one is applied inside the kernel that prepares q and k
(rotate-half over the full head, base theta; reference: crates/cuda/kernels/flint.cu:141-149,
where theta is the literal 10000); "none" leaves q and k as they are (the reference's per-layer
rope flag, crates/engine/src/flint.rs:254,408)."""
from __future__ import annotations

from .base import PositionEncoding, register_position_encoding


@register_position_encoding("rope")
class RotaryNeoX(PositionEncoding):
    def __init__(self, head_dim: int, theta: float):
        self.head_dim, self.theta = head_dim, float(theta)

    def fused_rope_theta(self):
        return self.theta


@register_position_encoding("none")
class NoPosition(PositionEncoding):
    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def apply(self, x, positions):
        return None
