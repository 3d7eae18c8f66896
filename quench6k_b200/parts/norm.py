"""RMSNorm with a plain weight: out = x * rsqrt(mean(x^2) + eps) * w, computed in FP32
(reference: crates/cuda/kernels/flint.cu:97-122)."""
from __future__ import annotations

from .. import ops
from ..spec import TensorSpec
from .base import Norm, WeightedRows, register_norm, to_f32


@register_norm("rmsnorm")
class RMSNorm(Norm):
    graph_safe = True

    def __init__(self, size: int, eps: float, init: str = "ones"):
        self.size, self.eps, self.init = size, float(eps), init

    def tensors(self):
        init = ("ones",) if self.init == "ones" else ("ones_plus", 0.1)
        return [TensorSpec("weight", (self.size,), "f32", init)]

    def bind(self, get, rt):
        self.rt = rt
        self.weight = to_f32(get("weight"), rt)

    fuses_weighted_rows = True

    def forward(self, h, rows=None, add=None):
        if isinstance(add, WeightedRows):
            return ops.rmsnorm(h, self.weight, self.eps, self.rt.dtype, rows=rows, weighted=(add.y, add.pair_row, add.weights))
        return ops.rmsnorm(h, self.weight, self.eps, self.rt.dtype, rows=rows, add=add)
