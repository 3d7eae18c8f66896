"""Arrangement of the parts in a block.  "prenorm": h += mixer(norm1(h)); h += ffn(norm2(h)),
the residual stream h staying FP32 (reference: crates/engine/src/flint.rs:815-1075, :617)."""
from __future__ import annotations

from .. import ops
from .base import Block, register_block


@register_block("prenorm")
class PreNormBlock(Block):
    def forward(self, h, ctx, cache, state, pending=None):
        if pending is not None and not self.norm1.fuses_weighted_rows:
            pending.apply(h)
            pending = None
        ops.current_tag = "norm.mixer"
        xn = self.norm1.forward(h, add=pending)         # the add the block before left is made here
        delta = self.mixer.forward(xn, ctx, cache, state, h)
        ops.current_tag = "norm.ffn"
        xn = self.norm2.forward(h, add=delta)           # h += delta inside the norm when the mixer returned its result
        if self.ffn.defers_add:
            return self.ffn.forward(xn, ctx, h, defer=True)
        self.ffn.forward(xn, ctx, h)
        return None
