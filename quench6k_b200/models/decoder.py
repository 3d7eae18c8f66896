"""The generic decoder: embedding, the executed list of blocks, final norm, LM head.

It is built from a spec.ModelSpec through the part registries and knows no architecture.  Tensor
names: `<embed_name>`, `<layer prefix>{input_layernorm,post_attention_layernorm}.*`,
`<layer prefix>self_attn.*` (the mixer's tensors), `<layer prefix>mlp.*` (the feed-forward's),
`<final_norm_prefix>*`, `<head_name>`.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .. import ops
from ..parts import linear
from ..parts.base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, CacheRequest, LayerCache, Runtime, make_part,
                          to_operand)
from ..spec import ModelSpec, TensorSpec

_SUB = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.", "ffn": "mlp."}


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        D = spec.hidden_size
        self.blocks = []
        for ls in spec.layers:
            if ls.block not in BLOCKS:
                raise KeyError(f"unknown block arrangement {ls.block!r}; registered: {', '.join(sorted(BLOCKS))}")
            norm1 = make_part(NORMS, "norm", ls.norm, size=D)
            norm2 = make_part(NORMS, "norm", ls.norm, size=D)
            mixer = make_part(MIXERS, "mixer", ls.mixer, hidden_size=D)
            ffn = make_part(FEED_FORWARDS, "feed-forward", ls.ffn, hidden_size=D)
            self.blocks.append(BLOCKS[ls.block](norm1, mixer, norm2, ffn))
        self.final_norm = make_part(NORMS, "norm", spec.final_norm, size=D)
        self.order = list(spec.order)
        self.kv_source = list(spec.kv_source)
        if len(self.kv_source) != len(self.order):
            raise ValueError("kv_source and order differ in length")
        self.rt: Optional[Runtime] = None

    # ------------------------------------------------------------------ declaration
    def tensors(self) -> List[TensorSpec]:
        s = self.spec
        out = [TensorSpec(s.embed_name, (s.vocab_size, s.hidden_size))]
        for ls, b in zip(s.layers, self.blocks):
            for sub, part in (("norm1", b.norm1), ("mixer", b.mixer), ("norm2", b.norm2), ("ffn", b.ffn)):
                out += [TensorSpec(ls.prefix + _SUB[sub] + t.name, t.shape, t.role, t.init) for t in part.tensors()]
        out += [TensorSpec(s.final_norm_prefix + t.name, t.shape, t.role, t.init) for t in self.final_norm.tensors()]
        if s.head_name is not None:
            out.append(TensorSpec(s.head_name, (s.vocab_size, s.hidden_size)))
        return out

    def cache_requests(self) -> List[Optional[CacheRequest]]:
        """Per executed position: the cache its mixer needs (None for positions that borrow one
        or whose mixer keeps no keys)."""
        out = []
        for p, i in enumerate(self.order):
            out.append(None if self.kv_source[p] is not None else self.blocks[i].mixer.cache_request())
        return out

    def state_shapes(self):
        """Per executed position: the shape of its mixer's fixed-size per-request state, or None."""
        return [self.blocks[i].mixer.state_shape() for i in self.order]

    def graph_safe(self) -> bool:
        parts = [self.final_norm]
        for b in self.blocks:
            parts += [b.norm1, b.mixer, b.norm2, b.ffn]
        return all(getattr(x, "graph_safe", False) for x in parts)

    # ------------------------------------------------------------------ weights
    def bind(self, get: Callable[[str], torch.Tensor], rt: Runtime) -> None:
        s = self.spec
        self.rt = rt
        self.embed = to_operand(get(s.embed_name), rt)
        for ls, b in zip(s.layers, self.blocks):
            for sub, part in (("norm1", b.norm1), ("mixer", b.mixer), ("norm2", b.norm2), ("ffn", b.ffn)):
                pre = ls.prefix + _SUB[sub]
                part.bind(lambda n, pre=pre: get(pre + n), rt)
        self.final_norm.bind(lambda n: get(s.final_norm_prefix + n), rt)
        self.head = self.embed if s.head_name is None else to_operand(get(s.head_name), rt)

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, caches: List[Optional[LayerCache]], states: List[Optional[torch.Tensor]]) -> Optional[torch.Tensor]:
        """Runs the tokens of `ctx` through the executed layers; returns FP32 logits
        [len(ctx.logit_rows), vocab] or None when no row is wanted."""
        ops.current_tag = "embedding"
        h = ops.embed(ctx.token_ids, self.embed, fed=ctx.fed)
        pending = None                      # an add into h that a block has left to the next norm
        for p, i in enumerate(self.order):
            ctx.position = p
            pending = self.blocks[i].forward(h, ctx, caches[p], states[p], pending)
        if ctx.n_logit_rows == 0:
            return None
        if pending is not None and not self.final_norm.fuses_weighted_rows:
            pending.apply(h)
            pending = None
        ops.current_tag = "norm.final"
        xn = self.final_norm.forward(h, rows=ctx.logit_rows, add=pending)
        ops.current_tag = "lm_head"
        return linear.matmul(xn, self.head, self.rt)
