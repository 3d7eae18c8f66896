"""Grouped-query self-attention over the paged cache, with optional per-head QK-norm, learned
sinks and a sliding window (reference: crates/engine/src/flint.rs:815-913 for the order of
operations, crates/cuda/kernels/flint.cu:125-173 and :211-561 for the arithmetic)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .. import ops
from ..spec import PartSpec, TensorSpec
from . import linear
from .base import (POSITION_ENCODINGS, CacheRequest, Mixer, make_part, register_mixer, to_f32, to_operand)


@register_mixer("attention")
class Attention(Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, eps: float,
                 pos: PartSpec, window: Optional[int] = None, sinks: bool = False, qk_norm: bool = False,
                 norm_init: str = "ones", sink_std: float = 1.0):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim}: the attention kernels take multiples of 16 up to 256")
        self.D, self.Hq, self.Hkv, self.hd = hidden_size, num_heads, num_kv_heads, head_dim
        self.eps, self.window, self.has_sinks, self.qk_norm = float(eps), window, sinks, qk_norm
        self.norm_init, self.sink_std = norm_init, sink_std
        self.pos = make_part(POSITION_ENCODINGS, "position encoding", pos)
        self.scale = 1.0 / math.sqrt(head_dim)

    def tensors(self):
        D, Hq, Hkv, hd = self.D, self.Hq, self.Hkv, self.hd
        out = [TensorSpec("q_proj.weight", (Hq * hd, D)), TensorSpec("k_proj.weight", (Hkv * hd, D)),
               TensorSpec("v_proj.weight", (Hkv * hd, D)), TensorSpec("o_proj.weight", (D, Hq * hd))]
        if self.qk_norm:
            init = ("ones",) if self.norm_init == "ones" else ("ones_plus", 0.1)
            out += [TensorSpec("q_norm.weight", (hd,), "f32", init), TensorSpec("k_norm.weight", (hd,), "f32", init)]
        if self.has_sinks:
            out.append(TensorSpec("sinks", (Hq,), "f32", ("normal", self.sink_std)))
        out += [TensorSpec("position." + t.name, t.shape, t.role, t.init) for t in self.pos.tensors()]
        return out

    def bind(self, get, rt):
        self.rt = rt
        # q, k and v rows stacked so one product yields [q | k | v] per token: each piece is copied into its place
        # on the device as it arrives, so that no two copies of the three are held at once
        nq, nk = self.Hq * self.hd, self.Hkv * self.hd
        self.w_qkv = torch.empty((nq + 2 * nk, self.D), dtype=rt.dtype, device=rt.device)
        for name, lo, hi in (("q_proj.weight", 0, nq), ("k_proj.weight", nq, nq + nk), ("v_proj.weight", nq + nk, nq + 2 * nk)):
            self.w_qkv[lo:hi].copy_(get(name))
        self.w_q = self.w_qkv[:nq]
        self.w_o = to_operand(get("o_proj.weight"), rt)
        self.q_norm = to_f32(get("q_norm.weight"), rt) if self.qk_norm else None
        self.k_norm = to_f32(get("k_norm.weight"), rt) if self.qk_norm else None
        self.sinks = to_f32(get("sinks"), rt) if self.has_sinks else None
        self.pos.bind(lambda n: get("position." + n), rt)

    def cache_request(self):
        if self.window is not None:
            return CacheRequest("sliding", int(self.window), self.Hkv, self.hd)
        return CacheRequest("full", None, self.Hkv, self.hd)

    def forward(self, xn, ctx, cache, state, out):
        rt = self.rt
        write = cache.write
        # which attention kernels this step takes, and the plan of the key splits, before anything of the layer is
        # launched: the kernel that splits the keys reads its plan while the kernel before it still runs
        ops.current_tag = "attention.plan"
        how = self._choose(cache, ctx)
        rotary = self.pos.rotary_table()
        fused_pos = rotary is not None or self.pos.is_identity
        # a step of a few tokens per request: the kernel that splits the keys normalises and rotates q itself and makes
        # the new keys and values (one launch less)
        in_attention = (self.prepare_in_attention and how[0] == "split" and fused_pos and
                        ops.attention_mma_prepares(self.hd, self.Hq // self.Hkv, how[1][0], rotary[1] if rotary else 0, bool(rotary and rotary[2])))
        # FP32 [T, (Hq + 2 Hkv) hd] or [T, Hq hd]; for few rows possibly as split-K partials, which the next kernel sums
        ops.current_tag = "attention.qkv"
        qkv = linear.matmul(xn, self.w_qkv if write else self.w_q, rt, partials_ok=fused_pos)
        table = ctx.block_tables[cache.group]
        if in_attention:
            ops.current_tag = "attention.keys"
            a = self._split_keys(None, cache, table, ctx, how[1],
                                 prepare={"qkv": qkv, "heads": self.Hq, "q_norm": self.q_norm, "k_norm": self.k_norm, "eps": self.eps,
                                          "rotary": rotary, "write": write})
            ops.current_tag = "attention.o"
            return linear.matmul(a, self.w_o, rt, partials_ok=True)
        ops.current_tag = "attention.prepare"
        if not fused_pos:
            qkv = self._unfused_position(qkv, ctx, write)
            q = ops.qk_prep(qkv, self.Hq, self.Hkv, self.hd, None, None, self.eps, None, ctx.positions, ctx.req_of_token,
                            table if write else None, cache.page_size, cache.k if write else None,
                            cache.v if write else None, rt.dtype)
        else:
            q = ops.qk_prep(qkv, self.Hq, self.Hkv, self.hd, self.q_norm, self.k_norm, self.eps, rotary, ctx.positions,
                            ctx.req_of_token, table if write else None, cache.page_size, cache.k if write else None,
                            cache.v if write else None, rt.dtype)
        ops.current_tag = "attention.keys"
        a = self._attend(q, cache, table, ctx, how)
        # the block adds it into the stream inside its next norm (which also sums split-K partials)
        ops.current_tag = "attention.o"
        return linear.matmul(a, self.w_o, rt, partials_ok=True)

    prepare_in_attention = True   # the kernel that splits the keys makes q and the new keys itself where it can (else qk_prep does)
    tc_min_fill = 0.5             # the tcgen05 prompt kernel runs when its CTAs (two tiles each) cover at least this share of the SMs

    def _choose(self, cache, ctx):
        """("generic",) | ("split", plan args) | ("tc", tile pairs, plan args of the short requests or None): the tensor-core
        kernels for bfloat16 where they cover the head and group size, else the generic one.  The plans are made here."""
        rt, G = self.rt, self.Hq // self.Hkv
        rows = 0 if rt.is_fp32 or not rt.tensor_cores else ops.attention_mma_tile_rows(self.hd, G, ctx.max_q_len)
        if not rows:
            return ("generic",)
        if rows > 16 and ops.attention_tc_supported(self.hd, G, cache.page_size):
            tile = ops.attention_tc_tile_tokens(G)
            # beside prompt portions, requests with a few tokens (decoded tokens, the stub of a prompt) go to the kernel
            # that splits the keys over CTAs: as a tile of their own they would walk their whole context in one CTA
            cut = tile // 2 if ctx.R > 1 else 0
            tok0, ntok, n_pairs = ctx.query_tile_pairs(tile, zigzag=False, more_than=cut)
            if n_pairs * self.Hkv >= self.tc_min_fill * self._sm_count():
                # prompt portions with enough tiles (two to a CTA) to fill that share of the SMs: both products on tcgen05, no key splits
                count, _, _, most, _ = ctx.short_requests(cut)
                short = self._plan(ctx, ops.attention_mma_tile_rows(self.hd, G, most), cut) if count else None
                return ("tc", (tok0, ntok), short)
        return ("split", self._plan(ctx, rows, None))

    def _plan(self, ctx, rows, at_most):
        """The tiles and the plan of the key splits for the mma.sync kernel over all requests of the step, or over those
        with at most `at_most` tokens.  The keys are split over one wave of resident CTAs, and no further (a second,
        partly filled wave would cost as much as a full one); the plan is made on the device, once per step for all
        layers with this window."""
        tokens = rows // (self.Hq // self.Hkv)
        tok0, ntok, n_tiles = ctx.query_tiles(tokens, at_most)
        key = ("attention_plan", tokens, at_most, self.window, self.Hkv)
        fresh = key not in ctx.made
        if fresh:                                   # the first layer of this pass with these tiles and this window
            ctx.plans[key] = ops.attention_plan(ctx.positions, ctx.req_of_token, tok0, ntok, self.window,
                                                ops.attention_mma_resident_ctas(self.hd, rows) // self.Hkv, min_per=2,
                                                into=ctx.plans.get(key))
            ctx.made.add(key)
        return rows, tok0, ntok, ctx.plans[key], fresh

    def _attend(self, q, cache, table, ctx, how):
        if how[0] == "generic":
            return ops.attention_generic(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, self.window, self.sinks, self.scale)
        if how[0] == "tc":
            (tok0, ntok), short = how[1], how[2]
            out = ops.attention_tc(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, tok0, ntok, self.window,
                                   self.sinks, scale=self.scale)
            return out if short is None else self._split_keys(q, cache, table, ctx, short, out)
        return self._split_keys(q, cache, table, ctx, how[1])

    def _split_keys(self, q, cache, table, ctx, planned, out=None, prepare=None):
        rows, tok0, ntok, plan, fresh = planned
        # The plan was made before this layer's first launch.  With q from qk_prep, the kernel before this one is that
        # one (or, beside prompt portions, the tcgen05 attention), which itself waited for everything before it: the plan
        # is complete when this kernel starts.  When this kernel prepares q itself, the kernel before it is the q/k/v
        # product, which may itself have started before the one before it ended: then only a plan of an earlier layer
        # is surely complete.
        return ops.attention_mma(q, cache.k, cache.v, table, ctx.req_of_token, ctx.positions, tok0, ntok, rows, self.window,
                                 self.sinks, scale=self.scale, out=out, plan=plan, plan_is_old=prepare is None or not fresh,
                                 prepare=prepare)

    def _sm_count(self) -> int:
        if "_sms" not in self.__dict__:
            self._sms = torch.cuda.get_device_properties(self.rt.device).multi_processor_count
        return self._sms

    def _unfused_position(self, qkv, ctx, write):
        """QK-norm, then a position encoding that is no rotation of pairs (its own `apply`), on FP32 q and k."""
        T = qkv.shape[0]
        nq, nk = self.Hq * self.hd, self.Hkv * self.hd
        q = qkv[:, :nq].reshape(T * self.Hq, self.hd).contiguous()
        if self.qk_norm:
            q = ops.rmsnorm(q, self.q_norm, self.eps, torch.float32)
        q = q.view(T, self.Hq, self.hd)
        self.pos.apply(q, ctx.positions)
        parts = [q.reshape(T, nq)]
        if write:
            k = qkv[:, nq:nq + nk].reshape(T * self.Hkv, self.hd).contiguous()
            if self.qk_norm:
                k = ops.rmsnorm(k, self.k_norm, self.eps, torch.float32)
            k = k.view(T, self.Hkv, self.hd)
            self.pos.apply(k, ctx.positions)
            parts += [k.reshape(T, nk), qkv[:, nq + nk:]]
        return torch.cat(parts, dim=1).contiguous()
