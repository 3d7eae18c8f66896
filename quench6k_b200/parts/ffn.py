"""Feed-forward parts: a dense SwiGLU MLP and a routed mixture of SwiGLU experts with an optional
ungated shared expert.

Reference: crates/engine/src/flint.rs:915-1075 (order of operations),
crates/cuda/kernels/flint.cu:829-868 (sigmoid routing), crates/cuda/kernels/moe.cu:19-71 (softmax
routing), flint.cu:1163-1239 (permutation, SwiGLU, combine in slot order).  The reference runs
its dense MLP and its shared expert as extra expert slots with weight 1; here they are the dense
part, added after the routed sum.
"""
from __future__ import annotations


from .. import ops
from ..spec import TensorSpec
from . import linear
from .base import FeedForward, WeightedRows, register_feed_forward, to_operand


@register_feed_forward("dense")
class DenseSwiGLU(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, intermediate_size: int):
        self.D, self.I = hidden_size, intermediate_size

    def tensors(self):
        return [TensorSpec("gate_proj.weight", (self.I, self.D)), TensorSpec("up_proj.weight", (self.I, self.D)),
                TensorSpec("down_proj.weight", (self.D, self.I))]

    def bind(self, get, rt):
        self.rt = rt
        self.w_gate, self.w_up = to_operand(get("gate_proj.weight"), rt), to_operand(get("up_proj.weight"), rt)
        self.w_down = to_operand(get("down_proj.weight"), rt)

    def forward(self, xn, ctx, out):
        ops.current_tag = "dense.gate_up"
        act = linear.swiglu_matmul(xn, self.w_gate, self.w_up, self.rt)
        ops.current_tag = "dense.down"
        linear.matmul(act, self.w_down, self.rt, out=out, accumulate=True)


@register_feed_forward("moe")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, intermediate_size: int, scoring: str = "softmax",
                 renormalize: bool = True, shared_intermediate_size: int = 0):
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unknown router scoring {scoring!r}")
        if not 0 < top_k <= num_experts:
            raise ValueError(f"top_k {top_k} outside 1..{num_experts}")
        self.D, self.E, self.k, self.I = hidden_size, num_experts, top_k, intermediate_size
        self.scoring, self.renorm = scoring, bool(renormalize)
        self.shared = DenseSwiGLU(hidden_size, shared_intermediate_size) if shared_intermediate_size > 0 else None
        self.routing_tap = None               # a parts.base.Tap: every forward records each row's chosen experts [T, k]
                                              # ("experts") and its router logits [T, E] ("router_logits") there

    def tensors(self):
        E, I, D = self.E, self.I, self.D
        out = [TensorSpec("gate.weight", (E, D)), TensorSpec("experts.gate_proj.weight", (E, I, D)),
               TensorSpec("experts.up_proj.weight", (E, I, D)), TensorSpec("experts.down_proj.weight", (E, D, I))]
        if self.shared is not None:
            out += [TensorSpec("shared_experts." + t.name, t.shape, t.role, t.init) for t in self.shared.tensors()]
        return out

    def bind(self, get, rt):
        self.rt = rt
        self.w_router = to_operand(get("gate.weight"), rt)
        self.w_gate = to_operand(get("experts.gate_proj.weight"), rt)
        self.w_up = to_operand(get("experts.up_proj.weight"), rt)
        self.w_down = to_operand(get("experts.down_proj.weight"), rt)
        if self.shared is not None:
            self.shared.bind(lambda n: get("shared_experts." + n), rt)

    defers_add = True

    def _tap(self, ctx, sel_e, logits):
        if logits.dim() == 3:                 # split-K slices of the router product: summed in order, as the routing kernel sums them
            total = logits[0].clone()
            for s in range(1, logits.shape[0]):
                total += logits[s]
            logits = total
        self.routing_tap.record("experts", ctx.position, sel_e)
        self.routing_tap.record("router_logits", ctx.position, logits)

    def forward(self, xn, ctx, out, defer=False):
        """Adds the experts' weighted results into `out`; with defer=True and no shared expert it
        returns them unsummed (WeightedRows) for the next norm to add."""
        rt = self.rt
        T = xn.shape[0]
        pairs = T * self.k
        defer = defer and self.shared is None
        if (rt.tensor_cores and not rt.is_fp32 and ops.router_small_supported(T, self.E, self.D, self.k)
                and ops.tc_supported(xn, self.w_gate) and self.I % 8 == 0):
            # a decode step: router and top-k in one launch, then one weight tile stream per
            # (token, slot) pair straight from the selection, no permutation and no gather
            ops.current_tag = "experts.router"
            sel_e, sel_w, order, logits = ops.router_small(xn, self.w_router, self.k, self.scoring, self.renorm, with_logits=True)
            if self.routing_tap is not None:
                self._tap(ctx, sel_e, logits)
            ops.current_tag = "experts.gate_up"
            if ops.gemv_preferred(T, self.I, self.D):                     # a token or two: the matrix-vector kernel per pair
                act = ops.gemv(xn, self.w_gate, w2=self.w_up, pair_expert=sel_e.view(-1), pair_div=self.k)
                ops.current_tag = "experts.down"
                y = ops.gemv(act, self.w_down, pair_expert=sel_e.view(-1), pair_div=1, pairs_are_old=True)   # the router made them, two kernels ago
            else:
                act = ops.gemm_tc_pairs(xn, self.w_gate, sel_e, self.k, w2=self.w_up, order=order)  # [pairs, I]
                ops.current_tag = "experts.down"
                y = ops.gemm_tc_pairs(act, self.w_down, sel_e, 1, order=order, pairs_are_old=True)   # FP32 [pairs, D]
            if defer:
                return WeightedRows(y, sel_w)
            ops.current_tag = "experts.combine"
            ops.combine(y, None, sel_w, out)
            if self.shared is not None:
                self.shared.forward(xn, ctx, out)
            return None
        ops.current_tag = "experts.router"
        logits = linear.matmul(xn, self.w_router, rt, partials_ok=True)    # FP32 [T, E], or split-K slices of it that route() sums
        sel_e, sel_w = ops.route(logits, self.k, self.scoring, self.renorm)
        if self.routing_tap is not None:
            self._tap(ctx, sel_e, logits)
        ops.current_tag = "experts.permute"
        plan = linear.group_plan(xn, self.w_gate, sel_e, rt)             # permutation by expert, row tiles, gathered rows
        ops.current_tag = "experts.gate_up"
        act = linear.grouped_swiglu(xn, plan, self.w_gate, self.w_up, rt)                         # [pairs, I]
        ops.current_tag = "experts.down"
        y = linear.grouped_matmul(act, plan, self.w_down, rt)                                     # FP32 [pairs, D]
        if defer:
            return WeightedRows(y, sel_w, plan.pair_row)
        ops.current_tag = "experts.combine"
        ops.combine(y, plan.pair_row, sel_w, out)
        if self.shared is not None:
            self.shared.forward(xn, ctx, out)
        return None
