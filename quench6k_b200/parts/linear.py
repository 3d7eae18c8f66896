"""Chooses the matrix-product kernel for an operand dtype and shape.

float32 operands always take the CUDA-core FP32 kernel (no reduced-precision matrix mode exists on
that path).  bfloat16 operands take the tcgen05 tensor-core kernel where the shape allows (K a
multiple of 8, rows starting on 16 bytes), the matrix-vector kernel or the mma.sync kernel for few tokens where the
library prefers them (steps of at most 16 tokens), and the CUDA-core kernel otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


def _tc(a: torch.Tensor, w: torch.Tensor, rt) -> bool:
    return rt.tensor_cores and not rt.is_fp32 and ops.tc_supported(a, w)


def matmul(a: torch.Tensor, w: torch.Tensor, rt, out: Optional[torch.Tensor] = None, accumulate: bool = False,
           partials_ok: bool = False) -> torch.Tensor:
    """FP32 out[r] (+)= a[r] @ w^T;  a: [M, K], w: [N, K].  partials_ok: the caller's next kernel
    can sum split-K partial products itself, so the result may come as [slices, M, N] (a view of
    the device's scratch buffer: consume it before the next kernel that uses scratch)."""
    if _tc(a, w, rt):
        if ops.gemv_preferred(a.shape[0], w.shape[0], w.shape[1]):       # a token or two: the matrix-vector kernel
            return ops.gemv(a, w, out=out, accumulate=accumulate)
        if ops.gemm_skinny_preferred(a.shape[0], w.shape[0], w.shape[1]):  # up to 16 tokens against many rows: mma.sync, K not split over blocks
            return ops.gemm_skinny(a, w, out=out, accumulate=accumulate)
        if partials_ok and out is None and not accumulate and w.shape[0] % 4 == 0:
            slices = ops.gemm_skinny_slices(a.shape[0], w.shape[0], w.shape[1])
            if slices:                                                   # a few tokens against few rows: the same kernel, K in slices
                return ops.gemm_skinny(a, w, slices=slices)
            return ops.gemm_tc(a, w, keep_partials=True)
        return ops.gemm_tc(a, w, out=out, accumulate=accumulate)
    return ops.gemm_simt(a, w, out=out, accumulate=accumulate)


def swiglu_matmul(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, rt) -> torch.Tensor:
    """act[r] = silu(a[r] @ w_gate^T) * (a[r] @ w_up^T) in a's dtype."""
    if _tc(a, w_gate, rt):
        if ops.gemv_preferred(a.shape[0], w_gate.shape[0], w_gate.shape[1]):
            return ops.gemv(a, w_gate, w2=w_up)
        if ops.gemm_skinny_preferred(a.shape[0], w_gate.shape[0], w_gate.shape[1]):
            return ops.gemm_skinny(a, w_gate, w2=w_up)
        return ops.gemm_tc(a, w_gate, w2=w_up)
    return ops.gemm_simt(a, w_gate, w2=w_up)


class GroupPlan:
    """The permutation of a step's (token, slot) pairs by expert and the row tiles of the experts'
    groups, for whichever kernel runs them; on the tensor-core path also the gathered input rows."""

    def __init__(self, a: torch.Tensor, sel_e: torch.Tensor, num_groups: int, rt, tc: bool):
        self.pairs, self.tc, self.xs = sel_e.numel(), tc, None
        if tc:
            avg = max(1, self.pairs // max(1, num_groups))
            want = avg + avg // 2
            self.bt_dual = ops.tc_token_tile(want, True)
            self.bt = self.bt_dual
            # permutation, tile list and the gathered input rows in three launches (the last one, a block per pair,
            # finishes the pair's rank and copies its row)
            if a.shape[1] * a.element_size() % 16 == 0:
                self.offsets, self.pair_row, self.row_token, self.tiles, self.xs = ops.moe_plan(sel_e, num_groups, self.bt, a)
            else:
                self.offsets, self.pair_row, self.row_token, self.tiles = ops.moe_plan(sel_e, num_groups, self.bt)
                self.xs = ops.gather_rows(a, self.row_token)
        else:
            self.offsets, self.pair_row, self.row_token, self.tiles = ops.moe_plan(sel_e, num_groups, ops.simt_tile_rows())


def group_plan(a: torch.Tensor, w: torch.Tensor, sel_e: torch.Tensor, rt) -> GroupPlan:
    return GroupPlan(a, sel_e, w.shape[0], rt, _tc(a, w, rt) and a.is_contiguous())


def grouped_swiglu(a: torch.Tensor, plan: GroupPlan, w_gate: torch.Tensor, w_up: torch.Tensor, rt) -> torch.Tensor:
    """act[row] = SwiGLU of a[row_token[row]] with the weights of the row's group; [pairs, I]."""
    if plan.tc:
        return ops.gemm_tc(plan.xs, w_gate, w2=w_up, groups=plan.tiles, bt=plan.bt, rows=plan.pairs)
    return ops.gemm_simt(a, w_gate, w2=w_up, a_rows=plan.row_token, groups=plan.tiles, rows=plan.pairs)


def grouped_matmul(a: torch.Tensor, plan: GroupPlan, w: torch.Tensor, rt) -> torch.Tensor:
    """FP32 y[row] = a[row] @ w_g^T with the weights of the row's group; [pairs, N]."""
    if plan.tc and ops.tc_supported(a, w):
        return ops.gemm_tc(a, w, groups=plan.tiles, bt=plan.bt, rows=plan.pairs)
    if plan.tc:
        return ops.gemm_simt(a, w, groups=ops.tile_list(plan.tiles[0], plan.pairs, ops.simt_tile_rows()), rows=plan.pairs)
    return ops.gemm_simt(a, w, groups=plan.tiles, rows=plan.pairs)
