"""Chooses the matrix-product kernel for an operand dtype and shape.

float32 operands always take the CUDA-core FP32 kernel (no reduced-precision matrix mode exists on
that path).  bfloat16 operands take the tensor-core kernels where the shape allows and the
CUDA-core kernel otherwise.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops


def matmul(a: torch.Tensor, w: torch.Tensor, rt, out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    """FP32 out[r] (+)= a[r] @ w^T;  a: [M, K], w: [N, K]."""
    return ops.gemm_simt(a, w, out=out, accumulate=accumulate)


def swiglu_matmul(a: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, rt) -> torch.Tensor:
    """act[r] = silu(a[r] @ w_gate^T) * (a[r] @ w_up^T) in a's dtype."""
    return ops.gemm_simt(a, w_gate, w2=w_up)


def grouped_swiglu(a: torch.Tensor, row_token: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, groups, pairs: int, rt):
    """act[row] = SwiGLU of a[row_token[row]] with the weights of the row's group; [pairs, I]."""
    return ops.gemm_simt(a, w_gate, w2=w_up, a_rows=row_token, groups=groups, rows=pairs)


def grouped_matmul(a: torch.Tensor, w: torch.Tensor, groups, pairs: int, rt) -> torch.Tensor:
    """FP32 y[row] = a[row] @ w_g^T with the weights of the row's group; [pairs, N]."""
    return ops.gemm_simt(a, w, groups=groups, rows=pairs)


def group_tiles(offsets: torch.Tensor, pairs: int, rt):
    return ops.tile_list(offsets, pairs, ops.simt_tile_rows())
