"""Greedy and sampled token choice.

As in the reference (crates/cli/src/flint.rs:293-431), the device delivers, per logits row, either
the argmax (greedy without penalties: ties to the lower id) or an exact pool of the top candidates
(at most 256, or top_k if smaller; at least 64 when penalties may reorder them); the host applies
presence and repetition penalties, sorts by (logit descending, id ascending), and for sampled
requests computes p_i = exp((l_i - l_0) / temperature) in double precision, drops p_i < min_p,
keeps the shortest prefix whose mass reaches top_p and inverts the CDF with u * total.

u is the next value of a splitmix64 stream that starts at the request's seed
(crates/cli/src/flint.rs:318-325), one value per sampled token of that request, so a request's
tokens do not depend on what else was in its batches.
"""
from __future__ import annotations

import math
from typing import List, Sequence

import numpy as np
import torch

from .. import ops
from .params import SamplingParams

POOL = 256
_M64 = (1 << 64) - 1


class SplitMix64:
    def __init__(self, seed: int):
        self.state = seed & _M64

    def uniform(self) -> float:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _M64
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
        z ^= z >> 31
        return (z >> 11) / float(1 << 53)


def pool_size(p: SamplingParams, vocab: int) -> int:
    if p.greedy and not p.penalized:
        return 1
    if p.top_k == 0:
        n = POOL
    else:
        n = min(max(p.top_k, 64 if p.penalized else 1), POOL)
    return min(n, vocab)


def pick_from_pool(ids: Sequence[int], vals: Sequence[float], p: SamplingParams, generated: Sequence[int], rng: SplitMix64) -> int:
    """One token from a candidate pool (any order) under the request's options."""
    vals = np.asarray(vals, dtype=np.float32).copy()
    ids = np.asarray(ids, dtype=np.int64)
    if p.penalized and len(generated):
        seen = np.isin(ids, np.asarray(list(set(generated)), dtype=np.int64))
        v = vals[seen] - np.float32(p.presence_penalty)
        v = np.where(v > 0, v / np.float32(p.repetition_penalty), v * np.float32(p.repetition_penalty)).astype(np.float32)
        vals[seen] = v
    order = np.lexsort((ids, -vals.astype(np.float64)))        # by logit descending, then id ascending
    if p.greedy:
        return int(ids[order[0]])
    keep = len(order) if p.top_k == 0 else min(p.top_k, len(order))
    order = order[:keep]
    top = vals[order[0]]
    scaled = ((vals[order] - top) / np.float32(p.temperature)).astype(np.float32)
    probs = [math.exp(float(s)) for s in scaled]
    min_p, top_p = float(np.float32(p.min_p)), float(np.float32(p.top_p))      # the options are 32-bit values
    if min_p > 0.0:
        probs = [q if q >= min_p else 0.0 for q in probs]
    total = 0.0
    for q in probs:                       # a plain running sum, as the reference's
        total += q
    cut = len(probs)
    if top_p < 1.0:
        acc = 0.0
        for i, q in enumerate(probs):
            acc += q / total
            if acc >= top_p:
                cut = i + 1
                break
    total = 0.0
    for q in probs[:cut]:
        total += q
    r = rng.uniform() * total
    for i in range(cut):
        r -= probs[i]
        if r <= 0.0:
            return int(ids[order[i]])
    return int(ids[order[cut - 1]])


def pick_rows_native(ids: np.ndarray, vals: np.ndarray, sizes: Sequence[int], params: Sequence[SamplingParams],
                     generated: Sequence[Sequence[int]], rngs: Sequence[SplitMix64]) -> List[int]:
    """pick_from_pool for every row with sizes[row] > 0 in one call of the C++ host library
    (csrc/host/host.cpp, q6k_sample_rows); ids / vals: int32 / float32 [rows, pool].  A row's
    random stream advances exactly when pick_from_pool would advance it."""
    from ..cache.native import host_lib, raise_for
    import ctypes
    rows, stride = ids.shape
    f32 = lambda xs: np.ascontiguousarray(xs, dtype=np.float32)
    sizes_a = np.ascontiguousarray(sizes, dtype=np.int32)
    u = np.zeros(rows, dtype=np.float64)
    starts = np.zeros(rows + 1, dtype=np.int64)
    gen: List[int] = []
    for i, p in enumerate(params):
        if sizes_a[i] > 0:
            if p.penalized:
                gen.extend(generated[i])
            if not p.greedy:
                u[i] = rngs[i].uniform()
        starts[i + 1] = len(gen)
    gen_a = np.ascontiguousarray(gen if gen else [0], dtype=np.int32)
    out = np.zeros(rows, dtype=np.int32)
    ptr = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t))
    cols = [f32([getattr(p, name) for p in params]) for name in ("temperature", "top_p", "min_p", "presence_penalty", "repetition_penalty")]
    top_k = np.ascontiguousarray([p.top_k for p in params], dtype=np.int32)
    ids, vals = np.ascontiguousarray(ids, dtype=np.int32), np.ascontiguousarray(vals, dtype=np.float32)
    raise_for(host_lib().q6k_sample_rows(rows, stride, ptr(ids, ctypes.c_int32), ptr(vals, ctypes.c_float), ptr(sizes_a, ctypes.c_int32),
                                         ptr(cols[0], ctypes.c_float), ptr(top_k, ctypes.c_int32), ptr(cols[1], ctypes.c_float),
                                         ptr(cols[2], ctypes.c_float), ptr(cols[3], ctypes.c_float), ptr(cols[4], ctypes.c_float),
                                         ptr(gen_a, ctypes.c_int32), ptr(starts, ctypes.c_int64), ptr(u, ctypes.c_double),
                                         ptr(out, ctypes.c_int32)))
    return out.tolist()


ROW_RECORD = np.dtype([("size", np.int32), ("top_k", np.int32), ("temperature", np.float32), ("top_p", np.float32),
                       ("min_p", np.float32), ("pad", np.int32), ("u", np.float64)])     # 32 bytes, as ops.sample_pool reads them


def device_rows(params: Sequence[SamplingParams], rngs: Sequence[SplitMix64], vocab: int, into: np.ndarray) -> int:
    """Fill `into` (ROW_RECORD per row) for ops.sample_pool and return the pool size to fetch.
    None of the requests may use penalties (those are applied on the host).  A row's random stream
    advances exactly when the host sampler would advance it."""
    k = 1
    for i, p in enumerate(params):
        if p.penalized:
            raise ValueError("penalties are applied by the host sampler")
        size = pool_size(p, vocab)
        k = max(k, size)
        into[i] = (size, p.top_k, p.temperature, p.top_p, p.min_p, 0, 0.0 if p.greedy else rngs[i].uniform())
    return k


class Sampler:
    """Chooses the next token of each row of a logits block [rows, vocab] (device, FP32).  The
    choice from the pools runs in the C++ host library unless Q6K_HOST=python asks for the
    Python twin (pick_from_pool)."""

    def __init__(self):
        import os
        self.native = os.environ.get("Q6K_HOST", "").lower() != "python"

    def sample(self, logits: torch.Tensor, params: List[SamplingParams], generated: List[Sequence[int]],
               rngs: List[SplitMix64]) -> List[int]:
        rows, vocab = logits.shape
        sizes = [pool_size(p, vocab) for p in params]
        out: List[int] = [0] * rows
        if all(s == 1 for s in sizes):
            picked = ops.argmax(logits).tolist()
            return [int(t) for t in picked]
        greedy_rows = [i for i, s in enumerate(sizes) if s == 1]
        if greedy_rows:
            picked = ops.argmax(logits).tolist()
            for i in greedy_rows:
                out[i] = int(picked[i])
        k = max(sizes)
        ids, vals = ops.topk_pool(logits, k)
        ids, vals = ids.cpu().numpy(), vals.cpu().numpy()
        if self.native:
            chosen = pick_rows_native(ids, vals, [0 if s == 1 else s for s in sizes], params, generated, rngs)
            for i, s in enumerate(sizes):
                if s != 1:
                    out[i] = int(chosen[i])
            return out
        for i, s in enumerate(sizes):
            if s == 1:
                continue
            out[i] = pick_from_pool(ids[i, :s], vals[i, :s], params[i], generated[i], rngs[i])
        return out
