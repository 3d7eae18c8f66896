"""Python faces of the hand-written CUDA kernels.

Each function checks devices, dtypes, shapes and contiguity, then calls the `extern "C"` launcher
through ctypes on the current CUDA stream.  There is no CPU path and no library fallback: on a
machine without the built extension or without a GPU these functions raise.
"""
from __future__ import annotations

import ctypes
import functools
import math
import os
from typing import Optional, Tuple

import torch

from .build import BuildError, build, library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return F32
    if dt == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 operands, not {dt}")


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream():
    """The current stream's handle (the short way where this torch has it: a launch costs the host a few microseconds)."""
    if _raw_stream is not None:
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, shape=None):
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on a CUDA device only")
    if not t.is_contiguous():
        raise KernelError(f"{name} is not contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} has shape {tuple(t.shape)}, expected {tuple(shape)}")


# kernels launched per exported function (for launch accounting in benchmarks)
_LAUNCHES = {"q6k_moe_permute": 3, "q6k_moe_plan": 3, "q6k_gemm_tc": 1, "q6k_attention_mma": 2, "q6k_argmax": 2, "q6k_gemm_tc_pairs_scratch": 0}
launch_count = 0


_functions = {}

# Where a step's time goes, without a profiler (the reference times its forward pass op by op the same way and can
# synchronise after every op: crates/engine/src/profile.rs:1-55, crates/engine/src/flint.rs:685-697).
# profile_begin() makes every launcher call stand between two CUDA events; profile_end() adds them up per (tag, launcher).
# Parts name what they are about to launch by setting ops.current_tag (a plain attribute: nothing is paid when no one
# is profiling).  Steps replayed from a CUDA graph run no Python and are not seen: profile eager steps.
# The environment variable Q6K_SYNC=op synchronises after every launcher call and raises where a kernel failed.
current_tag = ""
_profile = None
_sync_each = os.environ.get("Q6K_SYNC", "") == "op"


def profile_begin() -> None:
    global _profile
    _profile = []


def profile_end():
    """{(tag, launcher): (calls, milliseconds)} since profile_begin(), in the order of first use (synchronises)."""
    global _profile
    records, _profile = _profile or [], None
    torch.cuda.synchronize()
    out = {}
    for key, e0, e1 in records:
        calls, ms = out.get(key, (0, 0.0))
        out[key] = (calls + 1, ms + e0.elapsed_time(e1))
    return out


def _call(fn_name: str, *args):
    global launch_count
    launch_count += _LAUNCHES.get(fn_name, 1)
    fn = _functions.get(fn_name)
    if fn is None:
        fn = _functions[fn_name] = getattr(library(), fn_name)
        fn.restype = ctypes.c_int
    if _profile is not None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rc = fn(*args)
        e1.record()
        _profile.append(((current_tag, fn_name), e0, e1))
    else:
        rc = fn(*args)
    if rc != 0:
        lib = library()
        lib.q6k_last_error.restype = ctypes.c_char_p
        raise KernelError(lib.q6k_last_error().decode())
    if _sync_each:
        torch.cuda.synchronize()
        status = tc_status()
        if status:
            raise KernelError(f"{fn_name} ({current_tag}): a bounded wait ran out inside a kernel (status {status})")


_i = ctypes.c_int
_f = ctypes.c_float
_ll = ctypes.c_longlong


# --------------------------------------------------------------------------- elementwise
def embed(tokens: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, fed: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h[t] = float32(table[tokens[t]]).  With `fed` (int32 on the device), a token id -(i + 1)
    stands for fed[i]: a token the step before has sampled and the host has not read yet."""
    T = tokens.numel()
    V, D = table.shape
    _need(tokens, "tokens", torch.int32)
    _need(table, "table")
    if fed is not None:
        _need(fed, "fed", torch.int32)
    if out is None:
        out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    _need(out, "out", torch.float32, (T, D))
    _call("q6k_embed", _ptr(tokens), _ptr(table), _ptr(out), _i(T), _i(D), _i(V), _i(dtype_code(table.dtype)), _ptr(fed),
          _i(fed.numel() if fed is not None else 0), _stream())
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
            out: Optional[torch.Tensor] = None, add: Optional[torch.Tensor] = None, weighted=None) -> torch.Tensor:
    """out[r] = out_dtype(x[row] * rsqrt(mean(x[row]^2) + eps) * w); row = rows[r] if given.
    With `add` (float32, x's shape, or [splits, R, D] partial sums added in order), x += add is
    stored first: the block's residual add, fused.  With `weighted` = (y [pairs, D], pair_row [T, S]
    or None, weights [T, S]), x[t] += sum_s weights[t, s] * y[pair_row[t, s] or t*S + s] is stored
    first: the routed experts' combination (the arithmetic of `combine`)."""
    _need(x, "x", torch.float32)
    D = x.shape[-1]
    _need(w, "w", torch.float32, (D,))
    R = x.shape[0] if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if out is None:
        out = torch.empty((R, D), dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, (R, D))
    splits, stride = 1, 0
    if add is not None:
        _need(add, "add", torch.float32)
        if add.dim() == 3:                       # [splits, R, D]: partial sums, added in order
            splits, stride = add.shape[0], add.shape[1] * add.shape[2]
            if tuple(add.shape[1:]) != tuple(x.shape):
                raise KernelError("rmsnorm: the partial sums do not match x")
        elif tuple(add.shape) != tuple(x.shape):
            raise KernelError("rmsnorm: add does not match x")
    y = pair_row = pair_w = None
    S = 0
    if weighted is not None:
        y, pair_row, pair_w = weighted
        T, S = pair_w.shape
        _need(y, "weighted rows", torch.float32)
        _need(pair_w, "weights", torch.float32)
        if pair_row is not None:
            _need(pair_row, "pair_row", torch.int32)
        if T != x.shape[0] or y.shape[1] != D or y.shape[0] < T * S or (pair_row is not None and pair_row.numel() != T * S):
            raise KernelError("rmsnorm: the weighted rows do not match x")
        if not rmsnorm_fuses_weighted(D):
            combine(y, pair_row, pair_w, x)      # widths the register kernel does not take: two passes
            y = pair_row = pair_w = None
    _call("q6k_rmsnorm", _ptr(x), _ptr(add), _i(splits), _ll(stride), _ptr(rows), _ptr(w), _f(eps), _ptr(out), _i(R), _i(D),
          _i(dtype_code(out_dtype)), _ptr(y), _ptr(pair_row), _ptr(pair_w), _i(S), _stream())
    return out


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def rmsnorm_fuses_weighted(D: int) -> bool:
    lib = library()
    lib.q6k_rmsnorm_fuses_pairs.restype = ctypes.c_int
    return bool(lib.q6k_rmsnorm_fuses_pairs(_i(D)))


def combine(y: torch.Tensor, pair_row: torch.Tensor, sel_w: torch.Tensor, h: torch.Tensor) -> None:
    """h[t] += sum_s sel_w[t, s] * y[pair_row[t, s]] in slot order."""
    T, S = sel_w.shape
    D = h.shape[1]
    _need(y, "y", torch.float32)
    _need(sel_w, "sel_w", torch.float32)
    _need(h, "h", torch.float32, (T, D))
    if pair_row is not None:
        _need(pair_row, "pair_row", torch.int32)
    if y.shape[1] != D or (pair_row is not None and pair_row.numel() != T * S) or y.shape[0] < T * S:
        raise KernelError("combine: shapes disagree")
    _call("q6k_combine", _ptr(y), _ptr(pair_row), _ptr(sel_w), _i(T), _i(S), _i(D), _ptr(h), _stream())


def swiglu(gu: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """act = out_dtype(silu(gu[:, :I]) * gu[:, I:])."""
    _need(gu, "gu", torch.float32)
    rows, two_i = gu.shape
    act = torch.empty((rows, two_i // 2), dtype=out_dtype, device=gu.device)
    _call("q6k_swiglu", _ptr(gu), _ptr(act), _i(rows), _i(two_i // 2), _i(dtype_code(out_dtype)), _stream())
    return act


# --------------------------------------------------------------------------- matrix products (CUDA cores)
EPI_STORE, EPI_ADD, EPI_SWIGLU = 0, 1, 2


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
              w2: Optional[torch.Tensor] = None, a_rows: Optional[torch.Tensor] = None, groups=None,
              rows: Optional[int] = None) -> torch.Tensor:
    """out[r] (+)= a[row(r)] @ w_g^T with FP32 fused multiply-adds.

    a: [*, K]; w: [N, K] or, grouped, [G, N, K]; w2 (same shape) switches to the SwiGLU epilogue,
    whose output has a's dtype; otherwise the output is float32.  a_rows: int32 [M] gathers rows of
    a.  groups: (group_offsets [G+1], tile_group, tile_row0, num_tiles) from `tile_list`.
    """
    _need(a, "a")
    _need(w, "w", a.dtype)
    K = a.shape[1]
    grouped = w.dim() == 3
    N = w.shape[-2]
    if w.shape[-1] != K:
        raise KernelError(f"gemm: a has K={K}, w has K={w.shape[-1]}")
    if grouped and groups is None:
        raise KernelError("gemm: a grouped weight needs group offsets and a tile list")
    M = rows if rows is not None else (a_rows.numel() if a_rows is not None else a.shape[0])
    epi = EPI_SWIGLU if w2 is not None else (EPI_ADD if accumulate else EPI_STORE)
    out_dtype = a.dtype if w2 is not None else torch.float32
    if out is None:
        if accumulate:
            raise KernelError("gemm: accumulate needs an output")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _need(out, "out", out_dtype)
    if out.shape[0] < M or out.shape[1] != N:
        raise KernelError(f"gemm: out has shape {tuple(out.shape)}, needs [{M}, {N}]")
    if w2 is not None:
        _need(w2, "w2", a.dtype, w.shape)
    if a_rows is not None:
        _need(a_rows, "a_rows", torch.int32)
    stride = N * K if grouped else 0
    if grouped:
        offsets, tile_group, tile_row0, num_tiles = groups
        max_tiles = tile_group.numel()
    else:
        offsets = tile_group = tile_row0 = num_tiles = None
        max_tiles = 0
    _call("q6k_gemm_simt", _ptr(a), _i(a.stride(0)), _ptr(a_rows), _ptr(w), _ptr(w2), _ll(stride), _ptr(out), _i(out.stride(0)),
          _i(M), _i(N), _i(K), _ptr(tile_group), _ptr(tile_row0), _ptr(offsets), _ptr(num_tiles), _i(max_tiles), _i(epi),
          _i(dtype_code(a.dtype)), _stream())
    return out


def simt_tile_rows() -> int:
    lib = library()
    lib.q6k_gemm_tile_rows.restype = ctypes.c_int
    return lib.q6k_gemm_tile_rows()


def tile_list(offsets: torch.Tensor, pairs: int, bm: int):
    """(offsets, tile_group, tile_row0, num_tiles) for the groups' row tiles of bm rows."""
    _need(offsets, "offsets", torch.int32)
    G = offsets.numel() - 1
    max_tiles = pairs // bm + min(pairs, G)          # full tiles plus at most one ragged tile per non-empty group
    tile_group = torch.empty(max_tiles, dtype=torch.int32, device=offsets.device)
    tile_row0 = torch.empty(max_tiles, dtype=torch.int32, device=offsets.device)
    num_tiles = torch.empty(1, dtype=torch.int32, device=offsets.device)
    _call("q6k_tile_list", _ptr(offsets), _i(G), _i(bm), _ptr(tile_group), _ptr(tile_row0), _ptr(num_tiles), _i(max_tiles), _stream())
    return offsets, tile_group, tile_row0, num_tiles


# --------------------------------------------------------------------------- matrix products (tcgen05 tensor cores)
def gather_rows(x: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """out[r] = x[idx[r]] (rows of a multiple of 16 bytes)."""
    _need(x, "x")
    _need(idx, "idx", torch.int32)
    out = torch.empty((idx.numel(), x.shape[1]), dtype=x.dtype, device=x.device)
    _call("q6k_gather_rows", _ptr(x), _ptr(idx), _ptr(out), _i(idx.numel()), _i(x.shape[1] * x.element_size()), _stream())
    return out


def tc_supported(a: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands: bfloat16, K a multiple of 8, rows
    starting on 16 bytes."""
    return (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a.stride(0) % 8 == 0
            and a.stride(1) == 1 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def tc_token_tile(rows: int, dual: bool) -> int:
    lib = library()
    lib.q6k_tc_token_tile.restype = ctypes.c_int
    return lib.q6k_tc_token_tile(_i(rows), _i(1 if dual else 0))


def tc_status() -> int:
    """0, or the code of a bounded wait that ran out inside a tensor-core kernel (synchronises)."""
    lib = library()
    lib.q6k_tc_status.restype = ctypes.c_int
    lib.q6k_attention_status.restype = ctypes.c_int
    lib.q6k_attention_tc_status.restype = ctypes.c_int
    lib.q6k_router_status.restype = ctypes.c_int
    return lib.q6k_tc_status() or lib.q6k_attention_status() or lib.q6k_attention_tc_status() or lib.q6k_router_status()


def selftest_wait_runs_out(limit_cycles: int = 2_000_000):
    """Runs a kernel whose bounded mbarrier wait must run out (nothing ever arrives on its barrier):
    (status, cycles waited); status 1 is the run-out the kernel has to record.  The product kernels'
    waits go through the same routine with a limit of about two seconds."""
    status, waited = ctypes.c_int(-1), ctypes.c_longlong()
    _call("q6k_selftest_wait_runs_out", _ll(limit_cycles), ctypes.byref(status), ctypes.byref(waited), _stream())
    return status.value, waited.value


_workspaces = {}
_retired = []                             # outgrown scratch stays allocated: recorded CUDA graphs still point at it


def _workspace(nbytes: int, device, which: str = "") -> torch.Tensor:
    key = str(device) + which             # one scratch buffer per device and kind: the engine runs on one stream
    ws = _workspaces.get(key)
    if ws is None or ws.numel() * 4 < nbytes:
        if ws is not None:
            _retired.append(ws)
        ws = torch.empty(max(nbytes // 4, 1 << 20), dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
            w2: Optional[torch.Tensor] = None, groups=None, bt: int = 0, rows: Optional[int] = None,
            keep_partials: bool = False) -> torch.Tensor:
    """The same contract as gemm_simt without the row gather, on tcgen05 tensor cores: bfloat16
    operands, FP32 accumulation in tensor memory.  Grouped calls pass the tile list made for
    token tile `bt` (tile_list(offsets, pairs, bt)).  keep_partials (dense, plain store): when the
    kernel slices K over CTAs the result is the FP32 partial products [slices, M, N], a view of the
    device's scratch buffer that stays valid until the next kernel that uses scratch; the consumer
    sums the slices in order."""
    if not tc_supported(a, w):
        raise KernelError("gemm_tc: operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    K = a.shape[1]
    grouped = w.dim() == 3
    G = w.shape[0] if grouped else 1
    N = w.shape[-2]
    if w.shape[-1] != K:
        raise KernelError(f"gemm_tc: a has K={K}, w has K={w.shape[-1]}")
    if grouped and groups is None:
        raise KernelError("gemm_tc: a grouped weight needs group offsets and a tile list")
    M = rows if rows is not None else a.shape[0]
    epi = EPI_SWIGLU if w2 is not None else (EPI_ADD if accumulate else EPI_STORE)
    out_dtype = torch.bfloat16 if w2 is not None else torch.float32
    lib = library()
    splits = 1
    if keep_partials:
        if grouped or w2 is not None or accumulate or out is not None:
            raise KernelError("gemm_tc: partial products are kept only for a dense product that is stored")
        lib.q6k_gemm_tc_splits.restype = ctypes.c_int
        splits = lib.q6k_gemm_tc_splits(_i(M), _i(N), _i(K))
        keep_partials = splits > 1
    if out is None:
        if accumulate:
            raise KernelError("gemm_tc: accumulate needs an output")
        out = torch.empty((M, N) if not keep_partials else (1, N), dtype=out_dtype, device=a.device)
    _need(out, "out", out_dtype)
    if (out.shape[0] < M and not keep_partials) or out.shape[1] != N:
        raise KernelError(f"gemm_tc: out has shape {tuple(out.shape)}, needs [{M}, {N}]")
    if w2 is not None:
        _need(w2, "w2", torch.bfloat16, w.shape)
    ws = None
    ws_bytes = 0
    if grouped:
        offsets, tile_group, tile_row0, num_tiles = groups
        max_tiles = tile_group.numel()
    else:
        offsets = tile_group = tile_row0 = num_tiles = None
        max_tiles = 0
        if w2 is None:
            lib.q6k_gemm_tc_workspace.restype = ctypes.c_longlong
            ws_bytes = lib.q6k_gemm_tc_workspace(_i(M), _i(N), _i(K))
            if ws_bytes:
                ws = _workspace(ws_bytes, a.device)
                ws_bytes = ws.numel() * 4
    _call("q6k_gemm_tc", _ptr(a), _ll(a.stride(0)), _i(M), _ptr(w), _ptr(w2), _i(G), _i(N), _i(K), _ptr(out), _i(out.stride(0)),
          _i(epi), _ptr(tile_group), _ptr(tile_row0), _ptr(offsets), _ptr(num_tiles), _i(max_tiles), _i(bt), _ptr(ws),
          _ll(ws_bytes), _i(1 if keep_partials else 0), _stream())
    if keep_partials:
        return ws[: splits * M * N].view(splits, M, N)
    return out


# --------------------------------------------------------------------------- matrix-vector products (a step of very few tokens)
@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def gemv_preferred(tokens: int, N: int, K: int) -> bool:
    """Whether a bfloat16 product of `tokens` rows with an [N, K] matrix should go to the matrix-vector kernel."""
    lib = library()
    lib.q6k_gemv_preferred.restype = ctypes.c_int
    return bool(lib.q6k_gemv_preferred(_i(tokens), _i(N), _i(K)))


def gemv(x: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None, accumulate: bool = False,
         pair_expert: Optional[torch.Tensor] = None, pair_div: int = 1, pairs_are_old: bool = False) -> torch.Tensor:
    """out[t] (+)= x[t] @ w^T for one to four rows of x (bfloat16, FP32 sums and output); with w2 the SwiGLU epilogue
    silu(x w^T) * (x w2^T) in bfloat16.  With pair_expert (int32 [pairs]) and w [experts, N, K]: pair y multiplies row
    y // pair_div of x with the matrix of expert pair_expert[y] and writes row y (any number of pairs).
    The kernel streams its weights while the kernel launched before it on the stream still runs (only x and out wait
    for that kernel); with a pair list this needs the caller's word (pairs_are_old) that the list was not made by that
    very kernel."""
    if not tc_supported(x, w):
        raise KernelError("gemv: operands must be bfloat16 with K a multiple of 8 and 16-byte aligned rows")
    K = x.shape[1]
    N = w.shape[-2]
    if w.shape[-1] != K or (w.dim() == 3) != (pair_expert is not None):
        raise KernelError(f"gemv: x has K={K}, w has shape {tuple(w.shape)} (three dimensions go with pair_expert)")
    pairs = 0
    if pair_expert is not None:
        _need(pair_expert, "pair_expert", torch.int32)
        pairs = pair_expert.numel()
    rows = pairs if pair_expert is not None else x.shape[0]
    epi = EPI_SWIGLU if w2 is not None else (EPI_ADD if accumulate else EPI_STORE)
    out_dtype = torch.bfloat16 if w2 is not None else torch.float32
    if w2 is not None:
        _need(w2, "w2", torch.bfloat16, w.shape)
    if out is None:
        if accumulate:
            raise KernelError("gemv: accumulate needs an output")
        out = torch.empty((rows, N), dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype)
    if out.shape[0] < rows or out.shape[1] != N:
        raise KernelError(f"gemv: out has shape {tuple(out.shape)}, needs [{rows}, {N}]")
    early = pair_expert is None or pairs_are_old
    _call("q6k_gemv", _ptr(x), _ll(x.stride(0)), _i(x.shape[0]), _ptr(w), _ptr(w2), _i(N), _i(K), _ptr(pair_expert), _i(pairs), _i(pair_div),
          _ptr(out), _ll(out.stride(0)), _i(epi), _i(1 if early else 0), _stream())
    return out


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def gemm_skinny_preferred(tokens: int, N: int, K: int) -> bool:
    """Whether a bfloat16 product of `tokens` rows (3 to 16) with an [N, K] matrix should go to the mma.sync kernel for few tokens."""
    lib = library()
    lib.q6k_gemm_skinny_preferred.restype = ctypes.c_int
    return bool(lib.q6k_gemm_skinny_preferred(_i(tokens), _i(N), _i(K)))


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def gemm_skinny_slices(tokens: int, N: int, K: int) -> int:
    """Slices of K the mma.sync kernel for few tokens would cut a plain product into when the caller can add partial
    sums itself (a matrix with too few rows to fill the SMs otherwise); 0: the product is not for this kernel."""
    lib = library()
    lib.q6k_gemm_skinny_slices.restype = ctypes.c_int
    return lib.q6k_gemm_skinny_slices(_i(tokens), _i(N), _i(K))


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, w2: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                accumulate: bool = False, slices: int = 1) -> torch.Tensor:
    """out[t] (+)= x[t] @ w^T for at most 16 rows of x (bfloat16, FP32 sums and output) on mma.sync; with w2 the SwiGLU
    epilogue silu(x w^T) * (x w2^T) in bfloat16.  K is not split over blocks unless slices > 1 (plain products only):
    the result is then [slices, T, N] partial sums, a view of the device's scratch buffer that stays valid until the
    next kernel that uses scratch; the consumer adds the slices in order."""
    if not tc_supported(x, w) or w.dim() != 2:
        raise KernelError("gemm_skinny: operands must be bfloat16 matrices with K a multiple of 8 and 16-byte aligned rows")
    T, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"gemm_skinny: x has K={K}, w has K={w.shape[1]}")
    epi = EPI_SWIGLU if w2 is not None else (EPI_ADD if accumulate else EPI_STORE)
    out_dtype = torch.bfloat16 if w2 is not None else torch.float32
    if w2 is not None:
        _need(w2, "w2", torch.bfloat16, w.shape)
    if slices > 1:
        if out is not None or epi != EPI_STORE:
            raise KernelError("gemm_skinny: slices of K are for plain products into scratch")
        out = _workspace(slices * T * N * 4, x.device)[: slices * T * N].view(slices, T, N)
        _call("q6k_gemm_skinny", _ptr(x), _ll(x.stride(0)), _i(T), _ptr(w), _ptr(w2), _i(N), _i(K), _ptr(out), _ll(N), _i(epi), _i(slices),
              _ll(T * N), _stream())
        return out
    if out is None:
        if accumulate:
            raise KernelError("gemm_skinny: accumulate needs an output")
        out = torch.empty((T, N), dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype)
    if out.shape[0] < T or out.shape[1] != N:
        raise KernelError(f"gemm_skinny: out has shape {tuple(out.shape)}, needs [{T}, {N}]")
    _call("q6k_gemm_skinny", _ptr(x), _ll(x.stride(0)), _i(T), _ptr(w), _ptr(w2), _i(N), _i(K), _ptr(out), _ll(out.stride(0)), _i(epi), _i(1),
          _ll(0), _stream())
    return out


# --------------------------------------------------------------------------- attention
def qk_prep(qkv: torch.Tensor, Hq: int, Hkv: int, hd: int, q_norm, k_norm, eps: float, rotary,
            positions: torch.Tensor, req_of_token: torch.Tensor, block_table: Optional[torch.Tensor], page_size: int,
            k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """QK-norm, rotation, q -> out_dtype [T, Hq, hd]; k, v -> their pages (when k_pages is given).
    rotary: None, or (inv_freq float32 [rotary_dim / 2] on the device, rotary_dim, neighbours): the
    first rotary_dim dimensions of every q and k head turn by position * inv_freq[pair], paired by
    halves (d with d + rotary_dim / 2) or, neighbours=True, 2i with 2i + 1.
    qkv may be [slices, T, width]: split-K partial products, summed in order first."""
    _need(qkv, "qkv", torch.float32)
    splits, split_stride = 1, 0
    if qkv.dim() == 3:
        splits, split_stride = qkv.shape[0], qkv.shape[1] * qkv.shape[2]
        qkv = qkv[0]
    T = qkv.shape[0]
    if qkv.shape[1] < (Hq + 2 * Hkv) * hd and k_pages is not None:
        raise KernelError("qk_prep: qkv rows are too short")
    _need(positions, "positions", torch.int32)
    _need(req_of_token, "req_of_token", torch.int32)
    write = k_pages is not None
    if write:
        _need(k_pages, "k_pages", out_dtype)
        _need(v_pages, "v_pages", out_dtype, k_pages.shape)
        _need(block_table, "block_table", torch.int32)
        if k_pages.dim() != 4 or k_pages.shape[0] != Hkv or tuple(k_pages.shape[2:]) != (page_size, hd):
            raise KernelError(f"qk_prep: pages have shape {tuple(k_pages.shape)}, expected [{Hkv}, *, {page_size}, {hd}]")
    for nm, w in (("q_norm", q_norm), ("k_norm", k_norm)):
        if w is not None:
            _need(w, nm, torch.float32, (hd,))
    inv_freq, rotary_dim, neighbours = rotary if rotary is not None else (None, 0, False)
    if inv_freq is not None:
        if rotary_dim <= 0 or rotary_dim % 2 or rotary_dim > hd:
            raise KernelError(f"qk_prep: {rotary_dim} rotating dimensions of a head of {hd}")
        _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
    q = torch.empty((T, Hq, hd), dtype=out_dtype, device=qkv.device)
    max_blocks = block_table.shape[1] if block_table is not None else 1
    _call("q6k_qk_prep", _ptr(qkv), _i(qkv.stride(0)), _i(splits), _ll(split_stride), _i(T), _i(Hq), _i(Hkv), _i(hd), _ptr(q_norm), _ptr(k_norm), _f(eps),
          _ptr(inv_freq), _i(rotary_dim), _i(1 if neighbours else 0), _ptr(positions), _ptr(req_of_token), _ptr(block_table),
          _i(max_blocks), _i(page_size), _i(k_pages.shape[1] if write else 0), _ptr(q), _ptr(k_pages), _ptr(v_pages),
          _i(1 if write else 0), _i(dtype_code(out_dtype)), _stream())
    return q


def attention_generic(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                      req_of_token: torch.Tensor, positions: torch.Tensor, window: Optional[int],
                      sinks: Optional[torch.Tensor], scale: Optional[float] = None) -> torch.Tensor:
    """Causal (optionally windowed, optionally with sinks) attention of every row over its request's pages."""
    _need(q, "q")
    T, Hq, hd = q.shape
    _need(k_pages, "k_pages", q.dtype)
    _need(v_pages, "v_pages", q.dtype, k_pages.shape)
    Hkv, num_pages, page_size, hd2 = k_pages.shape
    if hd2 != hd:
        raise KernelError(f"attention: q has head_dim {hd}, the pages {hd2}")
    _need(block_table, "block_table", torch.int32)
    _need(req_of_token, "req_of_token", torch.int32)
    _need(positions, "positions", torch.int32)
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (Hq,))
    out = torch.empty((T, Hq * hd), dtype=q.dtype, device=q.device)
    _call("q6k_attention_generic", _ptr(q), _ptr(k_pages), _ptr(v_pages), _i(num_pages), _ptr(block_table), _i(block_table.shape[1]),
          _i(page_size), _ptr(req_of_token), _ptr(positions), _i(window or 0), _ptr(sinks),
          _f(scale if scale is not None else 1.0 / math.sqrt(hd)), _ptr(out), _i(T), _i(Hq), _i(Hkv), _i(hd),
          _i(dtype_code(q.dtype)), _stream())
    return out


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def attention_tc_supported(hd: int, G: int, page_size: int) -> bool:
    lib = library()
    lib.q6k_attention_tc_supported.restype = ctypes.c_int
    return bool(lib.q6k_attention_tc_supported(_i(hd), _i(G), _i(page_size)))


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def attention_tc_tile_tokens(G: int) -> int:
    """Tokens one tile of attention_tc may hold (128 // G: 128 query rows)."""
    lib = library()
    lib.q6k_attention_tc_tile_tokens.restype = ctypes.c_int
    return lib.q6k_attention_tc_tile_tokens(_i(G))


def attention_tc(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                 req_of_token: torch.Tensor, positions: torch.Tensor, tile_tok0: torch.Tensor, tile_ntok: torch.Tensor,
                 window: Optional[int], sinks: Optional[torch.Tensor], scale: Optional[float] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bfloat16 attention for prompt portions with both products on tcgen05 tensor cores
    (accumulators and probabilities in tensor memory, K/V pages by TMA).  Head size 128.
    tile_tok0 / tile_ntok: [n, 2], two tiles of one request per CTA (StepContext.query_tile_pairs),
    each of at most attention_tc_tile_tokens(G) tokens at consecutive positions; the second may be
    empty.  Each tile reads its whole key range; the two share the K/V stream.  Only the rows of
    the listed tiles are written (into `out` [T, Hq*hd] when given)."""
    _need(q, "q", torch.bfloat16)
    T, Hq, hd = q.shape
    _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16, k_pages.shape)
    Hkv, num_pages, page_size, hd2 = k_pages.shape
    if hd2 != hd:
        raise KernelError(f"attention: q has head_dim {hd}, the pages {hd2}")
    for nm, t in (("block_table", block_table), ("req_of_token", req_of_token), ("positions", positions),
                  ("tile_tok0", tile_tok0), ("tile_ntok", tile_ntok)):
        _need(t, nm, torch.int32)
    if tile_tok0.dim() != 2 or tile_tok0.shape[1] != 2 or tile_ntok.shape != tile_tok0.shape:
        raise KernelError("attention_tc: tile_tok0 and tile_ntok must be [pairs, 2]")
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (Hq,))
    if out is None:
        out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=q.device)
    else:
        _need(out, "out", torch.bfloat16, (T, Hq * hd))
    _call("q6k_attention_tc", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ll(num_pages), _ptr(block_table),
          _i(block_table.shape[1]), _i(page_size), _ptr(req_of_token), _ptr(positions), _ptr(tile_tok0), _ptr(tile_ntok),
          _i(tile_tok0.shape[0]), _i(window or 0), _ptr(sinks), _f(scale if scale is not None else 1.0 / math.sqrt(hd)), _ptr(out),
          _i(Hq), _i(Hkv), _i(hd), _stream())
    return out


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def attention_mma_supported(hd: int, G: int, wide: bool) -> bool:
    lib = library()
    lib.q6k_attention_mma_supported.restype = ctypes.c_int
    return bool(lib.q6k_attention_mma_supported(_i(hd), _i(G), _i(1 if wide else 0)))


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def attention_mma_tile_rows(hd: int, G: int, max_tokens: int) -> int:
    """Query rows of the tiles attention_mma should be given when no request brings more than
    max_tokens tokens to the step: 8, 16 or 128 (a tile holds rows // G tokens); 0 if the kernel
    does not take this head and group size."""
    lib = library()
    lib.q6k_attention_mma_tile_rows.restype = ctypes.c_int
    return lib.q6k_attention_mma_tile_rows(_i(hd), _i(G), _i(max_tokens))


_resident = {}


def attention_mma_resident_ctas(hd: int, rows: int) -> int:
    """CTAs of attention_mma (tiles of `rows` rows) the current device runs at once: the number of
    work items per launch (over all KV heads) that makes exactly one wave."""
    key = (torch.cuda.current_device(), hd, rows)
    if key not in _resident:
        lib = library()
        lib.q6k_attention_mma_resident_ctas.restype = ctypes.c_int
        n = lib.q6k_attention_mma_resident_ctas(_i(hd), _i(rows))
        if n <= 0:
            raise KernelError(f"attention_mma: no resident CTA count for head_dim {hd}, tiles of {rows} rows")
        _resident[key] = n
    return _resident[key]


def attention_plan(positions: torch.Tensor, req_of_token: torch.Tensor, tile_tok0: torch.Tensor, tile_ntok: torch.Tensor,
                   window: Optional[int], n_work: int, min_per: int = 2, into=None):
    """Which CTA of attention_mma walks which key tiles, made on the device from the step's
    positions: (work int32 [n_work, 8], tile_plan int32 [n_tiles, 4]).  n_work (at least the number
    of tiles) CTAs per KV head share the key tiles about evenly; a tile's keys are split into
    parts of at least min_per key tiles (of 64 keys).  One plan serves every layer with this
    window; recorded into a CUDA graph it is remade from the positions of each replay.
    into: the pair of tensors of an earlier call with the same sizes, to be filled again."""
    for nm, t in (("req_of_token", req_of_token), ("positions", positions), ("tile_tok0", tile_tok0), ("tile_ntok", tile_ntok)):
        _need(t, nm, torch.int32)
    n_tiles = tile_tok0.numel()
    n_work = max(int(n_work), n_tiles)
    if into is not None:
        work, tile_plan = into
        _need(work, "work", torch.int32, (n_work, 8))
        _need(tile_plan, "tile_plan", torch.int32, (n_tiles, 4))
    else:
        work = torch.empty((n_work, 8), dtype=torch.int32, device=positions.device)
        tile_plan = torch.empty((n_tiles, 4), dtype=torch.int32, device=positions.device)
    _call("q6k_attention_plan", _ptr(positions), _ptr(req_of_token), _ptr(tile_tok0), _ptr(tile_ntok), _i(n_tiles), _i(window or 0),
          _i(n_work), _i(min_per), _ptr(work), _ptr(tile_plan), _stream())
    return work, tile_plan


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def attention_mma_prepares(hd: int, G: int, rows: int, rotary_dim: int, neighbours: bool) -> bool:
    """Whether attention_mma with tiles of `rows` rows can make q and the new keys itself (its `prepare` argument)
    for heads of hd in groups of G with rotary_dim rotating dimensions (0: none)."""
    lib = library()
    lib.q6k_attention_mma_prepares.restype = ctypes.c_int
    return bool(lib.q6k_attention_mma_prepares(_i(hd), _i(G), _i(rows), _i(rotary_dim), _i(1 if neighbours else 0)))


def attention_mma(q: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, block_table: torch.Tensor,
                  req_of_token: torch.Tensor, positions: torch.Tensor, tile_tok0: torch.Tensor, tile_ntok: torch.Tensor,
                  rows: int, window: Optional[int], sinks: Optional[torch.Tensor], max_splits: int = 1, min_tiles: int = 2,
                  scale: Optional[float] = None, out: Optional[torch.Tensor] = None, plan=None, plan_is_old: bool = False,
                  prepare=None) -> torch.Tensor:
    """bfloat16 tensor-core attention over the pages.  Tiles: tile_tok0[i] is the first row and
    tile_ntok[i] the number of tokens (consecutive positions of one request, at most rows // G;
    rows: 8, 16 or 128, see attention_mma_tile_rows) of tile i.  plan: attention_plan(...) of these tiles and this
    window; without one it is made here for max_splits CTAs per tile on average, none with fewer
    than min_tiles key tiles.  Only the rows of the listed tiles are written (into `out`
    [T, Hq*hd] when given).  plan_is_old: the caller's word that the plan and the block table were
    made before the kernel launched just before this call (the one that writes this step's q and
    keys); narrow tiles then fetch their older key tiles while that kernel still runs.

    prepare (tiles of 8 or 16 rows, see attention_mma_prepares; q is then None): a dict with what
    qk_prep takes: qkv float32 [T, >= (Hq + 2 Hkv) hd], heads (Hq), q_norm, k_norm, eps, rotary,
    write (bool); qkv may be [slices, T, width] split-K partial products.  The kernel then normalises, rotates and rounds q itself, and with write=True
    makes the tiles' keys and values and puts them into the pages (every token of the step must
    then lie in a tile).  With plan_is_old the plan must be older than the kernel that made qkv
    AND the one before it."""
    _need(k_pages, "k_pages", torch.bfloat16)
    _need(v_pages, "v_pages", torch.bfloat16, k_pages.shape)
    Hkv, num_pages, page_size, hd = k_pages.shape
    qkv = q_norm = k_norm = inv_freq = None
    eps, rotary_dim, write, ld, splits, split_stride = 0.0, 0, False, 0, 1, 0
    if prepare is not None:
        qkv, Hq, write = prepare["qkv"], int(prepare["heads"]), bool(prepare.get("write", False))
        if not qkv.is_cuda or qkv.dtype != torch.float32 or qkv.dim() not in (2, 3) or qkv.stride(-1) != 1:
            raise KernelError("attention_mma: qkv must be float32 rows [T, width] or [slices, T, width] on the device (rows may have a pitch of their own)")
        if qkv.dim() == 3:                   # split-K partial products: summed in order by the kernel
            splits, split_stride = qkv.shape[0], qkv.stride(0)
        T, ld = qkv.shape[-2], qkv.stride(-2)
        if qkv.shape[-1] < (Hq + 2 * Hkv if write else Hq) * hd:
            raise KernelError(f"attention_mma: qkv of shape {tuple(qkv.shape)} for {Hq} + 2 x {Hkv} heads of {hd}")
        q_norm, k_norm, eps = prepare.get("q_norm"), prepare.get("k_norm"), float(prepare.get("eps", 0.0))
        for nm, w in (("q_norm", q_norm), ("k_norm", k_norm)):
            if w is not None:
                _need(w, nm, torch.float32, (hd,))
        if prepare.get("rotary") is not None:
            inv_freq, rotary_dim, neighbours = prepare["rotary"]
            _need(inv_freq, "inv_freq", torch.float32, (rotary_dim // 2,))
            if neighbours:
                raise KernelError("attention_mma: pairs of neighbours are rotated by qk_prep only")
        dev = qkv.device
    else:
        _need(q, "q", torch.bfloat16)
        T, Hq, hd2 = q.shape
        if hd2 != hd:
            raise KernelError(f"attention: q has head_dim {hd2}, the pages {hd}")
        dev = q.device
    _need(block_table, "block_table", torch.int32)
    if sinks is not None:
        _need(sinks, "sinks", torch.float32, (Hq,))
    n_tiles = tile_tok0.numel()
    if plan is None:
        plan_is_old = False
        plan = attention_plan(positions, req_of_token, tile_tok0, tile_ntok, window, n_tiles * max(1, max_splits), min_tiles)
    work, tile_plan = plan
    _need(work, "work", torch.int32)
    _need(tile_plan, "tile_plan", torch.int32, (n_tiles, 4))
    n_work = work.shape[0]
    if out is None:
        out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=dev)
    else:
        _need(out, "out", torch.bfloat16, (T, Hq * hd))
    part_o = part_ml = None
    if n_work > n_tiles:
        part_rows = n_work * Hkv * rows
        ws = _workspace(part_rows * (hd + 2) * 4, dev, "attention")       # a buffer of its own: qkv may be a view of the common one
        part_o = ws[: part_rows * hd]
        part_ml = ws[part_rows * hd: part_rows * (hd + 2)]
    _call("q6k_attention_mma", _ptr(q), _ptr(k_pages), _ptr(v_pages), _ll(num_pages), _ptr(block_table),
          _i(block_table.shape[1]), _i(page_size), _ptr(work), _ptr(tile_plan), _i(n_work), _i(n_tiles), _i(rows),
          _i(window or 0), _ptr(sinks), _f(scale if scale is not None else 1.0 / math.sqrt(hd)), _ptr(out), _ptr(part_o), _ptr(part_ml),
          _i(Hq), _i(Hkv), _i(hd), _i(1 if plan_is_old else 0), _ptr(qkv), _i(ld), _i(splits), _ll(split_stride), _ptr(q_norm), _ptr(k_norm), _f(eps),
          _ptr(inv_freq), _i(rotary_dim), _i(1 if write else 0), _stream())
    return out


# --------------------------------------------------------------------------- routing
def route(logits: torch.Tensor, k: int, scoring: str, renorm: bool):
    """(sel_e int32 [T, k], sel_w float32 [T, k]).  logits: [T, E], or [slices, T, E] split-K
    partial products of the router, which are summed in order first."""
    _need(logits, "logits", torch.float32)
    slices = logits.shape[0] if logits.dim() == 3 else 1
    T, E = logits.shape[-2:]
    if scoring not in ("softmax", "sigmoid"):
        raise KernelError(f"route: unknown scoring {scoring!r}")
    sel_e = torch.empty((T, k), dtype=torch.int32, device=logits.device)
    sel_w = torch.empty((T, k), dtype=torch.float32, device=logits.device)
    _call("q6k_route", _ptr(logits), _i(slices), _i(T), _i(E), _i(k), _i(1 if scoring == "sigmoid" else 0), _i(1 if renorm else 0),
          _ptr(sel_e), _ptr(sel_w), _stream())
    return sel_e, sel_w


@functools.lru_cache(maxsize=None)          # a question about sizes: asked of the library once
def router_small_supported(T: int, E: int, D: int, k: int) -> bool:
    """Whether the one-launch decode router (router_small, and with it the per-pair expert products) takes this step."""
    lib = library()
    lib.q6k_router_small_supported.restype = ctypes.c_int
    return bool(lib.q6k_router_small_supported(_i(T), _i(E), _i(D), _i(k)))



def router_small(xn: torch.Tensor, w: torch.Tensor, k: int, scoring: str, renorm: bool, with_logits: bool = False):
    """Router logits, scores and top-k of at most 16 tokens in one launch:
    (sel_e [T, k], sel_w [T, k], order [T*k]: the pairs sorted by expert); with_logits: also the
    FP32 router logits [T, E] the kernel left behind."""
    _need(xn, "xn", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    T, D = xn.shape
    E = w.shape[0]
    if w.shape[1] != D:
        raise KernelError("router_small: widths disagree")
    dev = xn.device
    logits = torch.empty((T, E), dtype=torch.float32, device=dev)
    sel_e = torch.empty((T, k), dtype=torch.int32, device=dev)
    sel_w = torch.empty((T, k), dtype=torch.float32, device=dev)
    order = torch.empty(T * k, dtype=torch.int32, device=dev)
    _call("q6k_router_small", _ptr(xn), _ptr(w), _i(T), _i(E), _i(D), _i(k), _i(1 if scoring == "sigmoid" else 0),
          _i(1 if renorm else 0), _ptr(logits), _ptr(sel_e), _ptr(sel_w), _ptr(order), _stream())
    return (sel_e, sel_w, order, logits) if with_logits else (sel_e, sel_w, order)


_pair_scratch = {}


def gemm_tc_pairs(a: torch.Tensor, w: torch.Tensor, pair_expert: torch.Tensor, pair_div: int, w2: Optional[torch.Tensor] = None,
                  order: Optional[torch.Tensor] = None, pairs_are_old: bool = False) -> torch.Tensor:
    """Expert products of a decode step without a permutation: pair y (= token * slots + slot)
    multiplies row y // pair_div of `a` with expert pair_expert[y]; output row y.  With w2 the
    SwiGLU epilogue (bfloat16 output), else FP32.  pairs_are_old: the caller's word that
    pair_expert and order were not made by the kernel launched just before this one; the kernel
    then fetches its first weights while that kernel still runs."""
    if not tc_supported(a, w) or w.dim() != 3:
        raise KernelError("gemm_tc_pairs: operands must be bfloat16, K a multiple of 8, weights [experts, N, K]")
    _need(pair_expert, "pair_expert", torch.int32)
    pairs = pair_expert.numel()
    if order is not None:
        _need(order, "order", torch.int32, (pairs,))
    G, N, K = w.shape
    if a.shape[1] != K:
        raise KernelError(f"gemm_tc_pairs: a has K={a.shape[1]}, w has K={K}")
    if w2 is not None:
        _need(w2, "w2", torch.bfloat16, w.shape)
    out = torch.empty((pairs, N), dtype=torch.bfloat16 if w2 is not None else torch.float32, device=a.device)
    # a few pairs only: K is sliced over CTAs, which meet through scratch kept per device (one stream uses it at a time)
    floats, counters = ctypes.c_longlong(), ctypes.c_int()
    _call("q6k_gemm_tc_pairs_scratch", _i(pairs), _i(N), _i(K), _i(1 if w2 is not None else 0), ctypes.byref(floats), ctypes.byref(counters))
    partial = tickets = None
    if floats.value:
        key = str(a.device)
        partial, tickets = _pair_scratch.get(key, (None, None))
        if partial is None or partial.numel() < floats.value or tickets.numel() < counters.value:
            _retired.append((partial, tickets))
            partial = torch.empty(max(floats.value, 1 << 18), dtype=torch.float32, device=a.device)
            tickets = torch.zeros(max(counters.value, 1024), dtype=torch.int32, device=a.device)
            _pair_scratch[key] = (partial, tickets)
    _call("q6k_gemm_tc_pairs", _ptr(a), _ll(a.stride(0)), _i(a.shape[0]), _ptr(w), _ptr(w2), _i(G), _i(N), _i(K), _ptr(out),
          _i(out.stride(0)), _i(EPI_SWIGLU if w2 is not None else EPI_STORE), _ptr(pair_expert), _ptr(order), _i(pairs), _i(pair_div),
          _ptr(partial), _ll(partial.numel() if partial is not None else 0), _ptr(tickets),
          _i(tickets.numel() if tickets is not None else 0), _i(1 if pairs_are_old else 0), _stream())
    return out


def moe_permute(sel_e: torch.Tensor, E: int):
    """(offsets [E+1], pair_row [T, k], row_token [T*k]): rows sorted by expert, stable in pair order."""
    _need(sel_e, "sel_e", torch.int32)
    T, k = sel_e.shape
    pairs = T * k
    dev = sel_e.device
    lib = library()
    lib.q6k_moe_permute_scratch_ints.restype = ctypes.c_int
    scratch = torch.empty(lib.q6k_moe_permute_scratch_ints(_i(pairs), _i(E)), dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    pair_row = torch.empty((T, k), dtype=torch.int32, device=dev)
    row_token = torch.empty(pairs, dtype=torch.int32, device=dev)
    _call("q6k_moe_permute", _ptr(sel_e), _i(pairs), _i(k), _i(E), _ptr(scratch), _ptr(offsets), _ptr(pair_row),
          _ptr(row_token), _stream())
    return offsets, pair_row, row_token


def moe_plan(sel_e: torch.Tensor, E: int, bm: int, x: Optional[torch.Tensor] = None):
    """The permutation of `moe_permute` and the row tiles of `tile_list(offsets, pairs, bm)` in three
    launches instead of four: (offsets, pair_row, row_token, (offsets, tile_group, tile_row0, num_tiles)).
    With x [T, D] (rows of a multiple of 16 bytes) the last launch also copies each pair's input
    row into its place, and the gathered rows [pairs, D] are returned as a fifth value."""
    _need(sel_e, "sel_e", torch.int32)
    T, k = sel_e.shape
    pairs = T * k
    dev = sel_e.device
    lib = library()
    lib.q6k_moe_permute_scratch_ints.restype = ctypes.c_int
    scratch = torch.empty(lib.q6k_moe_permute_scratch_ints(_i(pairs), _i(E)), dtype=torch.int32, device=dev)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=dev)
    pair_row = torch.empty((T, k), dtype=torch.int32, device=dev)
    row_token = torch.empty(pairs, dtype=torch.int32, device=dev)
    max_tiles = pairs // bm + min(pairs, E)          # full tiles plus at most one ragged tile per non-empty group
    tile_group = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    tile_row0 = torch.empty(max_tiles, dtype=torch.int32, device=dev)
    num_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    gathered, row_bytes = None, 0
    if x is not None:
        _need(x, "x")
        if x.dim() != 2 or x.shape[0] != T:
            raise KernelError(f"moe_plan: x has shape {tuple(x.shape)}, expected [{T}, D]")
        row_bytes = x.shape[1] * x.element_size()
        if row_bytes % 16:
            raise KernelError(f"moe_plan: rows of {row_bytes} bytes cannot be gathered 16 bytes at a time")
        gathered = torch.empty((pairs, x.shape[1]), dtype=x.dtype, device=dev)
    _call("q6k_moe_plan", _ptr(sel_e), _i(pairs), _i(k), _i(E), _ptr(scratch), _ptr(offsets), _ptr(pair_row), _ptr(row_token), _i(bm),
          _ptr(tile_group), _ptr(tile_row0), _ptr(num_tiles), _i(max_tiles), _ptr(x), _ptr(gathered), _i(row_bytes), _stream())
    plan = (offsets, pair_row, row_token, (offsets, tile_group, tile_row0, num_tiles))
    return plan if x is None else plan + (gathered,)


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """int32 [rows]; ties go to the lower id.  `out`: an int32 buffer of at least `rows` entries to write into."""
    _need(logits, "logits", torch.float32)
    rows, V = logits.shape
    if out is None:
        out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    else:
        _need(out, "out", torch.int32)
        if out.numel() < rows:
            raise KernelError(f"argmax: the output buffer holds {out.numel()} ids, {rows} rows are asked for")
        out = out[:rows]
    lib = library()
    lib.q6k_argmax_scratch_ints.restype = ctypes.c_int
    scratch = torch.empty(lib.q6k_argmax_scratch_ints(_i(rows), _i(V)), dtype=torch.int32, device=logits.device)
    _call("q6k_argmax", _ptr(logits), _i(rows), _i(V), _ptr(out), _ptr(scratch), _stream())
    return out


def row_logsumexp(logits: torch.Tensor, target: Optional[torch.Tensor] = None):
    """log(sum(exp(row))) of every row, FP32 [rows]; with target (int32 [rows]) also each row's logit at its target."""
    _need(logits, "logits", torch.float32)
    rows, V = logits.shape
    lse = torch.empty(rows, dtype=torch.float32, device=logits.device)
    picked = None
    if target is not None:
        _need(target, "target", torch.int32, (rows,))
        picked = torch.empty(rows, dtype=torch.float32, device=logits.device)
    _call("q6k_row_lse", _ptr(logits), _i(rows), _i(V), _ptr(target), _ptr(lse), _ptr(picked), _stream())
    return lse if target is None else (lse, picked)


def sample_pool(ids: torch.Tensor, vals: torch.Tensor, rows: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row from the sorted pools topk_pool made, chosen on the device with the
    host sampler's arithmetic (no penalties).  rows: int32 [n, 8] on the device, per row the
    32-byte record {int32 candidates, int32 top_k, float32 temperature, top_p, min_p, unused,
    float64 uniform}; a row with no candidates keeps what `out` held."""
    _need(ids, "ids", torch.int32)
    n, K = ids.shape
    _need(vals, "vals", torch.float32, (n, K))
    _need(rows, "rows", torch.int32, (n, 8))
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=ids.device)
    else:
        _need(out, "out", torch.int32)
        if out.numel() < n:
            raise KernelError(f"sample_pool: out holds {out.numel()} ids, {n} rows are sampled")
    _call("q6k_sample_pool", _ptr(ids), _ptr(vals), _i(n), _i(K), _ptr(rows), _ptr(out), _stream())
    return out[:n]


def topk_pool(logits: torch.Tensor, k: int):
    """(ids int32 [rows, k], vals float32 [rows, k]) sorted by (logit descending, id ascending); k <= 256."""
    _need(logits, "logits", torch.float32)
    rows, V = logits.shape
    ids = torch.empty((rows, k), dtype=torch.int32, device=logits.device)
    vals = torch.empty((rows, k), dtype=torch.float32, device=logits.device)
    _call("q6k_topk_pool", _ptr(logits), _i(rows), _i(V), _i(k), _ptr(ids), _ptr(vals), _stream())
    return ids, vals
