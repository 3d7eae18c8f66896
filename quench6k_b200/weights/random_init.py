"""Random-weights mode: tensors from a declaration and a seed, on any device, and a model folder
(config.json + model.safetensors) written from a configuration and a seed.

Every element is a pure function of (seed, tensor name, element index): a splitmix64 hash (the
generator the reference's samplers use, crates/cli/src/flint.rs:318-325) gives two uniforms and
Box-Muller a normal.  Tensors can therefore be produced one at a time, in pieces, on the host or on
the device, without holding the model twice.  The host (csrc/host/host.cpp) and the device
(csrc/fill.cu) run the same arithmetic (csrc/fill_normal.h) and give the same bits.
"""
from __future__ import annotations

import ctypes
import os
from typing import Callable, Dict, List, Optional

import torch

from ..spec import TensorSpec
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1


def _fnv1a(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def stream_key(seed: int, name: str) -> int:
    """The 64-bit key of the stream of (seed, tensor name)."""
    return (seed * 0x9E3779B97F4A7C15 + _fnv1a(name)) & _M64


def fill_normal(out: torch.Tensor, seed: int, name: str, start: int = 0, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
    """out.view(-1)[i] = out.dtype(N(0,1)[start + i] * std + mean) of the stream of (seed, name);
    out: contiguous float32 or bfloat16, on the CPU (the C++ host library fills it, with threads)
    or on a CUDA device (the fill kernel)."""
    if not out.is_contiguous() or out.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"fill_normal: needs a contiguous float32 or bfloat16 tensor, got {out.dtype}")
    code = 0 if out.dtype == torch.float32 else 1
    key = stream_key(seed, name)
    if out.is_cuda:
        from .. import ops
        with torch.cuda.device(out.device):
            ops._call("q6k_fill_normal", ctypes.c_void_p(out.data_ptr()), ctypes.c_int(code), ctypes.c_longlong(out.numel()),
                      ctypes.c_longlong(start), ctypes.c_ulonglong(key), ctypes.c_float(std), ctypes.c_float(mean), ops._stream())
    else:
        from ..cache.native import host_lib, raise_for
        raise_for(host_lib().q6k_fill_normal_host(out.data_ptr(), code, out.numel(), start, key, std, mean, min(32, os.cpu_count() or 1)))
    return out


def standard_normal(seed: int, name: str, start: int, count: int, device) -> torch.Tensor:
    """Elements start..start+count of the N(0,1) stream of (seed, name), float32."""
    return fill_normal(torch.empty(count, dtype=torch.float32, device=device), seed, name, start)


def make_tensor(spec: TensorSpec, seed: int, default_std: float, device="cpu", dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """One declared tensor.  Matrices are bfloat16 unless `dtype` says otherwise; 'f32' tensors are
    float32; 'i32' tensors are zeros."""
    if spec.role == "i32":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    out_dtype = torch.float32 if spec.role == "f32" else (dtype or torch.bfloat16)
    out = torch.empty(spec.shape, dtype=out_dtype, device=device)
    kind = spec.init[0]
    std = spec.init[1] if len(spec.init) > 1 and spec.init[1] is not None else default_std
    if kind == "ones":
        return out.fill_(1.0)
    if kind not in ("normal", "ones_plus"):
        raise ValueError(f"tensor {spec.name}: unknown init {spec.init!r}")
    return fill_normal(out, seed, spec.name, 0, std, 1.0 if kind == "ones_plus" else 0.0)


def random_getter(declared: List[TensorSpec], seed: int, default_std: float, device="cpu") -> Callable[[str], torch.Tensor]:
    by_name: Dict[str, TensorSpec] = {s.name: s for s in declared}

    def get(name: str) -> torch.Tensor:
        return make_tensor(by_name[name], seed, default_std, device)

    return get


def write_model_folder(folder: str, config, declared: List[TensorSpec], seed: int, default_std: float) -> None:
    """config.json and model.safetensors of a randomly initialised model."""
    os.makedirs(folder, exist_ok=True)
    config.save(folder)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      ((s.name, make_tensor(s, seed, default_std)) for s in declared))
