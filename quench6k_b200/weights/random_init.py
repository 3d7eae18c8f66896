"""Random-weights mode: tensors from a declaration and a seed, on any device, and a model folder
(config.json + model.safetensors) written from a configuration and a seed.

Every element is a pure function of (seed, tensor name, element index): a splitmix64 hash (the
generator the reference's samplers use, crates/cli/src/flint.rs:318-325) gives two uniforms and
Box-Muller a normal.  Tensors can therefore be produced one at a time, in pieces, on the host or on
the device, without holding the model twice.
"""
from __future__ import annotations

import os
from typing import Callable, Dict, List, Optional

import torch

from ..spec import TensorSpec
from .safetensors_io import write_safetensors

_M64 = (1 << 64) - 1
_CHUNK = 1 << 24


def _fnv1a(name: str) -> int:
    h = 0xCBF29CE484222325
    for b in name.encode():
        h = ((h ^ b) * 0x100000001B3) & _M64
    return h


def _i64(x: int) -> int:
    """A Python integer in [0, 2^64) as the int64 with the same bits."""
    return x - (1 << 64) if x >= (1 << 63) else x


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 bit patterns."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _i64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _i64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def standard_normal(seed: int, name: str, start: int, count: int, device) -> torch.Tensor:
    """Elements start..start+count of the N(0,1) stream of (seed, name), float32."""
    key = (seed * 0x9E3779B97F4A7C15 + _fnv1a(name)) & _M64
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    a = _mix(idx * 2 + _i64(key))
    b = _mix(idx * 2 + 1 + _i64(key))
    u1 = (_lsr(a, 11).to(torch.float64) + 1.0) / float(1 << 53)      # (0, 1]
    u2 = _lsr(b, 11).to(torch.float64) / float(1 << 53)              # [0, 1)
    z = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * torch.pi * u2)
    return z.to(torch.float32)


def make_tensor(spec: TensorSpec, seed: int, default_std: float, device="cpu", dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """One declared tensor.  Matrices are bfloat16 unless `dtype` says otherwise; 'f32' tensors are
    float32; 'i32' tensors are zeros."""
    n = 1
    for s in spec.shape:
        n *= s
    if spec.role == "i32":
        return torch.zeros(spec.shape, dtype=torch.int32, device=device)
    out_dtype = torch.float32 if spec.role == "f32" else (dtype or torch.bfloat16)
    out = torch.empty(n, dtype=out_dtype, device=device)
    kind = spec.init[0]
    std = spec.init[1] if len(spec.init) > 1 and spec.init[1] is not None else default_std
    if kind == "ones":
        out.fill_(1.0)
    else:
        for s0 in range(0, n, _CHUNK):
            c = min(_CHUNK, n - s0)
            z = standard_normal(seed, spec.name, s0, c, device) * std
            if kind == "ones_plus":
                z = z + 1.0
            elif kind != "normal":
                raise ValueError(f"tensor {spec.name}: unknown init {spec.init!r}")
            out[s0:s0 + c] = z.to(out_dtype)
    return out.reshape(spec.shape)


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
