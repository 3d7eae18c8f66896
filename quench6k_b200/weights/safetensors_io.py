"""Reading and writing safetensors files without a library: 8-byte little-endian header length,
a JSON header {name: {dtype, shape, data_offsets}}, then the raw little-endian data.

Behaviour follows the reference's index (crates/engine/src/checkpoint.rs:108-246): every
`*.safetensors` of a folder (or the shards that `model.safetensors.index.json` names) is indexed
by tensor name, byte ranges are checked against the file, and a name that occurs twice is an error.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Tuple

import torch

_DTYPES = {
    "BF16": (torch.bfloat16, 2), "F16": (torch.float16, 2), "F32": (torch.float32, 4), "F64": (torch.float64, 8),
    "I8": (torch.int8, 1), "U8": (torch.uint8, 1), "I16": (torch.int16, 2), "I32": (torch.int32, 4),
    "I64": (torch.int64, 8), "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


class SafetensorsError(ValueError):
    pass


@dataclass
class TensorEntry:
    name: str
    dtype: torch.dtype
    shape: Tuple[int, ...]
    path: str
    begin: int        # absolute byte offsets in the file
    end: int


class SafetensorsFile:
    """One file's tensors by name.  The header is parsed and the data read by the C++ host library
    (csrc/host/host.cpp, q6k_st_*: pread straight into the tensor's memory) unless Q6K_HOST=python
    (or native=False) asks for the Python twin below, which gives the same entries and messages."""

    def __init__(self, path: str, native: Optional[bool] = None):
        self.path = path
        self.entries: Dict[str, TensorEntry] = {}
        self._h = None
        self._mm = None
        if native is None:
            native = os.environ.get("Q6K_HOST", "").lower() != "python"
        if native:
            self._open_native()
        else:
            self._open_python()

    # ------------------------------------------------------------------ C++
    def _open_native(self) -> None:
        import ctypes
        from ..cache.native import host_lib
        lib = host_lib()
        h = ctypes.c_void_p()
        if lib.q6k_st_open(os.fsencode(self.path), ctypes.byref(h)):
            raise SafetensorsError(lib.q6k_host_last_error().decode())
        self._h, self._lib, self._index = h, lib, {}
        name, dtype = ctypes.create_string_buffer(4096), ctypes.create_string_buffer(8)
        shape, ndim = (ctypes.c_int64 * 8)(), ctypes.c_int32()
        begin, end = ctypes.c_int64(), ctypes.c_int64()
        for i in range(lib.q6k_st_count(h)):
            if lib.q6k_st_entry(h, i, name, 4096, dtype, shape, ctypes.byref(ndim), ctypes.byref(begin), ctypes.byref(end)):
                raise SafetensorsError(f"{self.path}: {lib.q6k_host_last_error().decode()}")
            n = name.value.decode()
            self.entries[n] = TensorEntry(n, _DTYPES[dtype.value.decode()][0], tuple(shape[d] for d in range(ndim.value)), self.path,
                                          begin.value, end.value)
            self._index[n] = i

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.q6k_st_close(h)

    # ------------------------------------------------------------------ Python twin
    def _open_python(self) -> None:
        path = self.path
        size = os.path.getsize(path)
        with open(path, "rb") as f:
            head = f.read(8)
            if len(head) < 8:
                raise SafetensorsError(f"{path}: shorter than a safetensors header")
            (n,) = struct.unpack("<Q", head)
            if n > size - 8:
                raise SafetensorsError(f"{path}: header length {n} exceeds the file ({size} bytes)")
            try:
                header = json.loads(f.read(n))
            except (json.JSONDecodeError, UnicodeDecodeError) as e:
                raise SafetensorsError(f"{path}: header is not JSON ({e})") from None
        base = 8 + n
        if not isinstance(header, dict):
            raise SafetensorsError(f"{path}: header is not JSON (expected an object)")
        for name, info in header.items():
            if name == "__metadata__":
                continue
            if not isinstance(info, dict) or not {"dtype", "shape", "data_offsets"} <= set(info) or len(info["data_offsets"]) != 2:
                raise SafetensorsError(f"{path}: tensor {name} lacks dtype, shape or data_offsets")
            if info["dtype"] not in _DTYPES:
                raise SafetensorsError(f"{path}: tensor {name} has unsupported dtype {info['dtype']}")
            dt, width = _DTYPES[info["dtype"]]
            shape = tuple(int(x) for x in info["shape"])
            b, e = info["data_offsets"]
            count = 1
            for s in shape:
                count *= s
            if min(shape, default=0) < 0 or e - b != count * width or b < 0 or base + e > size:
                raise SafetensorsError(f"{path}: tensor {name} has byte range {b}..{e} for shape {shape} {info['dtype']} in a file of {size} bytes")
            self.entries[name] = TensorEntry(name, dt, shape, path, base + b, base + e)

    def read(self, name: str) -> torch.Tensor:
        """A CPU tensor with the stored dtype and shape (a copy; nothing of the file is kept alive by it)."""
        ent = self.entries[name]
        nbytes = ent.end - ent.begin
        if nbytes == 0:
            return torch.empty(ent.shape, dtype=ent.dtype)
        if self._h is not None:
            out = torch.empty(ent.shape, dtype=ent.dtype)
            if self._lib.q6k_st_read(self._h, self._index[name], out.data_ptr(), nbytes):
                raise SafetensorsError(f"{self.path}: {self._lib.q6k_host_last_error().decode()}")
            return out
        if self._mm is None:
            self._f = open(self.path, "rb")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        buf = bytearray(self._mm[ent.begin:ent.end])
        return torch.frombuffer(buf, dtype=ent.dtype).reshape(ent.shape)


    def read_range(self, name: str, offset: int, out: torch.Tensor) -> None:
        """out.numel() bytes of the tensor's data from byte `offset` into `out` (uint8, contiguous, on the CPU;
        pinned memory when it is a staging buffer of an upload)."""
        ent = self.entries[name]
        n = out.numel()
        if out.dtype != torch.uint8 or not out.is_contiguous() or offset < 0 or offset + n > ent.end - ent.begin:
            raise SafetensorsError(f"{self.path}: bytes {offset}..{offset + n} of tensor {name} ({ent.end - ent.begin} bytes) into {out.dtype}")
        if n == 0:
            return
        if self._h is not None:
            if self._lib.q6k_st_read_range(self._h, self._index[name], offset, out.data_ptr(), n):
                raise SafetensorsError(f"{self.path}: {self._lib.q6k_host_last_error().decode()}")
            return
        if self._mm is None:
            self._f = open(self.path, "rb")
            self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)
        out.numpy()[:] = memoryview(self._mm)[ent.begin + offset:ent.begin + offset + n]


def index_folder(folder: str) -> Dict[str, Tuple[SafetensorsFile, TensorEntry]]:
    """name -> (file, entry) over a model folder's safetensors files."""
    idx_path = os.path.join(folder, "model.safetensors.index.json")
    if os.path.exists(idx_path):
        with open(idx_path) as f:
            files = sorted(set(json.load(f)["weight_map"].values()))
    else:
        files = sorted(p for p in os.listdir(folder) if p.endswith(".safetensors"))
    if not files:
        raise SafetensorsError(f"{folder}: no .safetensors file")
    out: Dict[str, Tuple[SafetensorsFile, TensorEntry]] = {}
    for fn in files:
        sf = SafetensorsFile(os.path.join(folder, fn))
        for name, ent in sf.entries.items():
            if name in out:
                raise SafetensorsError(f"duplicate tensor {name} in {out[name][0].path} and {sf.path}")
            out[name] = (sf, ent)
    return out


def write_safetensors(path: str, tensors: Iterable[Tuple[str, torch.Tensor]]) -> None:
    """Write CPU tensors in the given order."""
    items: List[Tuple[str, torch.Tensor]] = [(n, t.detach().cpu().contiguous()) for n, t in tensors]
    header = {}
    off = 0
    for name, t in items:
        if t.dtype not in _NAMES:
            raise SafetensorsError(f"tensor {name}: dtype {t.dtype} cannot be stored")
        nb = t.numel() * t.element_size()
        header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [off, off + nb]}
        off += nb
    blob = json.dumps(header, separators=(",", ":")).encode()
    blob += b" " * ((8 - len(blob) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(blob)))
        f.write(blob)
        for _, t in items:
            if t.numel():
                f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.dtype != torch.bool else t.numpy().tobytes())
