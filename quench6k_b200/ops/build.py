"""Compiles the CUDA sources under csrc/ for sm_100a into one shared library and loads it; the
C++ host sources under csrc/host/ (cache manager, scheduler, step packing: no CUDA in them) become
a second library built with the C++ compiler alone, so host-only tests need no nvcc.

The sources include no torch header, so a fresh checkout builds in well under a minute with plain
nvcc; the launchers are `extern "C"` and are called through ctypes with raw device pointers and
the current CUDA stream.  The library is built in-tree (next to this file) when that folder can be
written, else in a per-user folder under the system's temporary directory.  A line is printed to
stderr for every file compiled, so a first call is never silent for long.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
from concurrent.futures import ThreadPoolExecutor
from typing import List, Optional

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(_HERE), "csrc")
LIB_NAME = "libq6k_b200.so"
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

HOST_LIB_NAME = "libq6k_host.so"
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-ffp-contract=off", "-pthread"]

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_host_lib: Optional[ctypes.CDLL] = None


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("Q6K_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise BuildError("nvcc not found (looked at $Q6K_NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built")


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h")))


def _digest() -> str:
    h = hashlib.sha256()
    for p in sources() + _headers():
        h.update(os.path.basename(p).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def _writable(folder: str) -> bool:
    try:
        os.makedirs(folder, exist_ok=True)
        probe = os.path.join(folder, f".probe_{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return True
    except OSError:
        return False


def _build_dirs():
    """(folder of the .so, folder of the objects)"""
    if _writable(_HERE) and _writable(os.path.join(CSRC, "_build")):
        return _HERE, os.path.join(CSRC, "_build")
    base = os.path.join(tempfile.gettempdir(), f"q6k_b200_{os.getuid()}")
    os.makedirs(base, exist_ok=True)
    return base, os.path.join(base, "_build")


def _say(msg: str) -> None:
    print(f"[quench6k_b200 build] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True) -> str:
    """Build if the library is missing or older than the sources; return the library's path."""
    lib_dir, obj_dir = _build_dirs()
    lib_path = os.path.join(lib_dir, LIB_NAME)
    stamp = os.path.join(lib_dir, LIB_NAME + ".digest")
    digest = _digest()
    if os.path.exists(lib_path) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return lib_path
    nvcc = _nvcc()
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {lib_path}")

    def compile_one(src: str) -> str:
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + "." + digest + ".o")
        if not os.path.exists(obj):
            tmp = obj + f".tmp{os.getpid()}"
            r = subprocess.run([nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", tmp], capture_output=True, text=True)
            if r.returncode != 0:
                raise BuildError(f"nvcc failed on {os.path.basename(src)}:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, obj)
        if verbose:
            _say(f"compiled {os.path.basename(src)}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = lib_path + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-cudart", "static"], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib_path)
    with open(stamp, "w") as f:
        f.write(digest)
    for f in os.listdir(obj_dir):            # objects of older source versions
        if f.endswith(".o") and f".{digest}." not in f:
            try:
                os.remove(os.path.join(obj_dir, f))
            except OSError:
                pass
    if verbose:
        _say("done")
    return lib_path


def library() -> ctypes.CDLL:
    """The loaded kernel library.  Raises if it cannot be built or loaded: there is no fallback."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
        return _lib


# ---------------------------------------------------------------------------------- host library
def host_sources() -> List[str]:
    folder = os.path.join(CSRC, "host")
    return sorted(os.path.join(folder, f) for f in os.listdir(folder) if f.endswith((".cpp", ".h")))


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), "g++", "c++", "clang++"):
        path = shutil.which(cand) if cand else None
        if path:
            return path
    raise BuildError("no C++ compiler found (looked at $CXX, g++, c++, clang++): the host library cannot be built")


def build_host(verbose: bool = True) -> str:
    lib_dir, _ = _build_dirs()
    lib_path = os.path.join(lib_dir, HOST_LIB_NAME)
    stamp = lib_path + ".digest"
    h = hashlib.sha256()
    for p in host_sources() + [os.path.join(CSRC, "fill_normal.h")]:      # the generator's header is shared with the device code
        with open(p, "rb") as f:
            h.update(os.path.basename(p).encode() + f.read())
    h.update(" ".join(HOST_FLAGS).encode())
    digest = h.hexdigest()[:16]
    if os.path.exists(lib_path) and os.path.exists(stamp) and open(stamp).read().strip() == digest:
        return lib_path
    if verbose:
        _say(f"compiling the C++ host library into {lib_path}")
    tmp = lib_path + f".tmp{os.getpid()}"
    cpps = [p for p in host_sources() if p.endswith(".cpp")]
    r = subprocess.run([_cxx(), *HOST_FLAGS, "-o", tmp, *cpps], capture_output=True, text=True)
    if r.returncode != 0:
        raise BuildError(f"building {HOST_LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib_path)
    with open(stamp, "w") as f:
        f.write(digest)
    return lib_path


def host_library() -> ctypes.CDLL:
    """The loaded host library (cache manager, scheduler, step packing)."""
    global _host_lib
    with _lock:
        if _host_lib is None:
            path = build_host()
            try:
                _host_lib = ctypes.CDLL(path)
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from None
        return _host_lib
