"""Compile user CUDA kernels written against ``<iris/iris.cuh>`` and call them from Python.

Role in the reference: ``@triton.jit`` — users of the reference write their own kernels in Triton and call the
``iris.load / store / atomic_*`` device functions inside them (``README.md:31-70``).  Here a kernel is a CUDA C++
string (or file) that includes ``<iris/iris.cuh>``; it is compiled once by nvcc for sm_100a into a shared library
(cached by content hash) and its ``extern "C"`` launchers are called through ctypes with torch tensors, ints,
floats and the context's heap-base table as arguments.

    src = r'''
    #include <iris/iris.cuh>
    __global__ void put_ones(float* buf, int n, int cur, int dst, const uint64_t* heap_bases) {
      int i = blockIdx.x * blockDim.x + threadIdx.x;
      iris::store(buf + i, 1.0f, cur, dst, heap_bases, i < n);
    }
    extern "C" void launch_put_ones(float* buf, int n, int cur, int dst, const uint64_t* hb, void* stream) {
      put_ones<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(buf, n, cur, dst, hb);
    }'''
    mod = iris_b200.jit.compile(src)
    mod.launch_put_ones(buf, buf.numel(), ctx.get_rank(), 1, ctx.get_heap_bases(), mod.current_stream())
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import subprocess
import tempfile
from pathlib import Path
from typing import Iterable, Optional

import torch

PKG = Path(__file__).resolve().parent
NVCC = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
BASE_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
              "-gencode", "arch=compute_100a,code=sm_100a", "-I", str(PKG / "include"), "-cudart", "static"]


class JitError(RuntimeError):
    pass


def cache_dir() -> Path:
    d = Path(os.environ.get("IRIS_JIT_CACHE", os.path.join(tempfile.gettempdir(), f"iris_b200_jit_{os.getuid()}")))
    d.mkdir(parents=True, exist_ok=True)
    return d


def _as_c(arg):
    if isinstance(arg, torch.Tensor):
        return ctypes.c_void_p(arg.data_ptr())
    if isinstance(arg, bool):
        return ctypes.c_int(int(arg))
    if isinstance(arg, int):
        # 32-bit when it fits, as C ints; pass ctypes values explicitly for 64-bit parameters
        return ctypes.c_int(arg) if -2**31 <= arg < 2**31 else ctypes.c_int64(arg)
    if isinstance(arg, float):
        return ctypes.c_float(arg)
    if arg is None:
        return ctypes.c_void_p(0)
    return arg  # already a ctypes value


class Module:
    """A compiled library; attribute access returns a callable that converts tensors to device pointers."""

    def __init__(self, path: Path, log: str):
        self.path, self.log = path, log
        self._lib = ctypes.CDLL(str(path))

    def current_stream(self, device=None):
        return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)

    def __getattr__(self, name):
        try:
            fn = getattr(self._lib, name)
        except AttributeError:
            raise JitError(f"{self.path.name} exports no symbol {name!r} (is the launcher declared extern 'C'?)")
        fn.restype = None

        def call(*args):
            fn(*[_as_c(a) for a in args])
        call.__name__ = name
        return call


def compile(source: str, extra_flags: Iterable[str] = (), name: Optional[str] = None, verbose: bool = False) -> Module:
    """Compile CUDA source (a string, or a path to a ``.cu`` file) and load it."""
    if os.path.exists(source) and source.endswith((".cu", ".cuh")):
        text = Path(source).read_text()
    else:
        text = source
    flags = BASE_FLAGS + list(extra_flags) + (["-Xptxas", "-v"] if verbose else [])
    header_stamp = "".join(sorted(f"{p.name}:{p.stat().st_mtime_ns}" for p in (PKG / "include" / "iris").glob("*.cuh")))
    key = hashlib.sha256((text + "\0" + " ".join(flags) + header_stamp).encode()).hexdigest()[:20]
    out = cache_dir() / f"{name or 'kernel'}_{key}.so"
    log = ""
    if not out.exists():
        if not os.path.exists(NVCC):
            raise JitError(f"nvcc not found at {NVCC}; set CUDA_HOME")
        src_path = out.with_suffix(".cu")
        src_path.write_text(text)
        tmp = out.with_suffix(f".{os.getpid()}.tmp.so")
        p = subprocess.run([NVCC, *flags, "-o", str(tmp), str(src_path)], capture_output=True, text=True)
        log = p.stdout + p.stderr
        if p.returncode != 0:
            raise JitError("nvcc failed:\n" + log)
        os.replace(tmp, out)  # atomic: several ranks may compile the same source at once
    return Module(out, log)
