"""In-tree native build: compiles the C++ runtime, the pluggable allocator, the CPU back end and every CUDA
kernel for sm_100a into shared libraries under ``iris_b200/lib``.

Role in the reference: ``setup.py:13-84`` and ``csrc/finegrained_alloc/build.sh:5-15`` (one hipcc command).
Here nvcc cross-compiles without a GPU, so the same function serves the build check and the GPU box.

Run ``python -m iris_b200._build`` (add ``-v`` for ptxas resource usage, ``-f`` to force a rebuild).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG / "include"
LIB = PKG / "lib"
OBJ = PKG / "build"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-Wall", "-I", str(INCLUDE), "-I", str(CSRC)] + ARCH_FLAGS
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-I", str(INCLUDE), "-I", str(CSRC)]


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def _headers():
    return list(INCLUDE.rglob("*.cuh")) + list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h"))


def _run(cmd, verbose=False):
    if verbose:
        print(" ".join(map(str, cmd)), flush=True)
    p = subprocess.run(list(map(str, cmd)), capture_output=True, text=True)
    if p.returncode != 0:
        sys.stderr.write(p.stdout + p.stderr)
        raise RuntimeError("build step failed: " + " ".join(map(str, cmd)))
    if verbose and (p.stdout or p.stderr):
        print(p.stdout + p.stderr, flush=True)
    return p.stdout + p.stderr


def kernel_sources():
    return sorted((CSRC / "kernels").glob("*.cu"))


def build_cpu(force=False, verbose=False) -> Path:
    out = LIB / "libiris_cpu.so"
    src = CSRC / "cpu" / "iris_cpu_backend.cpp"
    if force or _newer(out, [src] + _headers()):
        _run(["g++", *CXX_FLAGS, "-shared", "-o", out, src, "-lrt", "-pthread"], verbose)
    return out


def _cuda_host_lib(out: Path, src: Path, force, verbose) -> Path:
    if force or _newer(out, [src] + _headers()):
        _run(["g++", *CXX_FLAGS, "-I", CUDA_HOME / "include", "-shared", "-o", out, src,
              "-L", CUDA_HOME / "lib64", "-lcudart_static", "-ldl", "-lrt", "-pthread"], verbose)
    return out


def build_runtime(force=False, verbose=False) -> Path:
    return _cuda_host_lib(LIB / "libiris_runtime.so", CSRC / "runtime" / "iris_runtime.cpp", force, verbose)


def build_allocator(force=False, verbose=False) -> Path:
    return _cuda_host_lib(LIB / "libiris_allocator.so", CSRC / "alloc" / "iris_allocator.cpp", force, verbose)


def build_kernels(force=False, verbose=False) -> Path:
    out = LIB / "libiris_kernels.so"
    OBJ.mkdir(exist_ok=True)
    srcs = kernel_sources()
    hdrs = _headers()
    objs, jobs = [], []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or _newer(o, [s] + hdrs):
            cmd = [NVCC, *NVCC_FLAGS, "-c", s, "-o", o]
            if verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda c: _run(c, verbose), jobs))
        if verbose:
            (OBJ / "ptxas.log").write_text("\n".join(logs))
    if jobs or force or _newer(out, objs):
        _run([NVCC, *ARCH_FLAGS, "-shared", "-o", out, *objs, "-cudart", "static"], verbose)
    return out


def build_all(force=False, verbose=False):
    """Build every native library; returns their paths.  Raises if a compiler is missing or fails."""
    LIB.mkdir(exist_ok=True)
    if shutil.which("g++") is None:
        raise RuntimeError("g++ not found")
    libs = {"cpu": build_cpu(force, verbose)}
    if not Path(NVCC).exists():
        raise RuntimeError(f"nvcc not found at {NVCC}; set CUDA_HOME")
    libs["runtime"] = build_runtime(force, verbose)
    libs["allocator"] = build_allocator(force, verbose)
    libs["kernels"] = build_kernels(force, verbose)
    return libs


if __name__ == "__main__":
    libs = build_all(force="-f" in sys.argv, verbose="-v" in sys.argv)
    for k, v in libs.items():
        print(f"{k}: {v}")
