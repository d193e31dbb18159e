"""In-tree native build: compiles the C++ runtime, the pluggable allocator, the CPU back end and every CUDA
kernel for sm_100a into shared libraries under ``iris_b200/lib``.

Role in the reference: ``setup.py:13-84`` and ``csrc/finegrained_alloc/build.sh:5-15`` (one hipcc command).
Here nvcc cross-compiles without a GPU, so the same function serves the build check and the GPU box.

Run ``python -m iris_b200._build`` (add ``-v`` for ptxas resource usage, ``-f`` to force a rebuild).
"""
from __future__ import annotations

import json
import os
import re
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
# host libraries build warning-free; the reference builds its allocator the same way (csrc/finegrained_alloc/build.sh:5-15)
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra", "-Werror", "-I", str(INCLUDE), "-I", str(CSRC)]


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


def parse_ptxas(log: str) -> dict:
    """Resource usage per kernel from the output of ``nvcc -Xptxas -v``: ``{mangled name: {registers, barriers,
    stack_bytes, spill_store_bytes, spill_load_bytes, smem_bytes}}`` (the figures the reference reads from Triton's
    compiled kernel as ``n_regs`` / ``n_spills``, ``examples/07_gemm_all_scatter/matmul_wrapper.py:152-155``)."""
    out, name, props_of = {}, None, None
    for line in log.splitlines():
        m = re.search(r"Compiling entry function '([^']+)'", line)
        if m:
            name = m.group(1)
            out[name] = dict(registers=0, barriers=0, stack_bytes=0, spill_store_bytes=0, spill_load_bytes=0, smem_bytes=0)
            continue
        m = re.search(r"Function properties for (\S+)", line)
        if m:
            props_of = m.group(1)   # may be a device function compiled out of line: not an entry of `out`
            continue
        m = re.search(r"(\d+) bytes stack frame, (\d+) bytes spill stores, (\d+) bytes spill loads", line)
        if m:
            if props_of in out:
                out[props_of].update(stack_bytes=int(m.group(1)), spill_store_bytes=int(m.group(2)),
                                     spill_load_bytes=int(m.group(3)))
            continue
        m = re.search(r"Used (\d+) registers", line)
        if m and name is not None:
            out[name]["registers"] = int(m.group(1))
            b = re.search(r"used (\d+) barriers", line)
            s_ = re.search(r"(\d+) bytes smem", line)
            out[name]["barriers"] = int(b.group(1)) if b else 0
            out[name]["smem_bytes"] = int(s_.group(1)) if s_ else 0
    return out


def _demangle(names):
    filt = shutil.which("c++filt")
    if not filt or not names:
        return {n: n for n in names}
    p = subprocess.run([filt], input="\n".join(names), capture_output=True, text=True)
    lines = p.stdout.splitlines()
    return dict(zip(names, lines)) if p.returncode == 0 and len(lines) == len(names) else {n: n for n in names}


def kernel_resources() -> dict:
    """``{demangled kernel name: resources}`` of the kernels in ``libiris_kernels.so``, as recorded at build time."""
    path = LIB / "kernel_resources.json"
    return json.loads(path.read_text()) if path.exists() else {}


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
            jobs.append((s, [NVCC, "-Xptxas", "-v", *NVCC_FLAGS, "-c", s, "-o", o]))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda j: _run(j[1], verbose), jobs))
        for (s, _), log in zip(jobs, logs):  # registers, spills, shared memory of every kernel of this source
            (OBJ / (s.stem + ".resources.json")).write_text(json.dumps(parse_ptxas(log)))
    res_path = LIB / "kernel_resources.json"
    if jobs or force or _newer(out, objs) or not res_path.exists():
        _run([NVCC, *ARCH_FLAGS, "-shared", "-o", out, *objs, "-cudart", "static"], verbose)
        merged = {}
        for s in srcs:
            f = OBJ / (s.stem + ".resources.json")
            if f.exists():
                merged.update(json.loads(f.read_text()))
        names = _demangle(list(merged))
        res_path.write_text(json.dumps({names[k]: dict(v, source_symbol=k) for k, v in merged.items()}, indent=1))
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
