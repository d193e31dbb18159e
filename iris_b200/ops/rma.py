"""Host entry points of the RMA primitives (load, store, get, put, atomic_*), applied element-wise.

On the device the primitives are C++ functions of ``include/iris/iris.cuh`` meant to be called from user
kernels (``iris/iris.py:317-521`` in the reference are Triton functions used the same way).  This module
launches the generic kernel ``csrc/kernels/rma_generic.cu`` — or, for a CPU context, the same code compiled
for the host — so every primitive x dtype x semantics x scope can be exercised from Python.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native

OPS = {"load": 0, "store": 1, "get": 2, "put": 3, "atomic_add": 4, "atomic_sub": 5, "atomic_cas": 6,
       "atomic_xchg": 7}
SEMS = {"relaxed": 0, "acquire": 1, "release": 2, "acq_rel": 3, None: 3}
SCOPES = {"cta": 0, "gpu": 1, "sys": 2, None: 1}
DTYPES = {torch.int8: 0, torch.int16: 1, torch.int32: 2, torch.int64: 3, torch.float16: 4, torch.bfloat16: 5,
          torch.float32: 6, torch.float64: 7}


class UnsupportedRma(TypeError):
    pass


def _ptr(t: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def rma(ctx, op: str, a: torch.Tensor, b: Optional[torch.Tensor] = None, c: Optional[torch.Tensor] = None, *,
        value=1, compare=0, target: int = -1, sem: Optional[str] = None, scope: Optional[str] = None,
        block: int = 256, n: Optional[int] = None, stream=None) -> None:
    """Apply primitive ``op`` to the first ``n`` elements.

    ``a`` is the symmetric operand (pointer into this rank's heap), ``b`` the second buffer of get/put,
    ``c`` the local result buffer (sums for load/get, old values for atomics).  ``target=-1`` applies the
    primitive to every rank including the caller, as the reference's unit tests do.
    """
    if op not in OPS:
        raise ValueError(f"unknown op {op!r}")
    if a.dtype not in DTYPES:
        raise UnsupportedRma(f"dtype {a.dtype} is not supported")
    n = a.numel() if n is None else int(n)
    hb = ctx.get_heap_bases()
    is_int = not a.dtype.is_floating_point
    fvalue = 0.0 if is_int else float(value)
    ivalue = int(compare) if op == "atomic_cas" else (int(value) if is_int else 0)
    ivalue2 = int(value) if op == "atomic_cas" else 0
    args = [OPS[op], DTYPES[a.dtype], SEMS[sem], SCOPES[scope], _ptr(a), _ptr(b), _ptr(c), n,
            ctypes.c_void_p(hb.data_ptr()), ctx.get_rank(), ctx.get_num_ranks(), int(target),
            ctypes.c_double(fvalue), ivalue, ivalue2]
    if ctx.backend == "cpu":
        rc = _native.cpu().iris_cpu_rma(*args, max(1, min(4, block // 64)))
    else:
        lib = _native.kernels()
        fn = lib.iris_k_rma
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_int] * 4 + [ctypes.c_void_p] * 3 + [ctypes.c_int64, ctypes.c_void_p] + \
            [ctypes.c_int] * 3 + [ctypes.c_double, ctypes.c_int64, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
        st = torch.cuda.current_stream(ctx.device).cuda_stream if stream is None else stream
        rc = fn(*args, int(block), ctypes.c_void_p(st))
    if rc == -2:
        raise UnsupportedRma(f"{op} is not supported for {a.dtype} on backend {ctx.backend}")
    if rc != 0:
        raise RuntimeError(f"rma {op} failed with code {rc}")


def load(ctx, src, out, target=-1, **kw):
    rma(ctx, "load", src, None, out, target=target, **kw)


def store(ctx, dst, value, target=-1, **kw):
    rma(ctx, "store", dst, value=value, target=target, **kw)


def get(ctx, src, local, out, target=-1, **kw):
    rma(ctx, "get", src, local, out, target=target, **kw)


def put(ctx, local_src, dst, target=-1, **kw):
    rma(ctx, "put", local_src, dst, target=target, **kw)


def atomic_add(ctx, buf, value=1, old=None, target=-1, **kw):
    rma(ctx, "atomic_add", buf, None, old, value=value, target=target, **kw)


def atomic_sub(ctx, buf, value=1, old=None, target=-1, **kw):
    rma(ctx, "atomic_sub", buf, None, old, value=value, target=target, **kw)


def atomic_cas(ctx, buf, compare, value, old=None, target=-1, **kw):
    rma(ctx, "atomic_cas", buf, None, old, value=value, compare=compare, target=target, **kw)


def atomic_xchg(ctx, buf, value, old=None, target=-1, **kw):
    rma(ctx, "atomic_xchg", buf, None, old, value=value, target=target, **kw)
