"""Collectives executed by the NVLink switch (``csrc/kernels/nvls.cu``, ``include/iris/nvls.cuh``).

They need a context whose heap is bound to a multicast object: ``iris_b200.iris(size, heap_mode="vmm")`` with
``IRIS_NVLS=1`` in the environment; ``ctx.mc_base`` is then non-zero.  No counterpart in the reference.
"""
from __future__ import annotations

import ctypes

import torch

from .. import _native


def available(ctx) -> bool:
    return bool(getattr(ctx, "mc_base", 0))


def _mc(ctx, t: torch.Tensor) -> int:
    return ctx.mc_base + ctx.offset_of(t)


def all_store(ctx, dst_sym: torch.Tensor, nbytes=None, grid=None, block=512, stream=None) -> None:
    """Write the 32-bit word index into ``dst`` of EVERY rank with one multicast store per vector."""
    if not available(ctx):
        raise RuntimeError("heap is not bound to an NVLS multicast object")
    n = dst_sym.numel() * dst_sym.element_size() if nbytes is None else int(nbytes)
    lib = _native.kernels()
    lib.iris_k_nvls_all_store.argtypes = [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    st = torch.cuda.current_stream(ctx.device).cuda_stream if stream is None else stream
    if lib.iris_k_nvls_all_store(_mc(ctx, dst_sym), n, grid or ctx.get_cu_count() * 4, block, ctypes.c_void_p(st)):
        raise RuntimeError("nvls_all_store launch failed")


class AllReduce:
    """In-place sum of a bf16 heap buffer over all ranks: ``multimem.ld_reduce`` + ``multimem.st`` per slice."""

    def __init__(self, ctx, timeout_ms: float = 5000.0):
        if not available(ctx):
            raise RuntimeError("heap is not bound to an NVLS multicast object")
        self.ctx = ctx
        self.counter = ctx.zeros(16, dtype=torch.int32)
        self.total = 0
        self.timeout_ns = int(timeout_ms * 1e6)
        ctx.barrier()   # construction is collective: no rank arrives on a counter its owner has not zeroed yet

    def reset(self) -> None:
        """Collective recovery after ``ctx.check_status()`` reported a time-out of this op (sites 80 / 81): a rank whose
        wait expired may have left a call half-way, so the cumulative counter no longer matches ``total`` everywhere.
        Every rank calls ``reset()``: the counters are zeroed between two barriers and counting starts again."""
        self.ctx.barrier()
        self.counter.zero_()
        self.total = 0
        self.ctx.barrier()

    def __call__(self, buf: torch.Tensor, grid=None, block=512, stream=None) -> torch.Tensor:
        ctx = self.ctx
        assert buf.dtype == torch.bfloat16 and (buf.numel() * 2) % 16 == 0
        grid = min(grid or ctx.get_cu_count(), ctx.get_cu_count())  # all blocks wait on one another: co-resident
        world = ctx.get_num_ranks()
        self.total += 2 * grid * world   # arrivals so far; the kernel keeps its own count in device memory
        lib = _native.kernels()
        lib.iris_k_nvls_all_reduce_bf16.argtypes = [ctypes.c_uint64, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64,
                                                    ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_void_p]
        st = torch.cuda.current_stream(ctx.device).cuda_stream if stream is None else stream
        rc = lib.iris_k_nvls_all_reduce_bf16(
            _mc(ctx, buf), ctypes.c_void_p(ctx.get_heap_bases().data_ptr()), ctx.offset_of(self.counter),
            ctx.offset_of(ctx.status), buf.numel() * 2, ctx.get_rank(), world, self.timeout_ns,
            ctx.mc_base, grid, block, ctypes.c_void_p(st))
        if rc:
            raise RuntimeError("nvls_all_reduce launch failed")
        return buf
