"""Host launchers of the point-to-point / all-peer RMA kernels and of message passing (``csrc/kernels/p2p.cu``).

Reference workloads: ``examples/00_load`` … ``examples/06_message_passing``.  Each function launches on the
current stream of the context's device and returns immediately.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native

_DT = {torch.float16: 4, torch.bfloat16: 5, torch.float32: 6}


def default_grid(ctx, per_sm: int = 4) -> int:
    return ctx.get_cu_count() * per_sm


def _stream(ctx, stream):
    return ctypes.c_void_p(torch.cuda.current_stream(ctx.device).cuda_stream if stream is None else stream)


def _hb(ctx):
    return ctypes.c_void_p(ctx.get_heap_bases().data_ptr())


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def _nbytes(t, nbytes):
    n = t.numel() * t.element_size() if nbytes is None else int(nbytes)
    if n % 16:
        raise ValueError("byte count must be a multiple of 16")
    if t.data_ptr() % 16:
        raise ValueError("buffer must be 16-byte aligned")
    return n


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what}: launch failed ({rc})")


def load(ctx, src_sym, dst_local, target: int, nbytes=None, grid=None, block=512, stream=None):
    """``dst_local = remote(target).src`` (examples/00_load/load_bench.py:20-48)."""
    lib = _native.kernels()
    n = _nbytes(src_sym, nbytes)
    _check(lib.iris_k_p2p_load(_p(src_sym), _p(dst_local), ctypes.c_uint64(n), ctx.get_rank(), int(target), _hb(ctx),
                               grid or default_grid(ctx), block, _stream(ctx, stream)), "p2p_load")


def store(ctx, dst_sym, target: int, nbytes=None, grid=None, block=512, stream=None):
    """Write the 32-bit word index into ``remote(target).dst`` (examples/01_store/store_bench.py:20-46)."""
    lib = _native.kernels()
    n = _nbytes(dst_sym, nbytes)
    _check(lib.iris_k_p2p_store(_p(dst_sym), ctypes.c_uint64(n), ctx.get_rank(), int(target), _hb(ctx),
                                grid or default_grid(ctx), block, _stream(ctx, stream)), "p2p_store")


def local_store(ctx, dst, nbytes=None, grid=None, block=512, stream=None):
    """Same write pattern into local memory: the overhead term the load benchmark subtracts."""
    lib = _native.kernels()
    n = _nbytes(dst, nbytes)
    _check(lib.iris_k_local_store(_p(dst), ctypes.c_uint64(n), grid or default_grid(ctx), block,
                                  _stream(ctx, stream)), "local_store")


def all_load(ctx, src_sym, out_local, active: Optional[int] = None, nbytes=None, grid=None, block=512, stream=None):
    """``out_local = sum over the first `active` ranks of remote(r).src`` (examples/02_all_load)."""
    lib = _native.kernels()
    n = _nbytes(src_sym, nbytes)
    if src_sym.dtype not in _DT:
        raise TypeError(f"all_load supports {list(_DT)}")
    rc = lib.iris_k_p2p_all_load(_p(src_sym), _p(out_local), ctypes.c_uint64(n), _DT[src_sym.dtype], ctx.get_rank(),
                                 int(active or ctx.get_num_ranks()), _hb(ctx), grid or default_grid(ctx), block,
                                 _stream(ctx, stream))
    _check(rc, "p2p_all_load")


def all_store(ctx, dst_sym, active: Optional[int] = None, nbytes=None, grid=None, block=512, stream=None):
    """Write the word index into ``dst`` of every OTHER rank (examples/03_all_store)."""
    lib = _native.kernels()
    n = _nbytes(dst_sym, nbytes)
    _check(lib.iris_k_p2p_all_store(_p(dst_sym), ctypes.c_uint64(n), ctx.get_rank(),
                                    int(active or ctx.get_num_ranks()), _hb(ctx), grid or default_grid(ctx), block,
                                    _stream(ctx, stream)), "p2p_all_store")


def atomic_add_f32(ctx, buf_sym, target: int, n=None, vec4=False, grid=None, block=512, stream=None):
    """``remote(target).buf[i] += 1`` with relaxed, system-scope reductions (examples/04_atomic_add)."""
    lib = _native.kernels()
    assert buf_sym.dtype == torch.float32
    n = buf_sym.numel() if n is None else int(n)
    _check(lib.iris_k_p2p_atomic_add_f32(_p(buf_sym), ctypes.c_uint64(n), ctx.get_rank(), int(target), _hb(ctx),
                                         int(bool(vec4)), grid or default_grid(ctx), block, _stream(ctx, stream)),
           "p2p_atomic_add")


_ATOMIC_DT = {torch.int32: 2, torch.int64: 3, torch.float16: 4, torch.bfloat16: 5, torch.float32: 6}


def atomic_add(ctx, buf_sym, target: int, n=None, grid=None, block=512, stream=None):
    """``remote(target).buf[i] += 1`` for int32 / int64 / fp16 / bf16 / fp32 buffers, one relaxed system-scope
    reduction per element (the ``--datatype`` choices of ``examples/04_atomic_add/atomic_add_bench.py:68`` of the
    reference that the hardware adds natively; there is no 8-bit atomic on sm_100a)."""
    lib = _native.kernels()
    if buf_sym.dtype not in _ATOMIC_DT:
        raise TypeError(f"atomic_add supports {list(_ATOMIC_DT)}")
    n = buf_sym.numel() if n is None else int(n)
    _check(lib.iris_k_p2p_atomic_add(_p(buf_sym), ctypes.c_uint64(n), _ATOMIC_DT[buf_sym.dtype], ctx.get_rank(),
                                     int(target), _hb(ctx), grid or default_grid(ctx), block, _stream(ctx, stream)),
           "p2p_atomic_add")


def atomic_xchg_i32(ctx, buf_sym, out_local, target: int, n=None, grid=None, block=512, stream=None):
    """``out_local[i] = atomic_xchg(remote(target).buf[i], 1)`` (examples/05_atomic_xchg)."""
    lib = _native.kernels()
    assert buf_sym.dtype == torch.int32 and out_local.dtype == torch.int32
    n = buf_sym.numel() if n is None else int(n)
    _check(lib.iris_k_p2p_atomic_xchg_i32(_p(buf_sym), _p(out_local), ctypes.c_uint64(n), ctx.get_rank(),
                                          int(target), _hb(ctx), grid or default_grid(ctx), block,
                                          _stream(ctx, stream)), "p2p_atomic_xchg")


class MessagePassing:
    """Producer/consumer hand-off of fixed-size chunks guarded by int32 flags.

    The producer copies chunk ``c`` into the consumer's landing buffer and then stores the call number into
    the CONSUMER's ``flags[c]`` with release semantics at system scope; the consumer polls its own flag with
    acquire loads (bounded by ``timeout_ms``), then writes ``out = 2 * landed``.  This is the protocol the
    reference's example intends (``examples/06_message_passing/message_passing_put.py:16-78``), with the flag
    in the consumer's memory and real release/acquire ordering.

    Every chunk is moved by ``parts`` thread blocks at once (default: enough to put about two blocks on every SM, at
    least 16 KB per block), so that a hand-off of a few large chunks runs at link rate instead of at the rate of one
    SM per chunk; the block that finishes a chunk last raises its flag.

    ``blocks`` (default: one per slice) is the number of thread blocks per side; with fewer, block ``b`` takes the
    (chunk, slice) pairs ``b, b + blocks, ...`` in order, so the chunks land one group after the other and the consumer
    works on early chunks while later ones are still on the link.  Only thread 0 of a producer block fences and
    publishes a slice (after the block's barrier: fences are cumulative) while the other warps copy the next slice.

    With ``device_epoch=True`` both sides count their calls in device memory instead of taking the call number as a
    launch argument, so that ``run()`` can be recorded into a CUDA graph and replayed, one hand-off per replay.

    All three buffers, the flags and the arrival counters are allocated on the heap here, in the same order on every
    rank.
    """

    def __init__(self, ctx, nchunks: int, chunk_bytes: int, producer: int = 0, consumer: int = 1,
                 timeout_ms: float = 1000.0, parts: Optional[int] = None, blocks: Optional[int] = None,
                 device_epoch: bool = False):
        if chunk_bytes % 16:
            raise ValueError("chunk_bytes must be a multiple of 16")
        self.ctx, self.nchunks, self.chunk_bytes = ctx, nchunks, chunk_bytes
        self.producer, self.consumer = producer, consumer
        sms = ctx.get_cu_count() if ctx.backend == "cuda" else 1
        if parts is None:
            parts = max(1, min((2 * sms) // max(1, nchunks), chunk_bytes // (16 << 10)))
        self.parts = max(1, int(parts))
        # thread blocks per role; fewer than one per slice makes the chunks complete in order (see mp_kernel)
        self.blocks = 0 if blocks is None else int(blocks)
        # two words beyond the per-chunk entries: this side's call counter and its count of blocks that have left
        self.arrive = ctx.zeros(nchunks + 2, dtype=torch.int32)
        n = nchunks * chunk_bytes // 4
        self.src = ctx.zeros(n, dtype=torch.float32)
        self.dst = ctx.zeros(n, dtype=torch.float32)
        self.out = ctx.zeros(n, dtype=torch.float32)
        self.flags = ctx.zeros(nchunks + 2, dtype=torch.int32)
        # device_epoch: both sides count their calls in device memory instead of taking the call number as a launch
        # argument, so that `run()` can be captured into a CUDA graph and replayed (every replay is one hand-off)
        self.device_epoch = bool(device_epoch)
        self.timeout_ns = int(timeout_ms * 1e6)
        self.epoch = 0
        ctx.barrier()   # construction is collective: the producer must not raise a flag its owner has yet to zero

    def run(self, roles: Optional[int] = None, use_put: bool = True, block: int = 512, stream=None,
            advance: bool = True) -> None:
        """Launch this rank's side.  ``roles``: 1 producer blocks, 2 consumer blocks, 3 both in one cooperative
        launch (ranks simulated on one GPU).  Default: chosen from the context's rank."""
        ctx = self.ctx
        if roles is None:
            roles = (1 if ctx.get_rank() == self.producer else 0) | (2 if ctx.get_rank() == self.consumer else 0)
        if advance:
            self.epoch += 1
        if roles == 0:
            return
        lib = _native.kernels()
        lib.iris_k_message_passing.argtypes = [ctypes.c_void_p] + [ctypes.c_uint64] * 6 + [ctypes.c_int] * 5 + \
            [ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int, ctypes.c_int, ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p]
        parts = self.parts   # with roles == 3 the launcher lowers the block count to what is resident at once
        rc = lib.iris_k_message_passing(
            _hb(ctx), ctx.offset_of(self.src), ctx.offset_of(self.dst), ctx.offset_of(self.out),
            ctx.offset_of(self.flags), ctx.offset_of(ctx.status), self.chunk_bytes, self.nchunks, self.producer,
            self.consumer, roles, int(use_put), 0 if self.device_epoch else self.epoch, self.timeout_ns, block, parts,
            ctx.offset_of(self.arrive), self.blocks, _stream(ctx, stream))
        _check(rc, "message_passing")


class DeviceBarrier:
    """Barrier across ranks executed on the GPUs (one tiny kernel per rank): every rank bumps a counter in every
    peer's heap and waits, bounded, for its own to reach ``calls * world``.  Used to align the ranks' streams
    before a timed region so that host-side launch skew is not charged to the kernel under test.  One process
    per GPU only (kernels that wait on one another must not share a GPU)."""

    def __init__(self, ctx, timeout_ms: float = 5000.0):
        if getattr(ctx, "_local_world", None) is not None:
            raise RuntimeError("DeviceBarrier is for one process per GPU")
        self.ctx = ctx
        self.counter = ctx.zeros(16, dtype=torch.int32)
        self.calls = 0
        self.timeout_ns = int(timeout_ms * 1e6)
        ctx.barrier()   # construction is collective: no rank bumps a counter its owner has not zeroed yet

    def __call__(self, stream=None) -> None:
        ctx = self.ctx
        self.calls += 1
        if ctx.get_num_ranks() == 1:
            return
        lib = _native.kernels()
        lib.iris_k_device_barrier.argtypes = [ctypes.c_void_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int,
                                              ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p]
        # no per-call argument (the kernel counts its calls in counter[1]): the launch can be replayed from a CUDA graph
        rc = lib.iris_k_device_barrier(_hb(ctx), ctx.offset_of(self.counter), ctx.offset_of(ctx.status),
                                       ctx.get_rank(), ctx.get_num_ranks(), self.timeout_ns, _stream(ctx, stream))
        _check(rc, "device_barrier")
