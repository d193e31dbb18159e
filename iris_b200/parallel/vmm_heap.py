"""Symmetric heap built on CUDA virtual memory management (``heap_mode="vmm"``).

Every rank creates its heap with ``cuMemCreate``, exports it as a POSIX file descriptor, passes the descriptor to
the other ranks of the machine over Unix sockets (``SCM_RIGHTS``), and maps all heaps into ONE contiguous virtual
range: rank r's heap sits at ``va + r * stride``.  Pointer translation is then a multiply-add; the base-address
table is still produced for API parity.  When ``IRIS_NVLS=1`` and the GPUs support it, the heaps are also bound
to an NVLink-switch multicast object, whose mapping (``mc_ptr``) accepts ``multimem`` stores / reductions /
load-reduces (``include/iris/nvls.cuh``).

Role in the reference: ``iris/iris.py:55-71`` + ``iris/_hip.py:23-59`` (HIP IPC handles); the reference has no
multicast path (xGMI has no switch).  The native calls are in ``csrc/runtime/iris_runtime.cpp``.
"""
from __future__ import annotations

import ctypes
import os
import uuid
from typing import List

from .. import _native


class VmmHeap:
    def __init__(self):
        self.own_ptr = 0
        self.peer_ptrs: List[int] = []
        self.mc_ptr = 0
        self.stride = 0
        self._va = 0
        self._va_bytes = 0
        self._handles: List[int] = []
        self._mc_handle = 0
        self._mc_va = 0
        self._mc_bound = False
        self._device = 0
        self._mapped: List[int] = []

    def release_multicast(self) -> None:
        """Undo whatever part of the multicast set-up exists (also the way back to plain peer access when a step of
        the set-up failed on some rank)."""
        rt = _native.runtime()
        if self._mc_va:
            rt.iris_rt_vmm_unmap(self._mc_va, self.stride)
            rt.iris_rt_vmm_address_free(self._mc_va, self.stride)
        if self._mc_handle:
            if self._mc_bound:
                rt.iris_rt_multicast_unbind(self._mc_handle, self._device, self.stride)
            rt.iris_rt_vmm_release(self._mc_handle)
        self._mc_va, self._mc_handle, self._mc_bound, self.mc_ptr = 0, 0, False, 0

    def close(self) -> None:
        rt = _native.runtime()
        try:
            self.release_multicast()
            for va in self._mapped:
                rt.iris_rt_vmm_unmap(va, self.stride)
            for h in self._handles:
                rt.iris_rt_vmm_release(h)
            if self._va:
                rt.iris_rt_vmm_address_free(self._va, self._va_bytes)
        finally:
            self._mapped, self._handles, self._va = [], [], 0


def _exchange_fds(ctx, token: str, own_fd: int, what: str) -> List[int]:
    """Every rank ends up with a descriptor for every rank's object (its own included)."""
    rt = _native.runtime()
    rank, world = ctx.cur_rank, ctx.num_ranks
    name = f"iris_b200_{token}_{what}_{rank}"
    sock = rt.iris_rt_fd_listen(name.encode())
    if sock < 0:
        raise RuntimeError("fd exchange: " + rt.iris_rt_last_error().decode())
    ctx.comm.barrier()  # all sockets are bound
    fds = [-1] * world
    fds[rank] = own_fd
    try:
        for peer in range(world):
            if peer != rank:
                if rt.iris_rt_fd_send(f"iris_b200_{token}_{what}_{peer}".encode(), own_fd, rank) != 0:
                    raise RuntimeError("fd exchange: " + rt.iris_rt_last_error().decode())
        for _ in range(world - 1):
            tag = ctypes.c_int(-1)
            fd = rt.iris_rt_fd_recv(sock, 30000, ctypes.byref(tag))
            if fd < 0 or not 0 <= tag.value < world:
                raise RuntimeError("fd exchange: " + rt.iris_rt_last_error().decode())
            fds[tag.value] = fd
    finally:
        rt.iris_rt_fd_close(sock)
    ctx.comm.barrier()
    return fds


def create(ctx) -> VmmHeap:
    rt = _native.runtime()
    dev, rank, world = ctx.gpu_id, ctx.cur_rank, ctx.num_ranks
    if not rt.iris_rt_vmm_supported(dev):
        raise RuntimeError("this GPU / driver does not export device memory as POSIX file descriptors")
    gran = rt.iris_rt_vmm_granularity(dev)
    if gran <= 0:
        raise RuntimeError("cuMemGetAllocationGranularity failed")
    want_mc = os.environ.get("IRIS_NVLS", "0") == "1" and world > 1 and bool(rt.iris_rt_multicast_supported(dev))
    if want_mc:
        mg = rt.iris_rt_multicast_granularity(world, ctx.heap_size)
        if mg > 0:
            gran = max(gran, mg)
    h = VmmHeap()
    h._device = dev
    h.stride = -(-ctx.heap_size // gran) * gran
    token = ctx.comm.broadcast_object(uuid.uuid4().hex[:10], 0)

    handle, fd = ctypes.c_uint64(), ctypes.c_int(-1)
    _native.rt_check(rt.iris_rt_vmm_create(dev, h.stride, ctypes.byref(handle), ctypes.byref(fd)), "cuMemCreate")
    h._handles.append(handle.value)
    va = ctypes.c_uint64()
    h._va_bytes = h.stride * world
    _native.rt_check(rt.iris_rt_vmm_reserve(h._va_bytes, gran, ctypes.byref(va)), "cuMemAddressReserve")
    h._va = va.value
    fds = _exchange_fds(ctx, token, fd.value, "heap") if world > 1 else [fd.value]
    for r in range(world):
        if r == rank:
            hr = handle.value
        else:
            imp = ctypes.c_uint64()
            _native.rt_check(rt.iris_rt_vmm_import(fds[r], ctypes.byref(imp)), f"import heap of rank {r}")
            hr = imp.value
            h._handles.append(hr)
        at = h._va + r * h.stride
        _native.rt_check(rt.iris_rt_vmm_map(at, h.stride, hr, dev), f"map heap of rank {r}")
        h._mapped.append(at)
    for f in fds:
        if f >= 0:
            rt.iris_rt_fd_close(f)
    h.peer_ptrs = [h._va + r * h.stride for r in range(world)]
    h.own_ptr = h.peer_ptrs[rank]
    _native.rt_check(rt.iris_rt_memset(ctypes.c_void_p(h.own_ptr), 0, ctx.heap_size), "heap memset")

    if want_mc:
        try:
            _bind_multicast(ctx, h, token, handle.value)
        except RuntimeError as e:  # NVLS is an optimisation: every rank falls back to plain peer access
            ctx.log(f"NVLS multicast not available: {e}")
            h.release_multicast()
    ctx.comm.barrier()
    return h


def _agree(ctx, error: str, what: str) -> None:
    """Collective verdict on one step of the set-up: every rank contributes its error text (empty: fine) and all
    ranks raise together when any failed, so that no rank is left with a binding the others do not have."""
    got = ctx.comm.allgather_bytes(error.encode()[:240])
    bad = {r: b.decode(errors="replace") for r, b in enumerate(got) if b}
    if bad:
        first = sorted(bad)[0]
        raise RuntimeError(f"{what} failed on rank(s) {sorted(bad)}: {bad[first]}")


def _err(rt, rc: int) -> str:
    return "" if rc == 0 else (rt.iris_rt_last_error().decode() or f"error {rc}")


def _bind_multicast(ctx, h: VmmHeap, token: str, mem_handle: int) -> None:
    """Create the multicast object on rank 0, hand it to every rank, add every device, bind every heap and map the
    object.  Each step is followed by a collective verdict (which also serves as the barrier the driver API asks for
    between the steps): on any failure every rank raises, and the caller falls back to plain peer access everywhere."""
    rt = _native.runtime()
    rank, world, dev = ctx.cur_rank, ctx.num_ranks, ctx.gpu_id
    mc, fd = ctypes.c_uint64(0), ctypes.c_int(-1)
    err = ""
    if rank == 0:
        err = _err(rt, rt.iris_rt_multicast_create(world, h.stride, ctypes.byref(mc), ctypes.byref(fd)))
    _agree(ctx, err, "cuMulticastCreate")
    # rank 0 hands its descriptor to everyone; the others contribute a dummy (their heap fd is closed already)
    dummy = os.open("/dev/null", os.O_RDONLY)
    try:
        fds = _exchange_fds(ctx, token, fd.value if rank == 0 else dummy, "mc")
    finally:
        os.close(dummy)
    err = ""
    if rank != 0:
        err = _err(rt, rt.iris_rt_vmm_import(fds[0], ctypes.byref(mc)))
    for r, f in enumerate(fds):
        if f >= 0 and r != rank:
            rt.iris_rt_fd_close(f)
    if rank == 0:
        rt.iris_rt_fd_close(fd.value)
    if not err:
        h._mc_handle = mc.value
        err = _err(rt, rt.iris_rt_multicast_add_device(mc.value, dev))
    _agree(ctx, err, "import / cuMulticastAddDevice")   # every device has joined before anyone binds memory
    err = _err(rt, rt.iris_rt_multicast_bind(mc.value, mem_handle, h.stride))
    h._mc_bound = not err     # a rank whose bind worked must unbind when another rank's did not
    _agree(ctx, err, "cuMulticastBindMem")
    va = ctypes.c_uint64()
    err = _err(rt, rt.iris_rt_vmm_reserve(h.stride, h.stride if h.stride < (1 << 30) else (1 << 21), ctypes.byref(va)))
    if not err:
        err = _err(rt, rt.iris_rt_vmm_map(va.value, h.stride, mc.value, dev))
        if err:
            rt.iris_rt_vmm_address_free(va.value, h.stride)
        else:
            h._mc_va = va.value
    _agree(ctx, err, "map multicast object")
    h.mc_ptr = h._mc_va
