"""Symmetric-heap context: the host API.

Role in the reference: ``class Iris`` and ``iris()`` in ``iris/iris.py:31-314,524-534``.  The surface is kept
(``get_rank``, ``get_num_ranks``, ``get_heap_bases``, ``barrier``, ``broadcast``, the torch-like tensor
factories that allocate on the heap, ``log*``); the machinery underneath is different:

* the heap is one ``cudaMalloc`` (or CUDA-VMM) region per GPU obtained from the native runtime
  (``csrc/runtime/iris_runtime.cpp``) and wrapped as a torch tensor without going through torch's
  caching allocator, so its base address is the address that is exported;
* peers are mapped with CUDA IPC handles (or imported VMM handles passed as file descriptors) that
  travel over a gloo control plane (``parallel/bootstrap.py``) instead of MPI;
* without a GPU the heap is a POSIX shared-memory segment and the same API runs on CPU ranks
  (``csrc/cpu/iris_cpu_backend.cpp``);
* ``Iris.local_world`` creates several ranks inside ONE process on ONE device — every fused kernel can
  then be launched once over all ranks' data, which is how multi-rank logic is tested on a single GPU.
"""
from __future__ import annotations

import ctypes
import math
import os
import uuid
from typing import List, Optional

import numpy as np
import torch

from . import _native
from .parallel import bootstrap as _bs

# Module-level switches, as in the reference (iris/iris.py:26-28).
STATS = True
LOGGING = True
DEBUG = False

# IRIS_LOG presets them: quiet (nothing), stats (log_stats only), info (log + log_stats, the default), debug (all).
_LOG_LEVELS = {"quiet": (False, False, False), "stats": (True, False, False), "info": (True, True, False),
               "debug": (True, True, True)}


def set_log_level(level: str) -> None:
    """Set the three switches at once: ``quiet``, ``stats``, ``info`` or ``debug``."""
    global STATS, LOGGING, DEBUG
    try:
        STATS, LOGGING, DEBUG = _LOG_LEVELS[level.lower()]
    except KeyError:
        raise ValueError(f"IRIS_LOG / set_log_level: {level!r} is not one of {sorted(_LOG_LEVELS)}") from None


if os.environ.get("IRIS_LOG"):
    set_log_level(os.environ["IRIS_LOG"])

STATUS_BYTES = 1024  # first allocation of every heap: the kernel status block (see iris.cuh StatusBlock)


class IrisTimeoutError(RuntimeError):
    """A bounded device-side wait expired; carries the decoded status block."""


class IrisDeviceCheckError(RuntimeError):
    """A checking build of a kernel recorded a bad pointer or rank."""


class IrisHeapCorruption(RuntimeError):
    """Debug heap: the guard bytes behind an allocation were overwritten."""


class IrisDivergenceError(RuntimeError):
    """Debug heap: the ranks did not make the same sequence of allocations, so equal offsets name different objects."""


CANARY = 0xA5        # guard byte of the debug heap


class _DeviceMemory:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can wrap it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


def _element_size(dtype: torch.dtype) -> int:
    return torch.empty((), dtype=dtype).element_size()


class Iris:
    """One rank's view of the symmetric heap.

    Args:
        heap_size: bytes of symmetric heap per rank (default 1 GiB, as ``iris/iris.py:32``).
        bootstrap: control-plane back end; default :func:`parallel.bootstrap.init_from_env`.
        backend: ``"cuda"`` or ``"cpu"``; default ``"cuda"`` when a GPU is visible.
        heap_mode: ``"ipc"`` (cudaMalloc + CUDA IPC, default) or ``"vmm"`` (CUDA virtual memory management
            with file-descriptor export; required for NVLS multicast).  Env ``IRIS_HEAP_MODE`` overrides.
        debug_heap: guard every allocation with ``alignment`` bytes of a known pattern and keep a record of the
            allocation sequence; :meth:`barrier` then checks the guards (``IrisHeapCorruption``) and that every rank
            allocated the same sequence (``IrisDivergenceError``).  Default: env ``IRIS_DEBUG_HEAP=1``.  Every rank
            must use the same setting (checked).  The reference has neither check: a divergent allocation there
            silently makes ``translate`` point at another object.
    """

    def __init__(self, heap_size: int = 1 << 30, *, bootstrap: Optional[_bs.Bootstrap] = None,
                 backend: Optional[str] = None, heap_mode: Optional[str] = None, debug_heap: Optional[bool] = None,
                 _local=None):
        self.alignment = 1024
        if debug_heap is None:
            debug_heap = os.environ.get("IRIS_DEBUG_HEAP", "0") not in ("", "0")
        self.debug_heap = bool(debug_heap)
        self._allocs: List[tuple] = []   # debug heap: (start, bytes asked for, bytes taken incl. guard, dtype name)
        self.heap_size = int(heap_size)
        self.heap_offset = 0
        self._closed = False
        self._peer_ptrs: List[int] = []
        self._opened_ipc: List[int] = []
        self._shm_names: List[str] = []
        self._shm_maps: List[tuple] = []
        self._own_ptr = 0
        self._vmm = None
        self.mc_base = 0  # NVLS multicast address of the heap (0: not bound)
        if backend is None:
            backend = "cuda" if torch.cuda.is_available() else "cpu"
        if backend not in ("cuda", "cpu"):
            raise ValueError(f"unknown backend {backend!r}")
        self.backend = backend
        self.heap_mode = (heap_mode or os.environ.get("IRIS_HEAP_MODE", "ipc")).lower()

        if _local is not None:  # rank of an in-process world: memory is set up by local_world()
            self.comm = _local["comm"]
            self.cur_rank, self.num_ranks = _local["rank"], _local["world"]
            self.gpu_id = _local["gpu_id"]
            self.device = _local["device"]
            self.memory_pool = _local["pool"]
            self.heap_bases = _local["heap_bases"]
            self._own_ptr = _local["ptr"]
            self._peer_ptrs = _local["ptrs"]
            self._local_world = _local["members"]
            self._init_status()
            return

        self._local_world = None
        self.comm = bootstrap if bootstrap is not None else _bs.init_from_env()
        self.cur_rank, self.num_ranks = self.comm.rank, self.comm.world
        # every rank must ask for the same heap size, otherwise equal offsets would not name equal objects
        hello = self.heap_size.to_bytes(8, "little") + bytes([int(self.debug_heap)])
        hellos = self.comm.allgather_bytes(hello)
        sizes = [int.from_bytes(b[:8], "little") for b in hellos]
        if any(s != self.heap_size for s in sizes):
            raise ValueError(f"heap_size differs across ranks: {sizes}")
        if any(b[8] != int(self.debug_heap) for b in hellos):
            raise ValueError(f"debug_heap differs across ranks: {[bool(b[8]) for b in hellos]}")
        if backend == "cuda":
            self._init_cuda()
        else:
            self._init_cpu()
        self._init_status()
        self.comm.barrier()

    # ------------------------------------------------------------------------------------------
    # construction
    # ------------------------------------------------------------------------------------------
    def _init_cuda(self) -> None:
        rt = _native.runtime()
        n_dev = rt.iris_rt_device_count()
        if n_dev <= 0:
            raise RuntimeError("backend='cuda' but no CUDA device is visible")
        self.gpu_id = self.comm.local_rank() % n_dev  # reference: rank % num_gpus, iris/iris.py:35-38
        torch.cuda.set_device(self.gpu_id)
        _native.rt_check(rt.iris_rt_set_device(self.gpu_id), "set_device")
        self.device = torch.device("cuda", self.gpu_id)
        if self.heap_mode == "vmm" and self.num_ranks >= 1:
            from .parallel import vmm_heap
            self._vmm = vmm_heap.create(self)
            self._own_ptr = self._vmm.own_ptr
            self._peer_ptrs = self._vmm.peer_ptrs
            self.mc_base = self._vmm.mc_ptr
        else:
            self.heap_mode = "ipc"
            p = ctypes.c_void_p()
            _native.rt_check(rt.iris_rt_malloc(self.gpu_id, self.heap_size, ctypes.byref(p)), "heap cudaMalloc")
            self._own_ptr = int(p.value)
            _native.rt_check(rt.iris_rt_memset(p, 0, self.heap_size), "heap memset")
            handle = (ctypes.c_ubyte * rt.iris_rt_ipc_handle_size())()
            if self.num_ranks > 1:
                _native.rt_check(rt.iris_rt_ipc_get_handle(p, handle), "cudaIpcGetMemHandle")
            handles = self.comm.allgather_bytes(bytes(handle))
            ptrs = []
            for r, h in enumerate(handles):  # reference: open every peer handle, own slot = own base (iris.py:65-71)
                if r == self.cur_rank:
                    ptrs.append(self._own_ptr)
                    continue
                q = ctypes.c_void_p()
                buf = (ctypes.c_ubyte * len(h)).from_buffer_copy(h)
                _native.rt_check(rt.iris_rt_ipc_open_handle(buf, ctypes.byref(q)), f"cudaIpcOpenMemHandle(rank {r})")
                ptrs.append(int(q.value))
                self._opened_ipc.append(int(q.value))
            self._peer_ptrs = ptrs
        self.memory_pool = torch.as_tensor(_DeviceMemory(self._own_ptr, self.heap_size), device=self.device)
        bases = np.array(self._peer_ptrs, dtype=np.uint64)
        self.heap_bases = torch.from_numpy(bases).to(self.device)

    def _init_cpu(self) -> None:
        lib = _native.cpu()
        self.gpu_id = -1
        self.device = torch.device("cpu")
        token = self.comm.broadcast_object(uuid.uuid4().hex[:12], 0)
        names = [f"/iris_b200_{token}_{r}" for r in range(self.num_ranks)]
        own = lib.iris_cpu_heap_map(names[self.cur_rank].encode(), self.heap_size, 1)
        if not own:
            raise RuntimeError("shared-memory heap: " + lib.iris_cpu_last_error().decode())
        self._shm_names = [names[self.cur_rank]]
        self._own_ptr = int(own)
        ctypes.memset(own, 0, self.heap_size)
        self.comm.barrier()
        ptrs = []
        for r, name in enumerate(names):
            if r == self.cur_rank:
                ptrs.append(self._own_ptr)
                continue
            p = lib.iris_cpu_heap_map(name.encode(), self.heap_size, 0)
            if not p:
                raise RuntimeError(f"attach to rank {r}'s heap: " + lib.iris_cpu_last_error().decode())
            ptrs.append(int(p))
            self._shm_maps.append((int(p), self.heap_size))
        self._peer_ptrs = ptrs
        buf = (ctypes.c_ubyte * self.heap_size).from_address(self._own_ptr)
        self.memory_pool = torch.frombuffer(buf, dtype=torch.uint8)
        self.heap_bases = torch.from_numpy(np.array(ptrs, dtype=np.uint64))
        self.comm.barrier()
        # every rank has attached: the names can go, the mappings stay until close()
        lib.iris_cpu_heap_unlink(names[self.cur_rank].encode())
        self._shm_names = []

    def _init_status(self) -> None:
        self.status = self.allocate(STATUS_BYTES // 4, torch.int32)
        self.status.zero_()
        self._base_mark = self.heap_offset   # everything below belongs to the context itself

    @classmethod
    def local_world(cls, world: int, heap_size: int = 1 << 26, backend: Optional[str] = None,
                    device: Optional[int] = None, debug_heap: Optional[bool] = None) -> List["Iris"]:
        """Create ``world`` ranks inside this process, all on one device (or all on the CPU).

        Their heaps are separate allocations and the base-address table lists all of them, so pointer
        translation, flags and pushes behave exactly as between GPUs; only the transport is local.  A kernel
        that involves several ranks must then be launched ONCE for all of them (kernels that wait on one
        another may not run as separate launches on one GPU).
        """
        if backend is None:
            backend = "cuda" if torch.cuda.is_available() else "cpu"
        comm = _bs.SingleBootstrap()
        pools, ptrs = [], []
        if backend == "cuda":
            gpu_id = torch.cuda.current_device() if device is None else device
            dev = torch.device("cuda", gpu_id)
            rt = _native.runtime()
            _native.rt_check(rt.iris_rt_set_device(gpu_id), "set_device")
            for _ in range(world):
                p = ctypes.c_void_p()
                _native.rt_check(rt.iris_rt_malloc(gpu_id, heap_size, ctypes.byref(p)), "heap cudaMalloc")
                _native.rt_check(rt.iris_rt_memset(p, 0, heap_size), "heap memset")
                ptrs.append(int(p.value))
                pools.append(torch.as_tensor(_DeviceMemory(int(p.value), heap_size), device=dev))
            bases = torch.from_numpy(np.array(ptrs, dtype=np.uint64)).to(dev)
        else:
            gpu_id, dev = -1, torch.device("cpu")
            for _ in range(world):
                t = torch.zeros(heap_size, dtype=torch.uint8)
                pools.append(t)
                ptrs.append(t.data_ptr())
            bases = torch.from_numpy(np.array(ptrs, dtype=np.uint64))
        members: List[Iris] = []
        for r in range(world):
            members.append(cls(heap_size, backend=backend, debug_heap=debug_heap, _local=dict(
                comm=comm, rank=r, world=world, gpu_id=gpu_id, device=dev, pool=pools[r], heap_bases=bases,
                ptr=ptrs[r], ptrs=ptrs, members=members)))
        members[0]._owns_local = True
        return members

    # ------------------------------------------------------------------------------------------
    # logging — reference: iris/iris.py:81-91
    # ------------------------------------------------------------------------------------------
    def log(self, message):
        if LOGGING:
            print(f"[Iris] [{self.cur_rank}/{self.num_ranks}] {message}", flush=True)

    def log_debug(self, message):
        if DEBUG:
            print(f"[Iris] [{self.cur_rank}/{self.num_ranks}] {message}", flush=True)

    def log_stats(self, message):
        if STATS:
            print(f"[Iris] [{self.cur_rank}/{self.num_ranks}] {message}", flush=True)

    # ------------------------------------------------------------------------------------------
    # queries and synchronisation — reference: iris/iris.py:93-94, 269-291
    # ------------------------------------------------------------------------------------------
    def broadcast(self, value, root=0):
        """Return ``value`` as held by rank ``root`` on every rank (call order as the reference's call sites,
        ``examples/00_load/load_bench.py:165``)."""
        if self._local_world is not None:
            return value
        return self.comm.broadcast_object(value, int(root))

    def get_heap_bases(self) -> torch.Tensor:
        return self.heap_bases

    def heap_base(self, rank: Optional[int] = None) -> int:
        return self._peer_ptrs[self.cur_rank if rank is None else rank]

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        """Wait for this rank's device work, then for every rank (``iris/iris.py:272-276``)."""
        if self.backend == "cuda":
            torch.cuda.synchronize(self.device)
        if self.debug_heap:
            self.check_heap()
        if self._local_world is None:
            self.comm.barrier(timeout_s)

    def get_device(self) -> torch.device:
        return self.memory_pool.device

    def get_cu_count(self) -> int:
        """Number of SMs of this rank's GPU (148 on B200); the reference returns compute units."""
        if self.backend == "cuda":
            return _native.runtime().iris_rt_sm_count(self.gpu_id)
        return os.cpu_count() or 1

    def get_rank(self) -> int:
        return self.cur_rank

    def get_num_ranks(self) -> int:
        return self.num_ranks

    def wall_clock_rate(self, rank: int = 0) -> int:
        """kHz of the device timer read by ``iris::globaltimer()`` (1 GHz nanosecond counter)."""
        return 1_000_000

    # ------------------------------------------------------------------------------------------
    # allocation — reference: iris/iris.py:96-116, 266-267
    # ------------------------------------------------------------------------------------------
    def allocate(self, num_elements: int, dtype: torch.dtype) -> torch.Tensor:
        self.log_debug(f"allocate: num_elements = {num_elements}, dtype = {dtype}")
        size_in_bytes = int(num_elements) * _element_size(dtype)
        aligned = math.ceil(size_in_bytes / self.alignment) * self.alignment
        if self.debug_heap:
            aligned += self.alignment  # guard bytes behind the allocation (and in its alignment slack)
        if self.heap_offset + aligned > self.heap_size:
            raise MemoryError("Heap out of memory")
        start = self.heap_offset
        self.heap_offset += aligned
        if self.debug_heap:
            guard0 = start + (size_in_bytes + 15) // 16 * 16   # kernels may round a store up to 16 bytes
            self.memory_pool[guard0:start + aligned] = CANARY
            self._allocs.append((start, size_in_bytes, aligned, str(dtype)))
        return self.memory_pool[start:start + size_in_bytes].view(dtype).reshape((int(num_elements),))

    def deallocate(self, pointer) -> None:
        """No-op, as in the reference: the heap is a bump allocator."""

    def mark(self) -> int:
        """Current top of the bump allocator; pass it to :meth:`reset` to free everything allocated after it."""
        return self.heap_offset

    def reset(self, to: Optional[int] = None) -> None:
        """Rewind the bump allocator to ``to`` (a value from :meth:`mark`; default: just above the status block).
        Every rank must do so at the same point of its allocation sequence."""
        to = self._base_mark if to is None else int(to)
        if not self._base_mark <= to <= self.heap_offset:
            raise ValueError("reset target is not a mark of this heap")
        self.heap_offset = to
        self._allocs = [a for a in self._allocs if a[0] < to]

    def allocation_digest(self) -> tuple:
        """(number of allocations, CRC of their sizes and dtypes): equal on every rank of a correct program.  Only
        kept by the debug heap."""
        import zlib
        crc = 0
        for _, size, taken, dt in self._allocs:
            crc = zlib.crc32(f"{size}:{taken}:{dt};".encode(), crc)
        return len(self._allocs), crc

    def check_heap(self) -> None:
        """Debug heap: verify the guard bytes of every allocation of this rank, then that all ranks made the same
        allocations.  Called by :meth:`barrier`; collective when the world has more than one process."""
        if not self.debug_heap:
            return
        overrun = ""
        for idx, (start, size, taken, dt) in enumerate(self._allocs):
            guard = self.memory_pool[start + (size + 15) // 16 * 16:start + taken]
            bad = (guard != CANARY).nonzero()
            if bad.numel():
                first = int(bad[0]) + (size + 15) // 16 * 16
                overrun = (f"rank {self.cur_rank}: allocation #{idx} ({size} bytes of {dt} at heap offset {start}) was "
                           f"overrun: byte {first - size} past its end is 0x{int(guard[int(bad[0])]):02x}")
                break
        mine = self.allocation_digest()
        if self._local_world is not None:
            if overrun:
                raise IrisHeapCorruption(overrun)
            theirs = [m.allocation_digest() for m in self._local_world]
        else:
            # the verdict travels with the digest, so that every rank leaves this collective the same way
            blob = mine[0].to_bytes(8, "little") + mine[1].to_bytes(4, "little") + bytes([1 if overrun else 0])
            got = self.comm.allgather_bytes(blob)
            theirs = [(int.from_bytes(b[:8], "little"), int.from_bytes(b[8:12], "little")) for b in got]
            hit = [r for r, b in enumerate(got) if b[12]]
            if overrun:
                raise IrisHeapCorruption(overrun)
            if hit:
                raise IrisHeapCorruption(f"rank {self.cur_rank}: guard bytes were overwritten on rank(s) {hit}")
        if any(t != mine for t in theirs):
            raise IrisDivergenceError(
                f"rank {self.cur_rank}: allocation sequences differ across ranks (count, digest per rank): {theirs}")

    def parse_size(self, size):
        if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
            size = tuple(size[0])
        return tuple(size), math.prod(size)

    def offset_of(self, tensor: torch.Tensor) -> int:
        """Byte offset of a heap tensor from the heap base (the rank-independent name of the object)."""
        off = tensor.data_ptr() - self._own_ptr
        if not 0 <= off < self.heap_size:
            raise RuntimeError("tensor is not on this rank's symmetric heap")
        return off

    def on_heap(self, tensor: torch.Tensor) -> bool:
        return tensor.device == self.memory_pool.device and 0 <= tensor.data_ptr() - self._own_ptr < self.heap_size

    def _check_out(self, tensor: torch.Tensor, num_elements: int, dtype: torch.dtype) -> None:
        if tensor.device != self.memory_pool.device:
            raise RuntimeError(f"The output tensor is on {tensor.device}, the heap is on {self.memory_pool.device}")
        if not self.on_heap(tensor):
            raise RuntimeError("The output tensor is not on the symmetric heap")
        if tensor.numel() != num_elements:
            raise RuntimeError(f"The output tensor has {tensor.numel()} elements, but {num_elements} are required")
        if tensor.dtype != dtype:
            raise RuntimeError(f"The output tensor has dtype {tensor.dtype}, but {dtype} is required")

    # ------------------------------------------------------------------------------------------
    # torch-like factories on the heap — reference: iris/iris.py:118-264
    # ------------------------------------------------------------------------------------------
    def zeros_like(self, tensor: torch.Tensor) -> torch.Tensor:
        """1-D zero tensor with ``tensor.numel()`` elements (the reference flattens, iris.py:118-123)."""
        t = self.allocate(tensor.numel(), tensor.dtype)
        t.zero_()
        return t

    def arange(self, start=0, end=None, step=1, out=None, dtype=None, layout=torch.strided, device=None,
               requires_grad=False):
        if end is None:
            start, end = 0, start
        n = math.ceil((end - start) / step)
        if dtype is None:
            dtype = torch.get_default_dtype() if any(isinstance(x, float) for x in (start, end, step)) else torch.int64
        if out is not None:
            self._check_out(out, n, dtype)
            t = out
        else:
            t = self.allocate(n, dtype)
        t[:] = torch.arange(start, end, step, dtype=dtype, device=self.memory_pool.device)
        if requires_grad:
            t.requires_grad_()
        return t

    def zeros(self, *size, dtype=torch.int, device=None, requires_grad=False, **kwargs):
        size, n = self.parse_size(size)
        t = self.allocate(n, dtype)
        t.zero_()
        if requires_grad:
            t.requires_grad_()
        return t.reshape(size)

    def randn(self, *size, generator=None, dtype=torch.float, layout=torch.strided, device=None,
              requires_grad=False, pin_memory=False):
        """Normal samples generated by torch on ``device`` (default: the heap's device) and copied into the
        heap; with equal seeds every rank holds identical data (``iris/iris.py:175-194``)."""
        size, n = self.parse_size(size)
        t = self.allocate(n, dtype)
        src_dev = self.memory_pool.device if device is None else device
        t.copy_(torch.randn(n, generator=generator, dtype=dtype, device=src_dev))
        if requires_grad:
            t.requires_grad_()
        return t.reshape(size)

    def ones(self, *size, out=None, dtype=None, layout=torch.strided, device=None, requires_grad=False):
        if dtype is None:
            dtype = torch.get_default_dtype()
        size, n = self.parse_size(size)
        if out is not None:
            self._check_out(out, n, dtype)
            t = out
        else:
            t = self.allocate(n, dtype)
        t.fill_(1)
        if requires_grad:
            t.requires_grad_()
        return t.reshape(size)

    def full(self, size, fill_value, dtype=torch.int):
        size, n = self.parse_size((size,) if isinstance(size, int) else (size,))
        t = self.allocate(n, dtype)
        t.fill_(fill_value)
        return t.reshape(size)

    def uniform(self, size, low=0.0, high=1.0, dtype=torch.float):
        size, n = self.parse_size((size,))
        t = self.allocate(n, dtype)
        t.uniform_(low, high)
        return t.reshape(size)

    def empty(self, size, dtype=torch.float):
        size, n = self.parse_size((size,))
        return self.allocate(n, dtype).reshape(size)

    def randint(self, size, low, high, dtype=torch.int):
        size, n = self.parse_size((size,))
        t = self.allocate(n, dtype)
        t[:] = torch.randint(low, high, (n,), device=self.memory_pool.device, dtype=dtype)
        return t.reshape(size)

    def linspace(self, start, end, steps, dtype=torch.float):
        """``steps`` evenly spaced values (the reference's version fails on an int ``steps``, iris.py:259-264)."""
        t = self.allocate(int(steps), dtype)
        t[:] = torch.linspace(start, end, int(steps), dtype=dtype, device=self.memory_pool.device)
        return t

    # ------------------------------------------------------------------------------------------
    # kernel status block
    # ------------------------------------------------------------------------------------------
    def status_ptr(self) -> int:
        return self.status.data_ptr()

    def check_status(self, clear: bool = True) -> None:
        """Raise if a kernel recorded a time-out or a bad pointer in this rank's status block."""
        words = self.status[:8].cpu().numpy().astype(np.uint32)
        code = int(words[0])
        if code == 0:
            return
        value = int(words[4]) | (int(words[5]) << 32)
        aux = int(words[6]) | (int(words[7]) << 32)
        info = dict(code=code, where=int(words[1]), rank=int(words[2]), detail=int(words[3]), value=value, aux=aux)
        if clear:
            self.status.zero_()
        if code == 1:
            raise IrisTimeoutError(f"device wait timed out: {info}")
        raise IrisDeviceCheckError(f"device check failed: {info}")

    # ------------------------------------------------------------------------------------------
    # teardown
    # ------------------------------------------------------------------------------------------
    def close(self) -> None:
        if self._closed:
            return
        self._closed = True
        try:
            if self.backend == "cuda":
                torch.cuda.synchronize(self.device)
                rt = _native.runtime()
                if self._local_world is not None:
                    if getattr(self, "_owns_local", False):
                        for m in self._local_world:
                            m.memory_pool = None
                        for p in self._peer_ptrs:
                            rt.iris_rt_free(ctypes.c_void_p(p))
                    return
                self.memory_pool = None
                if self._vmm is not None:
                    self._vmm.close()
                    return
                for p in self._opened_ipc:
                    rt.iris_rt_ipc_close_handle(ctypes.c_void_p(p))
                if self._own_ptr:
                    rt.iris_rt_free(ctypes.c_void_p(self._own_ptr))
            elif self._local_world is None:
                lib = _native.cpu()
                self.memory_pool = None
                for p, n in self._shm_maps:
                    lib.iris_cpu_heap_unmap(ctypes.c_void_p(p), n)
                if self._own_ptr:
                    lib.iris_cpu_heap_unmap(ctypes.c_void_p(self._own_ptr), self.heap_size)
                for name in self._shm_names:
                    lib.iris_cpu_heap_unlink(name.encode())
        except Exception:  # teardown must not mask the error that led here
            pass
        finally:
            if self._local_world is None:
                try:
                    self.comm.shutdown()
                except Exception:
                    pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False


def iris(heap_size: int = 1 << 30, **kwargs) -> Iris:
    """Create the symmetric-heap context (``iris/iris.py:524-534``)."""
    return Iris(heap_size, **kwargs)
