"""iris_b200 — a symmetric-heap RMA framework for one box of NVIDIA B200 GPUs (NVLink 5 / NVSwitch).

Host surface as the reference package (``iris/__init__.py:9-26,47-61``): ``iris(heap_size)`` / ``Iris`` with
torch-like factories on the heap, ``do_bench``, ``memset_tensor``; the device functions ``load``, ``store``,
``get``, ``put``, ``atomic_add``, ``atomic_sub``, ``atomic_cas``, ``atomic_xchg`` are C++ (``include/iris/iris.cuh``)
and are exposed here as element-wise host entry points for tests and small scripts.  Unlike the reference,
importing the package has no side effect on torch's allocator; ``install_allocator()`` opts in.
"""
from __future__ import annotations

from . import _native
from .context import (Iris, IrisDeviceCheckError, IrisTimeoutError, iris)  # noqa: F401
from .ops.rma import (atomic_add, atomic_cas, atomic_sub, atomic_xchg, get, load, put, store)  # noqa: F401
from .utils.bench import do_bench, memset_tensor  # noqa: F401

__version__ = "0.1.0"


def translate(ptr: int, cur_rank: int, target_rank: int, heap_bases) -> int:
    """Host mirror of ``iris::translate``: rebase an address of ``cur_rank``'s heap into ``target_rank``'s."""
    return int(heap_bases[target_rank]) + (int(ptr) - int(heap_bases[cur_rank]))


def include_dir() -> str:
    """Directory to pass to nvcc with ``-I`` so that user kernels can ``#include <iris/iris.cuh>``."""
    import os
    return os.path.join(os.path.dirname(__file__), "include")


def install_allocator():
    """Route every torch CUDA allocation of this process through the native pluggable allocator
    (what ``import iris`` does unconditionally in the reference, ``iris/__init__.py:40-45``).
    Must be called before the first CUDA allocation."""
    import torch
    path = _native.lib_path("allocator")
    if not path.exists():
        raise _native.NativeLibraryMissing(f"{path} not found; run python -m iris_b200._build")
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(path), "iris_malloc", "iris_free")
    torch.cuda.memory.change_current_allocator(alloc)
    return alloc
