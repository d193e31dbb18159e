"""ctypes access to the in-tree native libraries (``iris_b200/lib/*.so``).

The libraries are built by :mod:`iris_b200._build`.  Loading is lazy; a missing library raises with the
command that builds it (the reference raises at import when its allocator library is missing,
``iris/__init__.py:29-38``).
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, c_char_p, c_double, c_int, c_int64, c_uint32, c_uint64, c_void_p)
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "lib"
_cache = {}


class NativeLibraryMissing(RuntimeError):
    pass


def lib_path(name: str) -> Path:
    return LIB_DIR / f"libiris_{name}.so"


def _load(name: str) -> ctypes.CDLL:
    if name in _cache:
        return _cache[name]
    path = lib_path(name)
    if not path.exists():
        raise NativeLibraryMissing(
            f"{path} not found; build the native code first: python -m iris_b200._build")
    lib = ctypes.CDLL(str(path))
    _cache[name] = lib
    return lib


def cpu() -> ctypes.CDLL:
    lib = _load("cpu")
    if not getattr(lib, "_iris_typed", False):
        lib.iris_cpu_last_error.restype = c_char_p
        lib.iris_cpu_heap_map.restype = c_void_p
        lib.iris_cpu_heap_map.argtypes = [c_char_p, c_uint64, c_int]
        lib.iris_cpu_heap_unmap.argtypes = [c_void_p, c_uint64]
        lib.iris_cpu_heap_unlink.argtypes = [c_char_p]
        lib.iris_cpu_rma.restype = c_int
        lib.iris_cpu_rma.argtypes = [c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_void_p,
                                     c_int, c_int, c_int, c_double, c_int64, c_int64, c_int]
        lib.iris_cpu_mp_produce.restype = None
        lib.iris_cpu_mp_produce.argtypes = [c_void_p, c_void_p, c_uint64, c_void_p, c_uint32, c_void_p, c_int, c_int]
        lib.iris_cpu_translate_checked.restype = c_uint64
        lib.iris_cpu_translate_checked.argtypes = [c_uint64, c_void_p, c_uint64, c_int, c_int, c_int, c_void_p]
        lib.iris_cpu_wait_flag.restype = c_uint32
        lib.iris_cpu_wait_flag.argtypes = [c_void_p, c_uint32, c_uint64, c_void_p, c_uint32]
        lib._iris_typed = True
    return lib


def runtime() -> ctypes.CDLL:
    lib = _load("runtime")
    if not getattr(lib, "_iris_typed", False):
        lib.iris_rt_last_error.restype = c_char_p
        lib.iris_rt_malloc.argtypes = [c_int, c_uint64, POINTER(c_void_p)]
        lib.iris_rt_free.argtypes = [c_void_p]
        lib.iris_rt_memset.argtypes = [c_void_p, c_int, c_uint64]
        lib.iris_rt_ipc_get_handle.argtypes = [c_void_p, c_void_p]
        lib.iris_rt_ipc_open_handle.argtypes = [c_void_p, POINTER(c_void_p)]
        lib.iris_rt_ipc_close_handle.argtypes = [c_void_p]
        lib.iris_rt_memcpy_h2d.argtypes = [c_void_p, c_void_p, c_uint64]
        lib.iris_rt_memcpy_d2h.argtypes = [c_void_p, c_void_p, c_uint64]
        lib.iris_rt_vmm_granularity.restype = c_int64
        lib.iris_rt_vmm_create.argtypes = [c_int, c_uint64, POINTER(c_uint64), POINTER(c_int)]
        lib.iris_rt_vmm_import.argtypes = [c_int, POINTER(c_uint64)]
        lib.iris_rt_vmm_release.argtypes = [c_uint64]
        lib.iris_rt_vmm_reserve.argtypes = [c_uint64, c_uint64, POINTER(c_uint64)]
        lib.iris_rt_vmm_address_free.argtypes = [c_uint64, c_uint64]
        lib.iris_rt_vmm_map.argtypes = [c_uint64, c_uint64, c_uint64, c_int]
        lib.iris_rt_vmm_unmap.argtypes = [c_uint64, c_uint64]
        lib.iris_rt_multicast_granularity.restype = c_int64
        lib.iris_rt_multicast_granularity.argtypes = [c_int, c_uint64]
        lib.iris_rt_multicast_create.argtypes = [c_int, c_uint64, POINTER(c_uint64), POINTER(c_int)]
        lib.iris_rt_multicast_add_device.argtypes = [c_uint64, c_int]
        lib.iris_rt_multicast_bind.argtypes = [c_uint64, c_uint64, c_uint64]
        lib.iris_rt_multicast_unbind.argtypes = [c_uint64, c_int, c_uint64]
        lib.iris_rt_fd_listen.argtypes = [c_char_p]
        lib.iris_rt_fd_send.argtypes = [c_char_p, c_int, c_int]
        lib.iris_rt_fd_recv.argtypes = [c_int, c_int, POINTER(c_int)]
        lib._iris_typed = True
    return lib


class RuntimeCallError(RuntimeError):
    """A CUDA runtime/driver call made by the native runtime failed (reference: ``hip_try`` raising
    RuntimeError, ``iris/_hip.py:12-16``)."""


def rt_check(rc: int, what: str = "") -> None:
    if rc != 0:
        msg = runtime().iris_rt_last_error().decode(errors="replace")
        raise RuntimeCallError(f"{what or 'runtime call'} failed: {msg}")


def kernels() -> ctypes.CDLL:
    return _load("kernels")


def kernels_available() -> bool:
    return lib_path("kernels").exists()
