"""The pluggable device allocator (iris_b200/csrc/alloc/iris_allocator.cpp), counterpart of the reference's
fine-grained allocator plug-in (csrc/finegrained_alloc/finegrained_allocator.hip:27-56, installed by
iris/__init__.py:28-45).  On CPU: the exported ABI and the failure path (no device: null, no exit).  On a GPU, in a
child process because the allocator of a process can only be changed before its first CUDA allocation: torch tensors
come from the plug-in, the symmetric heap (which the native runtime allocates itself) works beside it, and
LOG_IRIS_ALLOCATOR switches the plug-in's log on."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

from iris_b200 import _build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    so = ctypes.CDLL(str(_build.build_all()["allocator"]))
    so.iris_malloc.argtypes = [ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
    so.iris_malloc.restype = ctypes.c_void_p
    so.iris_free.argtypes = [ctypes.c_void_p, ctypes.c_ssize_t, ctypes.c_int, ctypes.c_void_p]
    so.iris_free.restype = None
    return so


@pytest.mark.skipif(torch.cuda.is_available(), reason="failure path: needs a machine without a CUDA device")
def test_allocation_failure_returns_null_and_does_not_exit(capfd):
    so = _lib()
    p = so.iris_malloc(1 << 20, 0, None)
    assert not p
    assert "[iris allocator] cudaMalloc(1048576) on device 0 failed" in capfd.readouterr().err


CHILD = r"""
import ctypes, os, sys, torch
import iris_b200 as iris
from iris_b200 import _native
iris.install_allocator()
x = torch.ones(1 << 20, device="cuda")            # 4 MB: one call of the plug-in (torch does not cache plug-in memory)
assert float(x.sum()) == float(1 << 20)
so = ctypes.CDLL(str(_native.lib_path("allocator")))     # the instance torch loaded
so.iris_allocator_export_fd.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_size_t)]
mode = os.environ.get("IRIS_ALLOCATOR_MODE", "vmm")
nbytes = ctypes.c_size_t(0)
fd = so.iris_allocator_export_fd(ctypes.c_void_p(x.data_ptr()), ctypes.byref(nbytes))
if mode == "vmm":
    # the tensor's memory is a shareable VMM object: it exports as a file descriptor another process could map
    assert fd >= 0 and nbytes.value >= 4 << 20 and so.iris_allocator_vmm_live() >= 1, (fd, nbytes.value)
    os.close(fd)
else:
    assert fd == -1 and so.iris_allocator_vmm_live() == 0
ctx = iris.iris(1 << 24)
t = ctx.arange(0, 1024, dtype=torch.int32)
assert int(t.sum()) == 1023 * 1024 // 2
assert ctx.on_heap(t)
ctx.close()
del x, t
torch.cuda.synchronize()
print("allocator OK")
"""


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["vmm", "cudamalloc"])
@pytest.mark.parametrize("log", [False, True])
def test_torch_allocates_through_the_plugin(log, mode):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    env["IRIS_ALLOCATOR_MODE"] = mode
    env.pop("LOG_IRIS_ALLOCATOR", None)
    if log:
        env["LOG_IRIS_ALLOCATOR"] = "1"
    run = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, timeout=240, env=env, cwd=ROOT)
    assert run.returncode == 0, run.stdout + run.stderr
    assert "allocator OK" in run.stdout
    lines = [ln for ln in run.stderr.splitlines() if ln.startswith("[iris allocator]")]
    if log:
        assert any("malloc 4194304 bytes on device 0" in ln for ln in lines), run.stderr
        assert any(ln.startswith("[iris allocator] free") for ln in lines), run.stderr
    else:
        assert not lines, run.stderr
