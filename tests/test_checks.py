"""Checking pointer translation and repository hygiene.

The pool has no compute-sanitizer, so out-of-heap pointers and bad ranks are caught by ``iris::translate_checked``,
which records the violation in the status block and returns null instead of a pointer (nothing faults).  The same
header is exercised on the CPU here and, compiled for the GPU through ``iris_b200.jit``, in the gpu-marked test.
"""
import ctypes
import os
import re

import pytest
import torch

import iris_b200 as iris
from iris_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_translate_checked_cpu():
    ranks = iris.Iris.local_world(2, heap_size=1 << 16, backend="cpu")
    c = ranks[0]
    buf = c.zeros(16, dtype=torch.float32)
    lib = _native.cpu()
    hb = ctypes.c_void_p(c.get_heap_bases().data_ptr())
    st = ctypes.c_void_p(c.status_ptr())
    good = lib.iris_cpu_translate_checked(buf.data_ptr(), hb, c.heap_size, 0, 2, 1, st)
    assert good == ranks[1].heap_base() + c.offset_of(buf)
    c.check_status()
    assert lib.iris_cpu_translate_checked(buf.data_ptr() + c.heap_size, hb, c.heap_size, 0, 2, 1, st) == 0
    with pytest.raises(iris.IrisDeviceCheckError, match="'code': 2"):
        c.check_status()
    assert lib.iris_cpu_translate_checked(buf.data_ptr(), hb, c.heap_size, 0, 2, 5, st) == 0
    with pytest.raises(iris.IrisDeviceCheckError, match="'code': 3"):
        c.check_status()


CHECKED_SRC = r'''
#include <iris/iris.cuh>
__global__ void checked_store(float* buf, float v, int target, iris::Context c) {
  float* dst = iris::translate_checked(buf + threadIdx.x, c, target, 91);
  if (dst) *dst = v;   // a rejected pointer is skipped, never dereferenced
}
extern "C" void launch_checked_store(float* buf, float v, int target, const uint64_t* hb, unsigned long long heap_size,
                                     void* status, int rank, int world, void* stream) {
  iris::Context c{hb, heap_size, 0, (iris::StatusBlock*)status, rank, world};
  checked_store<<<1, 32, 0, (cudaStream_t)stream>>>(buf, v, target, c);
}
'''


@pytest.mark.gpu
def test_translate_checked_gpu(tmp_path, monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from iris_b200 import jit
    monkeypatch.setenv("IRIS_JIT_CACHE", str(tmp_path))
    mod = jit.compile(CHECKED_SRC, name="checked")
    ranks = iris.Iris.local_world(2, heap_size=1 << 20)
    c = ranks[0]
    bufs = [r.zeros(32, dtype=torch.float32) for r in ranks]
    args = (c.get_heap_bases(), ctypes.c_uint64(c.heap_size), ctypes.c_void_p(c.status_ptr()), 0, 2, mod.current_stream())
    mod.launch_checked_store(bufs[0], 3.0, 1, *args)
    torch.cuda.synchronize()
    c.check_status()
    assert float(bufs[1].sum()) == 96.0
    outside = torch.zeros(32, device="cuda")              # not on the heap: rejected, untouched
    mod.launch_checked_store(outside, 5.0, 1, *args)
    torch.cuda.synchronize()
    with pytest.raises(iris.IrisDeviceCheckError):
        c.check_status()
    assert float(outside.sum()) == 0.0
    mod.launch_checked_store(bufs[0], 5.0, 7, *args)      # rank 7 does not exist
    torch.cuda.synchronize()
    with pytest.raises(iris.IrisDeviceCheckError):
        c.check_status()
    ranks[0].close()


def test_every_tma_load_is_per_cta():
    """No TMA / bulk load carries the cluster-wide delivery qualifier in any source file of the package."""
    # the qualifier is spelled in two pieces so that this test file does not itself contain it
    pat = re.compile(r"cp\.async\.bulk[^\n]*" + "multi" + "cast::cluster")
    bad = []
    for base, _, files in os.walk(os.path.join(ROOT, "iris_b200")):
        if os.sep + "build" in base or os.sep + "lib" in base:
            continue
        for f in files:
            if f.endswith((".cu", ".cuh", ".cpp", ".h", ".py")):
                text = open(os.path.join(base, f), errors="replace").read()
                if pat.search(text):
                    bad.append(os.path.join(base, f))
    assert not bad, bad


def test_no_triton_in_product():
    for base, _, files in os.walk(os.path.join(ROOT, "iris_b200")):
        for f in files:
            if f.endswith(".py"):
                text = open(os.path.join(base, f)).read()
                assert "import triton" not in text, os.path.join(base, f)
