"""User-kernel compilation against the device header (the README example of the reference, README.md:31-70,
rewritten as a CUDA kernel).  Compiling needs no GPU; running the kernel does."""
import pytest
import torch

import iris_b200 as iris
from iris_b200 import jit

SRC = r'''
#include <iris/iris.cuh>
__global__ void put_value(float* buf, int n, float v, int cur, int dst, const uint64_t* heap_bases) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  iris::store(buf + i, v, cur, dst, heap_bases, i < n);
}
__global__ void count_all(int* counter, int cur, int world, const uint64_t* heap_bases) {
  for (int t = 0; t < world; ++t)
    iris::atomic_add<iris::Sem::relaxed, iris::Scope::sys>(counter, 1, cur, t, heap_bases);
}
extern "C" void launch_put_value(float* buf, int n, float v, int cur, int dst, const uint64_t* hb, void* stream) {
  put_value<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(buf, n, v, cur, dst, hb);
}
extern "C" void launch_count_all(int* counter, int cur, int world, const uint64_t* hb, void* stream) {
  count_all<<<1, 1, 0, (cudaStream_t)stream>>>(counter, cur, world, hb);
}
'''


def test_compile_and_cache(tmp_path, monkeypatch):
    monkeypatch.setenv("IRIS_JIT_CACHE", str(tmp_path))
    m1 = jit.compile(SRC, name="readme")
    assert m1.path.exists()
    m2 = jit.compile(SRC, name="readme")
    assert m2.path == m1.path and m2.log == ""  # second call hits the cache
    with pytest.raises(jit.JitError):
        m1.no_such_symbol
    with pytest.raises(jit.JitError):
        jit.compile("this is not CUDA", name="broken")


@pytest.mark.gpu
def test_readme_example_runs(tmp_path, monkeypatch):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    monkeypatch.setenv("IRIS_JIT_CACHE", str(tmp_path))
    mod = jit.compile(SRC, name="readme")
    ranks = iris.Iris.local_world(2, heap_size=1 << 22)
    bufs = [c.zeros(4096, dtype=torch.float32) for c in ranks]
    cnts = [c.zeros(1, dtype=torch.int32) for c in ranks]
    c0 = ranks[0]
    mod.launch_put_value(bufs[0], 4096, 1.0, 0, 1, c0.get_heap_bases(), mod.current_stream())
    for r, c in enumerate(ranks):
        mod.launch_count_all(cnts[r], r, 2, c.get_heap_bases(), mod.current_stream())
    torch.cuda.synchronize()
    assert float(bufs[1].sum()) == 4096.0 and float(bufs[0].sum()) == 0.0
    assert int(cnts[0][0]) == 2 and int(cnts[1][0]) == 2
    ranks[0].close()
