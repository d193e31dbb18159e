"""The GEMM entry point for callers that may not allocate device memory (``csrc/kernels/gemm_noalloc.h``).

Some callers — a plug-in running inside another framework's step, a server that has given all its memory to a
pool, anything that must not provoke the device-wide stall of ``cudaMalloc`` — can pass buffers they own but
cannot supply a kernel's working memory.  ``iris_gemm_noalloc`` keeps that working memory in a fixed array
inside the library.  Here it is called through its exported C symbol, twice in a row with different data (the
second call finds the first call's leftovers in the scratch), and each result is compared with the plan-based
entry point and with a plain PyTorch fp32 product.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

import iris_b200 as iris  # noqa: E402
from iris_b200 import _native  # noqa: E402
from iris_b200.ops import gemm as G  # noqa: E402


def _entry():
    lib = _native.kernels()
    fn = lib.iris_gemm_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.iris_gemm_noalloc_status.restype = ctypes.c_int
    lib.iris_gemm_last_error.restype = ctypes.c_char_p
    return lib, fn


def _rand(shape, seed, scale=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(torch.bfloat16)


def _close(got, ref):
    ref = ref.float()
    tol = 2.0 * (2.0 ** -8) * ref.abs() + 1e-3 * ref.abs().max().item() + 1e-6
    err = (got.float() - ref).abs()
    assert not bool((err > tol).any()), f"max err {err.max().item():.4g}"


def test_noalloc_matches_plan_entry_twice_in_a_row():
    lib, fn = _entry()
    m, n, k = 1000, 1024, 1376          # row tail in M, half-filled last K slice
    out = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ctx = iris.Iris.local_world(1, heap_size=32 << 20)[0]
    stream = torch.cuda.current_stream().cuda_stream
    for call, seed in enumerate((11, 12)):
        a, bt = _rand((m, k), seed), _rand((n, k), seed + 100, 0.05)
        out.fill_(float("nan"))
        rc = fn(a.data_ptr(), a.stride(0), bt.data_ptr(), bt.stride(0), out.data_ptr(), out.stride(0), m, n, k,
                ctypes.c_void_p(stream))
        assert rc == 0, lib.iris_gemm_last_error().decode()
        torch.cuda.synchronize()
        assert lib.iris_gemm_noalloc_status() == 0
        # existing entry point, same mode and schedule of the same kernel (single CTAs, whole tiles), scratch on a heap
        plan = G.FusedGemm(ctx, [a], [bt], "one_shot", cta_group=1, stream_k=False)
        ref_entry = plan()[0]
        plan.check()
        _close(out, ref_entry)
        assert torch.equal(out, ref_entry), f"call {call}: differs from the plan-based entry point"
        _close(out, a.float() @ bt.float().t())
        plan.close()
        ctx.reset()
    ctx.close()


@pytest.mark.parametrize("m,n,k,pad,side_stream", [(100, 1024, 512, 0, False), (1000, 520, 320, 0, False),
                                                    (384, 512, 256, 64, False), (512, 768, 448, 0, True)])
def test_noalloc_shapes_pitches_streams_and_no_allocation(m, n, k, pad, side_stream):
    """A matrix shorter than one tile, a width that ends inside a 64-column sub-tile, an output with padded rows and a
    launch on a side stream; and the property in the name: the device's free memory is the same before and after the
    first and the second call (nothing was allocated on the caller's behalf, by this library or by a library it uses)."""
    lib, fn = _entry()
    a, bt = _rand((m, k), 21), _rand((n, k), 22, 0.05)
    out_full = torch.full((m, n + pad), float("nan"), dtype=torch.bfloat16, device="cuda")
    out = out_full[:, :n]
    st = torch.cuda.Stream() if side_stream else torch.cuda.current_stream()
    ref = a.float() @ bt.float().t()
    torch.cuda.synchronize()
    rc = fn(a.data_ptr(), a.stride(0), bt.data_ptr(), bt.stride(0), out.data_ptr(), out.stride(0), m, n, k,
            ctypes.c_void_p(st.cuda_stream))       # first use on this device may do the one-time set-up
    assert rc == 0, lib.iris_gemm_last_error().decode()
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for call in range(2):
        out_full.fill_(float("nan"))
        torch.cuda.synchronize()
        rc = fn(a.data_ptr(), a.stride(0), bt.data_ptr(), bt.stride(0), out.data_ptr(), out.stride(0), m, n, k,
                ctypes.c_void_p(st.cuda_stream))
        assert rc == 0, lib.iris_gemm_last_error().decode()
        st.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0, f"call {call}: free device memory changed"
        assert lib.iris_gemm_noalloc_status() == 0
        _close(out, ref)
        if pad:
            assert bool(torch.isnan(out_full[:, n:].float()).all()), "wrote past the row's N columns"


def test_noalloc_rejects_oversize_and_bad_arguments():
    lib, fn = _entry()
    a, bt = _rand((128, 64), 1), _rand((256, 64), 2)
    out = torch.empty((128, 256), dtype=torch.bfloat16, device="cuda")
    big = 4096  # 4096 * 4096 elements > the built-in scratch
    rc = fn(a.data_ptr(), 64, bt.data_ptr(), 64, out.data_ptr(), big, big, big, 64, None)
    assert rc == -2
    assert b"exceeds the built-in scratch" in lib.iris_gemm_last_error()
    rc = fn(a.data_ptr(), 64, bt.data_ptr(), 64, out.data_ptr(), 256, 128, 252, 64, None)
    assert rc == -1
    rc = fn(None, 64, bt.data_ptr(), 64, out.data_ptr(), 256, 128, 256, 64, None)
    assert rc == -1
    rc = fn(a.data_ptr(), 56, bt.data_ptr(), 64, out.data_ptr(), 256, 128, 256, 64, None)      # lda < K
    assert rc == -1 and b"row pitches" in lib.iris_gemm_last_error()
    rc = fn(a.data_ptr(), 64, bt.data_ptr(), 64, out.data_ptr(), 1 << 31, 128, 256, 64, None)  # ldo does not fit
    assert rc == -1
