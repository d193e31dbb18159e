"""RMSNorm, residual add + RMSNorm in one pass, SwiGLU and residual add (``csrc/kernels/elementwise.cu``): bf16 tensors with a contiguous last
dimension, arbitrary row pitch, fp32 arithmetic.  Used by the tensor-parallel decoder block; no counterpart in the
reference."""
from __future__ import annotations

import ctypes

import torch

from .. import _native


def _st(t, stream):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream if stream is None else stream)


def _check2d(t, name):
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1 or t.data_ptr() % 16 or (t.stride(0) * 2) % 16:
        raise ValueError(f"{name}: need a 2-D bf16 tensor, contiguous rows, 16-byte aligned")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float = 1e-6, stream=None) -> torch.Tensor:
    """``out = x * rsqrt(mean(x^2, -1) + eps) * weight`` row by row; ``out`` may be a row block of a larger matrix."""
    _check2d(x, "x"), _check2d(out, "out")
    lib = _native.kernels()
    lib.iris_k_rmsnorm_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int64, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    rc = lib.iris_k_rmsnorm_bf16(x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0),
                                 x.shape[0], x.shape[1], eps, _st(x, stream))
    if rc:
        raise RuntimeError(f"rmsnorm launch failed ({rc})")
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
    """``out = silu(gate_up[:, :I]) * gate_up[:, I:]`` with ``I = out.shape[1]``."""
    _check2d(gate_up, "gate_up"), _check2d(out, "out")
    inter = out.shape[1]
    if gate_up.shape[1] != 2 * inter:
        raise ValueError("gate_up must have twice the columns of out")
    lib = _native.kernels()
    lib.iris_k_swiglu_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                       ctypes.c_int, ctypes.c_void_p]
    rc = lib.iris_k_swiglu_bf16(gate_up.data_ptr(), gate_up.stride(0), out.data_ptr(), out.stride(0), out.shape[0],
                                inter, _st(out, stream))
    if rc:
        raise RuntimeError(f"swiglu launch failed ({rc})")
    return out


def residual_add(x: torch.Tensor, y: torch.Tensor, stream=None) -> torch.Tensor:
    """``x += y`` in place."""
    _check2d(x, "x"), _check2d(y, "y")
    lib = _native.kernels()
    lib.iris_k_residual_add_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                             ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    rc = lib.iris_k_residual_add_bf16(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), x.shape[0], x.shape[1],
                                      _st(x, stream))
    if rc:
        raise RuntimeError(f"residual_add launch failed ({rc})")
    return x


def add_rmsnorm(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float = 1e-6,
                stream=None) -> torch.Tensor:
    """``x += y`` (in place) and ``out = rmsnorm(x) * weight`` in one pass over the rows: the residual add at the end
    of one sub-block fused with the norm that opens the next.  ``out`` may be a row block of a larger matrix."""
    _check2d(x, "x"), _check2d(y, "y"), _check2d(out, "out")
    lib = _native.kernels()
    lib.iris_k_add_rmsnorm_bf16.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64,
                                            ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int,
                                            ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    rc = lib.iris_k_add_rmsnorm_bf16(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), weight.data_ptr(),
                                     out.data_ptr(), out.stride(0), x.shape[0], x.shape[1], eps, _st(x, stream))
    if rc == -3:     # row too long for the register-resident kernel
        residual_add(x, y, stream)
        return rmsnorm(x, weight, out, eps, stream)
    if rc:
        raise RuntimeError(f"add_rmsnorm launch failed ({rc})")
    return out
