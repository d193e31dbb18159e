"""Self-attention forward on the tcgen05 kernel of ``csrc/kernels/attention.cu`` (head dimension 128, bf16 / fp16).

No counterpart in the reference, which has no model code; the tensor-parallel decoder block
(``iris_b200/models/tp_block.py``) uses it for the attention core between its fused all-gather -> GEMM (which produces
``qkv``) and its fused GEMM -> all-reduce (which consumes ``out``), so that no phase of the block is a library kernel.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _native

HEAD_DIM = 128
_DT = {torch.bfloat16: 0, torch.float16: 1}


def attention_fwd(qkv: torch.Tensor, out: torch.Tensor, batch: int, seq: int, heads: int, causal: bool = True,
                  status: Optional[torch.Tensor] = None, timeout_ms: float = 2000.0, stream=None) -> torch.Tensor:
    """``out[b*seq + s, h*128:(h+1)*128] = softmax(q . k^T / sqrt(128)) . v`` per batch ``b`` and head ``h``.

    ``qkv`` is ``[batch * seq, 3 * heads * 128]`` with the Q, K and V column blocks side by side (head ``h`` in columns
    ``h * 128 ..`` of each block), ``out`` is ``[batch * seq, heads * 128]``; rows may be strided views.  ``seq`` must be
    a multiple of 128.  ``status``: the int32 status block of an ``Iris`` context (``ctx.status``), in which a bounded
    wait of the kernel records a time-out; ``None``: not recorded.
    """
    if qkv.dtype not in _DT or out.dtype != qkv.dtype:
        raise TypeError("qkv and out must both be bfloat16 or both float16")
    if qkv.dim() != 2 or out.dim() != 2 or qkv.stride(1) != 1 or out.stride(1) != 1:
        raise ValueError("qkv and out must be 2-D with contiguous rows")
    if qkv.shape != (batch * seq, 3 * heads * HEAD_DIM) or out.shape != (batch * seq, heads * HEAD_DIM):
        raise ValueError(f"expected qkv [{batch * seq}, {3 * heads * HEAD_DIM}] and out [{batch * seq}, "
                         f"{heads * HEAD_DIM}], got {tuple(qkv.shape)} and {tuple(out.shape)}")
    lib = _native.kernels()
    fn = lib.iris_k_attention_fwd
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64, ctypes.c_void_p]
    lib.iris_attention_last_error.restype = ctypes.c_char_p
    st = torch.cuda.current_stream(qkv.device).cuda_stream if stream is None else stream
    rc = fn(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), batch, seq, heads, int(bool(causal)),
            _DT[qkv.dtype], ctypes.c_void_p(status.data_ptr() if status is not None else 0), int(timeout_ms * 1e6),
            ctypes.c_void_p(st))
    if rc != 0:
        raise RuntimeError(lib.iris_attention_last_error().decode() or f"attention launch failed ({rc})")
    return out
