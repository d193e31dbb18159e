"""Operators: RMA primitives, P2P bandwidth kernels, fused GEMM + collective kernels, element-wise kernels."""
from . import rma  # noqa: F401
