"""Roofline arithmetic for the fused GEMM + collective kernels.

The target time of a fused kernel is the slower of (FLOPs / measured GEMM peak) and (bytes that must cross
NVLink / link bandwidth per direction); the achieved fraction is target / measured.  Peaks come from the
machine-written ``MEASURED_PEAKS.json`` when it exists, else from an earlier measurement on the same pool.
(The reference's only such arithmetic is ``scripts/link_bandwidth.py:50-54``.)
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass

FALLBACK = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
NVLINK_GBS_MEASURED = 770.0  # peer copy, per direction per GPU
NVLINK_GBS_NOMINAL = 900.0


@dataclass
class Peaks:
    hbm_gbs: float
    bf16_tflops: float
    bf16_tflops_sustained: float
    nvlink_gbs: float
    source: str


def load_peaks(path: str = None) -> Peaks:
    path = path or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                "MEASURED_PEAKS.json")
    d, src = dict(FALLBACK), "fallback"
    if os.path.exists(path):
        try:
            with open(path) as f:
                m = json.load(f)
            d.update({k: float(m[k]) for k in FALLBACK if k in m})
            src = "measured"
        except (OSError, ValueError):
            pass
    return Peaks(d["hbm_gbs"], d["bf16_tflops"], d["bf16_tflops_sustained"], NVLINK_GBS_MEASURED, src)


def gemm_flops(m: int, n: int, k: int) -> float:
    return 2.0 * m * n * k


# Tensor-core rate of an element type relative to bf16 (nominal ratios of the dense peaks: tf32 half, int8 twice), and
# bytes per element.  Only the bf16 rate is measured on this hardware; the others are that figure scaled.
DTYPE_RATE = {"bf16": 1.0, "fp16": 1.0, "fp32": 0.5, "int8": 2.0}
DTYPE_BYTES = {"bf16": 2, "fp16": 2, "fp32": 4, "int8": 1}


def all_scatter_roofline_us(m, n, k, world, peaks: Peaks, dtype: str = "bf16") -> dict:
    """C[m, n] = A[m, k] B[k, n], B column-sharded: each rank computes m*n/world outputs and receives the rest."""
    compute = gemm_flops(m, n // world, k) / (peaks.bf16_tflops * DTYPE_RATE[dtype] * 1e12) * 1e6
    ingress = (world - 1) * m * (n // world) * DTYPE_BYTES[dtype]
    link = ingress / (peaks.nvlink_gbs * 1e9) * 1e6
    return {"compute_us": compute, "link_us": link, "bound": "compute" if compute >= link else "link",
            "target_us": max(compute, link)}


def all_reduce_roofline_us(m, n, k, world, peaks: Peaks, variant: str = "one_shot") -> dict:
    """K-sharded GEMM + all-reduce of the [m, n] bf16 partials.  one_shot / atomic: every rank moves
    (world-1) full partials; two_shot: 2 (world-1)/world of one; reduce_scatter (every rank keeps m / world rows of
    the sum): (world-1)/world of one."""
    compute = gemm_flops(m, n, k // world) / (peaks.bf16_tflops * 1e12) * 1e6
    full = m * n * 2
    if variant in ("one_shot", "atomic"):
        ingress = (world - 1) * full
    elif variant == "reduce_scatter":
        ingress = (world - 1) / world * full
    else:
        ingress = 2 * (world - 1) / world * full
    link = ingress / (peaks.nvlink_gbs * 1e9) * 1e6
    return {"compute_us": compute, "link_us": link, "bound": "compute" if compute >= link else "link",
            "target_us": max(compute, link)}


def effective_link_bandwidth(result: dict) -> dict:
    """From one result record of a fused all-scatter run (the JSON of ``examples/07_gemm_all_scatter``): bytes every
    rank receives, and the NVLink bandwidth that would be needed to hide them behind the measured kernel time
    (the reference's ``scripts/link_bandwidth.py:50-54`` prints the same quantity for its sample record)."""
    m, n, w = int(result["m"]), int(result["n"]), int(result.get("world_size", 1))
    ms = float(result.get("fused_ms") or result.get("ms"))
    ingress = (w - 1) * m * (n // w) * 2
    return {"ingress_bytes_per_rank": ingress, "kernel_ms": ms, "gbs_per_rank": ingress / (ms * 1e-3) / 1e9,
            "fraction_of_measured_link": ingress / (ms * 1e-3) / 1e9 / NVLINK_GBS_MEASURED}


if __name__ == "__main__":
    import sys
    if len(sys.argv) != 2:
        raise SystemExit("usage: python -m iris_b200.utils.roofline <result.json from examples/07_gemm_all_scatter>")
    with open(sys.argv[1]) as f:
        rec = json.load(f)
    out = effective_link_bandwidth(rec)
    print(json.dumps(out, indent=2))
