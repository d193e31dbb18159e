"""Typed description of one benchmark point of the fused GEMM + collective workloads, with its validity rules and the
tile-table lookup, shared by the sweep driver and by tests.

Role in the reference: the shape / tile bookkeeping spread over ``examples/benchmark/bench_all_shapes.py:105-170``
(per-rank shape, lookup in ``dataset/tiling.json``) and the per-script ``argparse`` dictionaries
(``examples/07_gemm_all_scatter/benchmark.py:24-75``), which are neither typed nor validated.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Tuple

# workload -> example script (relative to the repository root) and the --variant it needs, if any
WORKLOADS: Dict[str, Tuple[str, Optional[str]]] = {
    "all_scatter": ("examples/07_gemm_all_scatter/benchmark.py", None),
    "atomic": ("examples/08_gemm_atomics_all_reduce/benchmark.py", None),
    "one_shot": ("examples/09_gemm_one_shot_all_reduce/benchmark.py", "one_shot"),
    "two_shot": ("examples/09_gemm_one_shot_all_reduce/benchmark.py", "two_shot"),
    "reduce_scatter": ("examples/11_gemm_reduce_scatter/benchmark.py", None),
}


@dataclass(frozen=True)
class TileConfig:
    """What can vary per shape on this kernel: the tile (``BLK_M`` 128 = one CTA per tile, 256 = a CTA pair per tile,
    0 = chosen from M; ``BLK_N`` 64 / 128 / 256 columns; the k-block is fixed at 64), the raster group, the size of
    the persistent grid (0 = all SMs), the K pieces per tile of the short-matrix forms (0 = chosen by the planner)
    and the column split of a ragged last wave (0 = off)."""
    BLK_M: int = 0
    BLK_N: int = 256
    BLK_K: int = 64
    gsize_m: int = 8
    gemm_sms: int = 0
    ksplit: int = 0
    tail_split: int = 0

    def problems(self) -> List[str]:
        out = []
        if self.BLK_M not in (0, 128, 256):
            out.append("BLK_M must be 128 or 256 (0: chosen from M)")
        if self.BLK_N not in (64, 128, 256):
            out.append("BLK_N must be 64, 128 or 256")
        if self.BLK_K != 64:
            out.append("BLK_K is fixed at 64")
        return out


@dataclass(frozen=True)
class GemmPoint:
    """One (workload, shape, number of ranks) point."""
    workload: str
    m: int
    n: int
    k: int
    world: int = 1
    name: str = ""
    dtype: str = "bf16"
    num_experiments: int = 50
    num_warmup: int = 10
    extra: Tuple[str, ...] = field(default_factory=tuple)

    def problems(self) -> List[str]:
        """Why this point cannot run (empty list: it can).  The rules are the kernel's: 16-byte rows, whole 64-column
        sub-tiles when tiles are pushed to peers, K shards that are multiples of 8, whole tiles per keeper."""
        w, out = self.world, []
        if self.workload not in WORKLOADS:
            return [f"unknown workload {self.workload!r}"]
        if self.dtype not in ("bf16", "fp16", "fp32", "int8"):
            out.append("the element type must be bf16, fp16, fp32 or int8")
        elif self.dtype in ("fp32", "int8") and self.workload != "all_scatter":
            out.append("fp32 and int8 are offered by the all-scatter kernel only")
        if min(self.m, self.n, self.k, w) < 1 or w > 8:
            out.append("m, n, k must be positive and 1 <= world <= 8")
            return out
        es = {"fp32": 4, "int8": 1}.get(self.dtype, 2)
        sub, vec = 128 // es, 16 // es      # columns of a 128-byte sub-tile row, elements of a 16-byte vector
        if self.workload == "all_scatter":
            if self.n % w:
                out.append("N must divide by the number of ranks")
            elif (self.n // w) % (sub if w > 1 else vec):
                out.append(f"N per rank must be a multiple of {sub} ({vec} on one rank)")
            if self.k % vec:
                out.append(f"K must be a multiple of {vec}")
        else:
            if self.k % w or (self.k // w) % 8:
                out.append("K per rank must be a multiple of 8")
            if self.n % (64 if (w > 1 and self.workload == "atomic") else 8):
                out.append("N must be a multiple of 8 (64 for the atomic variant across ranks)")
            if self.workload == "reduce_scatter" and self.m % (w * 128):
                out.append("M must be a multiple of ranks x 128")
        return out

    def per_rank_shape(self) -> Tuple[int, int, int]:
        """The GEMM each rank computes: N is sharded for all-scatter, K for the reductions."""
        w = self.world
        return (self.m, self.n // w, self.k) if self.workload == "all_scatter" else (self.m, self.n, self.k // w)

    def tile(self, table: dict) -> TileConfig:
        """Look the per-rank shape up in a table of the form of ``configs/tiling_b200.json``."""
        cfg = dict(table.get("default", {}))
        m, n, k = self.per_rank_shape()
        for o in table.get("overrides", []):
            if (o["m"], o["n"], o["k"]) == (m, n, k):
                cfg.update({k_: v for k_, v in o.items() if k_ not in ("m", "n", "k")})
        known = {f for f in TileConfig.__dataclass_fields__}
        return TileConfig(**{k_: v for k_, v in cfg.items() if k_ in known})

    def command(self, root: str, table: dict, output_file: str = "", python: str = "python",
                timeout_s: float = 300.0) -> List[str]:
        """The launcher command line that runs this point with validation and timing."""
        script, variant = WORKLOADS[self.workload]
        t = self.tile(table)
        blk_n = max(t.BLK_N, 128) if self.dtype == "int8" else t.BLK_N   # an int8 sub-tile row is 128 columns
        cmd = [python, "-m", "iris_b200.launch", "-np", str(self.world), "--timeout", str(timeout_s),
               f"{root.rstrip('/')}/{script}", "-m", str(self.m), "-n", str(self.n), "-k", str(self.k), "-v", "-b",
               "--gsize_m", str(t.gsize_m), "--gemm_sms", str(t.gemm_sms), "--num_experiments",
               str(self.num_experiments), "--num_warmup", str(self.num_warmup), "--datatype", self.dtype,
               "--BLK_N", str(blk_n)]
        if t.BLK_M:
            cmd += ["--BLK_M", str(t.BLK_M)]
        if t.ksplit:
            cmd += ["--ksplit", str(t.ksplit)]
        if t.tail_split:
            cmd += ["--tail_split", str(t.tail_split)]
        if variant:
            cmd += ["--variant", variant]
        if output_file:
            cmd += ["--output_file", output_file]
        return cmd + list(self.extra)

    def to_json(self) -> str:
        return json.dumps(asdict(self))


def load_points(shapes: dict, worlds=(1, 2, 4, 8)) -> List[GemmPoint]:
    """All points of a shape file of the form of ``configs/shapes.json`` x the given rank counts.  A shape may name
    its element type (``"dtype"``: bf16, fp16, fp32 or int8; default bf16)."""
    pts = []
    for s in shapes["shapes"]:
        for wl in s["workloads"]:
            for w in worlds:
                pts.append(GemmPoint(wl, s["m"], s["n"], s["k"], w, name=s["name"], dtype=s.get("dtype", "bf16")))
    return pts
