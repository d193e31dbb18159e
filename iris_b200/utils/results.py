"""Result writers and per-tile timestamps.

Role in the reference: ``examples/common/utils.py:22-128`` (``JSONWriter`` that collects fields and dumps one
JSON document; ``Timestamps`` holding per-tile begin/end device times and converting them to microseconds).
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, List

import torch


class JSONWriter:
    """Collects key/value pairs and writes them as one JSON object."""

    def __init__(self, file_path: str):
        self.file_path = file_path
        self.data: Dict[str, Any] = {}
        if file_path and os.path.exists(file_path):
            os.remove(file_path)

    def add_field(self, key: str, value: Any) -> None:
        self.data[key] = value

    def add_fields(self, **kw) -> None:
        self.data.update(kw)

    def add_environment(self, device=None) -> None:
        """Record where the numbers come from: time, host, package and torch versions, the source revision when the
        package sits in a git checkout, and the GPU (name, SM count, memory) when one is given or current."""
        import datetime
        import platform
        import subprocess
        env: Dict[str, Any] = {"time_utc": datetime.datetime.now(datetime.timezone.utc).isoformat(timespec="seconds"),
                               "host": platform.node(), "python": platform.python_version(),
                               "torch": torch.__version__, "cuda": torch.version.cuda}
        try:
            from .. import __version__
            env["iris_b200"] = __version__
        except Exception:
            pass
        root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        try:
            rev = subprocess.run(["git", "-C", root, "rev-parse", "--short", "HEAD"], capture_output=True, text=True,
                                 timeout=5)
            if rev.returncode == 0:
                env["git"] = rev.stdout.strip()
        except Exception:
            pass
        if torch.cuda.is_available():
            props = torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device())
            env["gpu"] = {"name": props.name, "sms": props.multi_processor_count,
                          "memory_gb": round(props.total_memory / 2 ** 30, 1),
                          "capability": f"{props.major}.{props.minor}"}
        self.data["environment"] = env

    def flush(self) -> None:
        if not self.file_path:
            return
        d = os.path.dirname(self.file_path)
        if d:
            os.makedirs(d, exist_ok=True)
        with open(self.file_path, "w") as f:
            json.dump(self.data, f, indent=2, default=str)

    def display(self) -> None:
        print(json.dumps(self.data, indent=2, default=str))


class Timestamps:
    """Per-tile begin/end times in nanoseconds of ``iris::globaltimer()`` (1 GHz)."""

    FIELDS = ("mm_begin", "mm_end", "comm_begin", "comm_end")

    def __init__(self, num_tiles: int, device="cuda"):
        self.num_tiles = num_tiles
        big = torch.iinfo(torch.int64).max
        self.mm_begin = torch.full((num_tiles,), big, dtype=torch.int64, device=device)
        self.mm_end = torch.zeros(num_tiles, dtype=torch.int64, device=device)
        self.comm_begin = torch.full((num_tiles,), big, dtype=torch.int64, device=device)
        self.comm_end = torch.zeros(num_tiles, dtype=torch.int64, device=device)

    def reset(self) -> None:
        big = torch.iinfo(torch.int64).max
        self.mm_begin.fill_(big)
        self.mm_end.zero_()
        self.comm_begin.fill_(big)
        self.comm_end.zero_()

    def to_records(self) -> List[dict]:
        cols = {k: getattr(self, k).cpu().tolist() for k in self.FIELDS}
        t0 = min(cols["mm_begin"]) if cols["mm_begin"] else 0
        recs = []
        for t in range(self.num_tiles):
            recs.append({"tile_id": t, **{k: (cols[k][t] - t0) / 1e3 for k in self.FIELDS}})  # microseconds
        return recs

    def to_json(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump(self.to_records(), f)


# Phases of a fused-GEMM tile record (``FusedGemm.trace_records``): name, begin key, end key, lane inside the CTA.
TILE_PHASES = (("main loop", "mma_begin", "mma_end", 0), ("epilogue", "epi_begin", "epi_end", 1),
               ("flag wait", "wait_begin", "wait_end", 2), ("sum", "wait_end", "pull_end", 2))


def tile_trace_to_chrome(records: List[dict], rank: int = 0) -> dict:
    """Per-tile device timestamps as a Chrome / Perfetto trace (``chrome://tracing``, ui.perfetto.dev): one process per
    rank, one thread per (tile record, role), complete events in microseconds.  The reference dumps a flat JSON list
    (``examples/common/utils.py:66-128``) and draws its timelines by hand (``docs/FINEGRAINED_OVERLAP.md`` figures)."""
    events = [{"ph": "M", "name": "process_name", "pid": rank, "args": {"name": f"rank {rank}"}}]
    for rec in records:
        for name, kb, ke, lane in TILE_PHASES:
            b, e = rec.get(kb), rec.get(ke)
            if b is None or e is None or e < b:
                continue
            events.append({"ph": "X", "name": name, "cat": "tile", "pid": rank, "tid": 3 * int(rec["record"]) + lane,
                           "ts": float(b), "dur": float(e - b),
                           "args": {"tile_id": rec.get("tile_id"), "cta_in_pair": rec.get("cta_in_pair")}})
    return {"traceEvents": events, "displayTimeUnit": "ns"}


def validate_gemm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor, ctx=None, atol: float = 1.0) -> bool:
    """``A @ B`` against ``C`` with an absolute tolerance (``examples/common/validation.py:7-23``)."""
    expected = (A.float() @ B.float()).to(C.dtype)
    close = torch.isclose(C.float(), expected.float(), atol=atol, rtol=0)
    if bool(close.all()):
        return True
    idx = (~close).nonzero()[0].tolist()
    msg = f"mismatch at {idx}: C = {C[tuple(idx)].item()}, expected = {expected[tuple(idx)].item()}"
    if ctx is not None:
        ctx.log(msg)
    else:
        print(msg)
    return False
