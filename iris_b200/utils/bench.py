"""Benchmark timer and small device utilities.

Role in the reference: ``iris/util.py:62-128`` (``do_bench`` with a 256 MB cache-flush buffer, 25 warm-ups and
100 repeats, barrier before every iteration; ``memset_tensor`` for int32 flag arrays).  The signature of
``do_bench`` is kept.  Differences: the timed region is bracketed by CUDA events on the launching stream only
(host barriers sit outside it), and ``reduce_ranks`` returns the maximum over ranks, which is the figure a
multi-GPU kernel is judged by.
"""
from __future__ import annotations

import ctypes
import statistics
import subprocess
import threading
import time
from typing import Callable, List, Optional

import torch

from .. import _native

_cache_buffers = {}


def _noop():
    return None


def flush_l2(device=None) -> None:
    """Overwrite a buffer larger than the L2 (256 MB against 126 MB on B200) so the next kernel starts cold."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _cache_buffers.get(dev)
    if buf is None:
        buf = torch.empty(256 << 20, dtype=torch.int8, device=dev)
        _cache_buffers[dev] = buf
    buf.zero_()


def _summarise(times: List[float], quantiles, return_mode: str):
    if quantiles is not None:
        t = torch.tensor(times, dtype=torch.float64)
        q = torch.quantile(t, torch.tensor(quantiles, dtype=torch.float64)).tolist()
        return q[0] if len(q) == 1 else q
    if return_mode == "all":
        return times
    return {"mean": statistics.fmean, "min": min, "max": max, "median": statistics.median}[return_mode](times)


def do_bench(fn: Callable, barrier_fn: Callable = _noop, preamble_fn: Callable = _noop, n_warmup: int = 25,
             n_repeat: int = 100, quantiles=None, return_mode: str = "mean", flush: bool = True):
    """Time ``fn`` in milliseconds (CUDA events when a GPU is present, ``perf_counter`` otherwise).

    Every iteration: ``barrier_fn(); preamble_fn(); flush L2; barrier_fn(); start; fn(); end``.
    """
    cuda = torch.cuda.is_available()
    barrier_fn()
    preamble_fn()
    fn()
    barrier_fn()
    times: List[float] = []
    if cuda:
        starts = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
        ends = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(-n_warmup, n_repeat):
        barrier_fn()
        preamble_fn()
        if cuda and flush:
            flush_l2()
        barrier_fn()
        if cuda:
            if i >= 0:
                starts[i].record()
            fn()
            if i >= 0:
                ends[i].record()
        else:
            t0 = time.perf_counter()
            fn()
            if i >= 0:
                times.append((time.perf_counter() - t0) * 1e3)
    barrier_fn()
    if cuda:
        torch.cuda.synchronize()
        times = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    return _summarise(times, quantiles, return_mode)


def reduce_ranks(ctx, value: float, how: str = "max") -> float:
    """Combine one float per rank on the host control plane (max by default)."""
    if ctx.get_num_ranks() == 1 or getattr(ctx, "_local_world", None) is not None:
        return float(value)
    import struct
    vals = [struct.unpack("d", b)[0] for b in ctx.comm.allgather_bytes(struct.pack("d", float(value)))]
    return {"max": max, "min": min, "mean": statistics.fmean}[how](vals)


def memset_tensor(tensor: torch.Tensor, value: int, stream=None) -> None:
    """Fill a contiguous int32 tensor without a host synchronisation (``iris/util.py:117-128``)."""
    assert tensor.is_contiguous(), "Tensor must be contiguous"
    assert tensor.dtype == torch.int32, "Only torch.int32 tensors are supported"
    if not tensor.is_cuda:
        tensor.fill_(value)
        return
    lib = _native.kernels()
    fn = lib.iris_k_memset_i32
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_uint64, ctypes.c_void_p]
    st = torch.cuda.current_stream(tensor.device).cuda_stream if stream is None else stream
    if fn(ctypes.c_void_p(tensor.data_ptr()), int(value), tensor.numel(), ctypes.c_void_p(st)) != 0:
        raise RuntimeError("memset kernel launch failed")


class ClockSampler:
    """Samples SM clock, power and throttle reasons with ``nvidia-smi`` while a timed region runs (read-only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc: Optional[subprocess.Popen] = None
        self.lines: List[str] = []
        self._thread: Optional[threading.Thread] = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-i",
                 str(self.gpu_index), "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
        except (FileNotFoundError, OSError):
            self.proc = None
            return self

        def pump():
            for line in self.proc.stdout:
                self.lines.append(line.strip())
        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def wait_first_sample(self, timeout_s: float = 10.0) -> bool:
        """Block until the first sample has arrived (``nvidia-smi`` takes a second or more to start on a machine
        with several GPUs): call it before the region of interest, so that the start-up neither falls into the timed
        region nor leaves it without samples."""
        t_end = time.monotonic() + timeout_s
        while self.proc is not None and not self.lines and time.monotonic() < t_end and self.proc.poll() is None:
            time.sleep(0.01)
        return bool(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax.append(float(f[2]))
                power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # "under load" = samples in the upper half of the power range seen
        if sm:
            thr = (max(power) + min(power)) / 2
            loaded = [c for c, p in zip(sm, power) if p >= thr] or sm
            return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(smax), "reasons": sorted(reasons),
                    "samples": len(sm), "power_w_max": max(power)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": sorted(reasons), "samples": 0}
