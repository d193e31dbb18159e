"""Fused bf16 / fp16 GEMM + collective operators on the tcgen05 kernel of ``csrc/kernels/gemm_fused.cu``.

Role in the reference: the ``matmul`` autograd-Function wrappers that launch the persistent Triton kernels
(``examples/07_gemm_all_scatter/matmul_wrapper.py:19-219`` and its copies in 08/09) together with the buffer
set-up of the drivers (``examples/07_gemm_all_scatter/benchmark.py:103-142``).

Operand convention (as the reference: ``A = randn(m, k)``, ``B = randn(n, k).T``,
``examples/07_gemm_all_scatter/benchmark.py:103-104``): ``A`` is ``[M, K]`` and ``B`` is given as ``Bt = [N, K]``,
both K-contiguous with an arbitrary 16-byte-aligned row pitch, so K-shards that are views work without copies.

A ``FusedGemm`` is built once for fixed buffers (tensor maps are encoded at construction) and called many
times; flags are cumulative counters, so nothing is reset between calls.

``ctxs`` is one :class:`~iris_b200.context.Iris` (one process per GPU) or the list returned by
``Iris.local_world`` (several ranks simulated by ONE launch on one GPU).
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence, Union

import torch

from .. import _native
from ..context import Iris
from .gemm_plan import (BK, BM, BN, DTYPES, FLAG_HEADER, MODES, PUSH_KINDS, SK_SLOTS, TILE_WIDTHS, GemmPlan,  # noqa: F401
                        plan_gemm)

MAX_RANKS = 8
# How GEMM + all-scatter tiles are pushed unless the caller says otherwise (see FusedGemm, ``push_kind``).
DEFAULT_PUSH_KIND = "tma"
# Atomic all-reduce: outputs up to this size are cleared by the kernel itself instead of by a launch before it.
ZERO_IN_KERNEL_MAX_BYTES = 8 << 20


class _Desc(ctypes.Structure):
    _fields_ = [
        ("a_ptr", ctypes.c_uint64 * MAX_RANKS), ("b_ptr", ctypes.c_uint64 * MAX_RANKS),
        ("c_ptr", ctypes.c_uint64 * MAX_RANKS), ("c2_ptr", ctypes.c_uint64 * MAX_RANKS),
        ("heap_base", ctypes.c_uint64 * MAX_RANKS),
        ("lda", ctypes.c_int64 * MAX_RANKS), ("ldb", ctypes.c_int64 * MAX_RANKS),
        ("ldc", ctypes.c_int64), ("c_cols", ctypes.c_int64), ("c_rows", ctypes.c_int64),
        ("flags_off", ctypes.c_uint64), ("partial_off", ctypes.c_uint64 * 2), ("out_off", ctypes.c_uint64),
        ("status_off", ctypes.c_uint64), ("agsrc_off", ctypes.c_uint64), ("trace_off", ctypes.c_uint64),
        ("ws_off", ctypes.c_uint64), ("mc_base", ctypes.c_uint64),
        ("timeout_ns", ctypes.c_uint64),
        ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int), ("ldo", ctypes.c_int),
        ("part_row0", ctypes.c_int * 2), ("out_row0", ctypes.c_int),
        ("col_off_per_rank", ctypes.c_int),
        ("world", ctypes.c_int), ("num_local", ctypes.c_int), ("rank0", ctypes.c_int), ("ctas_per_rank", ctypes.c_int),
        ("mode", ctypes.c_int), ("group_m", ctypes.c_int), ("ag", ctypes.c_int), ("ag_slices", ctypes.c_int),
        ("store_all", ctypes.c_int), ("tile_flag_base", ctypes.c_int), ("ag_flag_base", ctypes.c_int),
        ("device", ctypes.c_int), ("cta_group", ctypes.c_int),
        ("dp_tiles", ctypes.c_int), ("sk_units", ctypes.c_int), ("sk_flag_base", ctypes.c_int),
        ("push_partials", ctypes.c_int), ("part_slot_rows", ctypes.c_int), ("ksplit", ctypes.c_int),
        ("rs_rows", ctypes.c_int), ("rs_bcast", ctypes.c_int),
        ("bn", ctypes.c_int), ("dtype", ctypes.c_int), ("push_kind", ctypes.c_int),
        ("tail_tiles", ctypes.c_int), ("tail_split", ctypes.c_int), ("sk_slots", ctypes.c_int),
        ("c_off", ctypes.c_uint64), ("zero_bytes", ctypes.c_uint64),
    ]


def _lib():
    lib = _native.kernels()
    if not getattr(lib, "_gemm_typed", False):
        lib.iris_gemm_last_error.restype = ctypes.c_char_p
        lib.iris_gemm_plan_create.restype = ctypes.c_void_p
        lib.iris_gemm_plan_create.argtypes = [ctypes.POINTER(_Desc)]
        lib.iris_gemm_plan_destroy.argtypes = [ctypes.c_void_p]
        lib.iris_gemm_plan_ctas_per_rank.argtypes = [ctypes.c_void_p]
        lib.iris_gemm_plan_cta_group.argtypes = [ctypes.c_void_p]
        lib.iris_gemm_plan_launch.restype = ctypes.c_int
        lib.iris_gemm_plan_launch.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        if lib.iris_gemm_desc_size() != ctypes.sizeof(_Desc):
            raise RuntimeError("IrisGemmDesc layout mismatch between Python and the native library")
        lib._gemm_typed = True
    return lib


_TORCH_DTYPES = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32", torch.int8: "int8"}


def _check_operand(t: torch.Tensor, name: str, dtype: Optional[torch.dtype] = None):
    if t.dtype not in _TORCH_DTYPES:
        raise TypeError(f"{name} must be bfloat16, float16, float32 or int8, got {t.dtype}")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} is {t.dtype}, the other operands are {dtype}")
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be 2-D with a contiguous last dimension (K-major)")
    if t.data_ptr() % 16 or (t.stride(0) * t.element_size()) % 16:
        raise ValueError(f"{name}: base address and row pitch must be multiples of 16 bytes")


def as_kmajor_bt(b: torch.Tensor) -> torch.Tensor:
    """Accept ``B`` as ``[K, N]`` with strides ``(1, ld)`` (the reference's ``randn(n, k).T``) or as ``Bt = [N, K]``
    with a contiguous last dimension, and return the ``[N, K]`` K-major view."""
    if b.dim() != 2:
        raise ValueError("B must be 2-D")
    if b.stride(1) == 1:
        return b
    if b.stride(0) == 1:
        return b.t()
    raise ValueError("B must be K-contiguous (pass randn(n, k).T or an [N, K] tensor)")


class FusedGemm:
    """One fused GEMM + collective on fixed buffers.

    Args:
        ctxs: one ``Iris`` or the list from ``Iris.local_world``.
        a: per local rank, ``[M, K]`` K-major (with ``ag=True``: ignored, the gathered buffer ``a_full`` is used).
        bt: per local rank, ``[N, K]`` K-major.
        mode: ``"store"`` (all-scatter when ``store_all``), ``"reduce"`` (atomic all-reduce), ``"one_shot"``,
            ``"two_shot"``.
        store_all: push each tile to every rank (``store`` / ``reduce``).
        c_cols / col_off_per_rank: width of the output buffer and column offset per rank (all-scatter:
            ``c_cols = world * N``, ``col_off_per_rank = N``).
        ag: run the all-gather prologue (A rows sharded M / world per rank; see ``a_full``).
        reduce_scatter: with ``mode="one_shot"``: every rank keeps only its own ``M / world`` rows of the sum
            (``out[l]`` is that block); partial tiles are pushed to the keeper of their rows only.
        bcast: with ``reduce_scatter``: the keeper writes its summed rows into every rank's output, which makes the
            op an all-reduce whose traffic is all one-way pushes ("push two-shot"; ``out[l]`` has all ``M`` rows).
        push / ksplit: one-shot for short matrices: partials pushed into inbox slots of every rank, K cut into pieces.
            With ``mode="reduce"`` (atomic all-reduce) ``ksplit`` cuts K into pieces computed by different CTAs that
            all add into the outputs, which spreads a short matrix over the whole GPU.
        nvls: two-shot on a heap bound to an NVLS multicast object: ``None`` = use it when available.
        trace: record per-tile device timestamps (``trace_records()``).
        bn: tile width in columns, 64 / 128 / 256 (default 256).  Together with ``cta_group`` (128 or 256 rows) this
            gives the six tile shapes of the kernel (the reference's per-shape ``BLK_M`` / ``BLK_N``,
            ``dataset/tiling.json``).
        tail_split: cut the tiles of a ragged last wave into column pieces: ``True`` = two, an integer = at most that
            many (store / reduce modes, whole-tile schedule; default off).
        push_kind: how tiles travel in the all-scatter and atomic all-reduce forms: ``"tma"`` (one thread issues a TMA
            store / reduce-add per rank), ``"tma_spread"`` (four issuing threads), ``"stores"`` (16-byte stores by all
            epilogue threads; all-scatter only) or ``"multimem"`` (one ``multimem.st`` / ``multimem.red.add`` per 16
            bytes on a heap bound to an NVLS multicast object: the switch delivers it to every rank).  ``None``:
            ``DEFAULT_PUSH_KIND``.

    The element type is taken from ``bt``: bf16 or fp16 (fp32 accumulation) for every mode; float32 (multiplied as
    tf32, fp32 accumulation) and int8 (32-bit integer accumulation, the low 8 bits of the sum as the result, which is
    what the reference's kernel stores when it casts its int32 accumulator to the output type) for mode ``"store"``:
    plain GEMM, GEMM + all-scatter and all-gather + GEMM.  The reference's drivers offer
    ``--datatype fp16|fp32|int8|bf16`` (``examples/07_gemm_all_scatter/benchmark.py:36-41``).
    """

    def __init__(self, ctxs: Union[Iris, Sequence[Iris]], a: Optional[Sequence[torch.Tensor]],
                 bt: Sequence[torch.Tensor], mode: str = "store", *, M: Optional[int] = None,
                 store_all: bool = False, c_cols: Optional[int] = None, col_off_per_rank: int = 0,
                 out: Optional[Sequence[torch.Tensor]] = None, ag: bool = False, ag_slices: int = 8,
                 ctas_per_rank: Optional[int] = None, group_m: Optional[int] = None, timeout_ms: float = 2000.0,
                 cta_group: Optional[int] = None, trace: bool = False, stream_k: Optional[bool] = None,
                 push: Optional[bool] = None, ksplit: Optional[int] = None, nvls: Optional[bool] = None,
                 reduce_scatter: bool = False, bn: Optional[int] = None, tail_split: Optional[bool] = None,
                 push_kind: Optional[str] = None, bcast: bool = False):
        self._ctor = (ctxs, a, bt, mode, dict(
            M=M, store_all=store_all, c_cols=c_cols, col_off_per_rank=col_off_per_rank, out=out, ag=ag,
            ag_slices=ag_slices, ctas_per_rank=ctas_per_rank, group_m=group_m, timeout_ms=timeout_ms,
            cta_group=cta_group, trace=trace, stream_k=stream_k, push=push, ksplit=ksplit, nvls=nvls,
            reduce_scatter=reduce_scatter, bn=bn, tail_split=tail_split, push_kind=push_kind, bcast=bcast))
        self.ctxs: List[Iris] = [ctxs] if isinstance(ctxs, Iris) else list(ctxs)
        c0 = self.ctxs[0]
        if c0.backend != "cuda":
            raise RuntimeError("FusedGemm needs a CUDA context (the kernel is sm_100a only)")
        self.world = c0.get_num_ranks()
        self.num_local = len(self.ctxs)
        if self.num_local != 1 and self.num_local != self.world:
            raise ValueError("pass one context, or all members of a local world")
        if mode not in MODES:
            raise ValueError(f"mode must be one of {sorted(MODES)}")
        self.mode = mode
        self.rank0 = c0.get_rank()
        bt = [as_kmajor_bt(x) for x in bt]
        self.dtype = bt[0].dtype
        for x in bt:
            _check_operand(x, "B", self.dtype)
        self.N, self.K = bt[0].shape
        self.ag = bool(ag)
        if mode in ("one_shot", "two_shot") and ag:
            raise ValueError("the all-gather prologue is combined with mode='store' only")
        if self.ag:
            if M is None:
                raise ValueError("ag=True needs M (rows of the gathered A)")
            self.M = int(M)
            # gathered A lives on the heap: peers write their rows into it
            self.a_full = [c.zeros((self.M, self.K), dtype=self.dtype) for c in self.ctxs]
            a_use = self.a_full
        else:
            a_use = list(a)
            for x in a_use:
                _check_operand(x, "A", self.dtype)
            self.M = a_use[0].shape[0]
            if a_use[0].shape[1] != self.K:
                raise ValueError(f"K mismatch: A has {a_use[0].shape[1]}, B has {self.K}")
        self.a, self.bt = a_use, bt
        dev = c0.device
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        # tile shape, persistent grid, schedule, flag count and buffer layout: a pure function of the problem
        pl = plan_gemm(self.M, self.N, self.K, self.world, self.num_local, mode, sms, ag=self.ag, cta_group=cta_group,
                       ctas_per_rank=ctas_per_rank, group_m=group_m, stream_k=stream_k, push=push, ksplit=ksplit,
                       reduce_scatter=reduce_scatter, store_all=store_all, own_out=out is not None, bn=bn,
                       tail_split=tail_split, bcast=bcast, dtype=_TORCH_DTYPES[self.dtype])
        self.plan = pl
        cta_group, group_m = pl.cta_group, pl.group_m
        self.cta_group, self.rs_rows, self.ctas_per_rank = pl.cta_group, pl.rs_rows, pl.ctas_per_rank
        self.total_tiles, self.dp_tiles, self.sk_units = pl.total_tiles, pl.dp_tiles, pl.sk_units
        self.push, self.ksplit, self.store_all = pl.push, pl.ksplit, pl.store_all
        sk_tiles, pulls, chunks_per_shard, tile_flags, nflags = (pl.sk_tiles, pl.pulls, pl.chunks_per_shard,
                                                                 pl.tile_flags, pl.nflags)
        # ---- symmetric allocations (identical sequence on every rank) ----
        self.flags = [c.zeros(nflags, dtype=torch.int32) for c in self.ctxs]
        self.trace = [c.zeros((self.total_tiles * cta_group, 10), dtype=torch.int64) for c in self.ctxs] if trace else None
        # stream-K: SK_SLOTS parked fp32 pieces per split tile part (never read before written: no clearing needed)
        self.workspace = [c.empty((max(sk_tiles, 1) * cta_group * max(pl.sk_slots, 1) * BM, BN), dtype=torch.float32)
                          for c in self.ctxs] if sk_tiles else None
        self.c_cols = int(c_cols) if c_cols else self.N
        if pulls:
            # One matrix per rank holds both partial buffers (call parity) and, unless the caller brings its own,
            # the output: [partial 0 | partial 1 | out], each padded to whole 256-row tiles, so that one tensor
            # map per rank serves partial stores, partial loads and output stores.
            rows, mp, slots, regions = pl.rows, pl.slot_rows, pl.slots, pl.regions
            self._pull_buf = [c.zeros((regions * mp, self.N), dtype=self.dtype) for c in self.ctxs]
            self.partial = [[b[q * slots * mp:q * slots * mp + rows] for b in self._pull_buf] for q in range(2)]
            self.out = list(out) if out is not None else [b[2 * slots * mp:2 * slots * mp + pl.out_rows]
                                                          for b in self._pull_buf]
            c_bufs, c2_bufs = self._pull_buf, None
            ldc, c_cols_eff = self.N, self.N
            c_rows, part_row0, out_row0 = pl.c_rows, pl.part_row0, pl.out_row0
            self._slot_rows = mp
        else:
            self.out = list(out) if out is not None else [c.zeros((self.M, self.c_cols), dtype=self.dtype)
                                                          for c in self.ctxs]
            c_bufs, c2_bufs = self.out, None
            ldc, c_cols_eff = self.out[0].stride(0), self.c_cols
            c_rows, part_row0, out_row0 = 0, (0, 0), -1
        for o in self.out:
            _check_operand(o, "output", self.dtype)
        d = _Desc()
        for l, ctx in enumerate(self.ctxs):
            d.a_ptr[l], d.lda[l] = a_use[l].data_ptr(), a_use[l].stride(0)
            d.b_ptr[l], d.ldb[l] = bt[l].data_ptr(), bt[l].stride(0)
        for t in range(self.world):
            d.heap_base[t] = c0.heap_base(t)
        if pulls or self.store_all:
            # buffers that peers touch are named by their symmetric offset
            c_off = c0.offset_of(c_bufs[0])
            c2_off = c0.offset_of(c2_bufs[0]) if c2_bufs else 0
            for t in range(self.world):
                d.c_ptr[t] = c0.heap_base(t) + c_off
                d.c2_ptr[t] = c0.heap_base(t) + c2_off if c2_bufs else 0
        else:
            # output stays on the computing rank: any device buffer will do
            c_off = c2_off = 0
            for l in range(self.num_local):
                d.c_ptr[self.rank0 + l] = c_bufs[l].data_ptr()
        d.ldc, d.c_cols, d.c_rows = ldc, c_cols_eff, c_rows
        d.part_row0[0], d.part_row0[1], d.out_row0 = part_row0[0], part_row0[1], out_row0
        d.flags_off = c0.offset_of(self.flags[0])
        d.partial_off[0] = d.partial_off[1] = c_off if pulls else 0  # base of [partials | out] (inbox reads)
        d.out_off = c0.offset_of(self.out[0]) if pulls else 0
        d.status_off = c0.offset_of(c0.status)
        d.agsrc_off = c0.offset_of(self.a_full[0]) if self.ag else 0
        d.trace_off = c0.offset_of(self.trace[0]) if self.trace else 0
        d.timeout_ns = int(timeout_ms * 1e6)
        d.M, d.N, d.K = self.M, self.N, self.K
        d.ldo = self.out[0].stride(0)
        d.col_off_per_rank = int(col_off_per_rank)
        d.world, d.num_local, d.rank0, d.ctas_per_rank = self.world, self.num_local, self.rank0, self.ctas_per_rank
        d.mode, d.group_m, d.ag, d.ag_slices = MODES[mode], int(group_m), int(self.ag), int(ag_slices)
        self.group_m = int(group_m)
        d.store_all = int(self.store_all)
        d.tile_flag_base = FLAG_HEADER
        d.ag_flag_base = FLAG_HEADER + tile_flags
        d.device = c0.gpu_id
        d.cta_group = cta_group
        d.push_partials = int(self.push)
        d.part_slot_rows = getattr(self, "_slot_rows", 0)
        d.ksplit = self.ksplit
        d.rs_rows = self.rs_rows
        d.rs_bcast = int(pl.bcast)
        self.bcast = pl.bcast
        d.dp_tiles = self.dp_tiles if self.sk_units else -1
        d.sk_units = self.sk_units
        d.sk_flag_base = FLAG_HEADER + tile_flags + self.world * chunks_per_shard
        d.sk_slots = pl.sk_slots
        d.ws_off = c0.offset_of(self.workspace[0]) if self.workspace else 0
        d.bn, d.dtype = pl.bn, DTYPES[_TORCH_DTYPES[self.dtype]]
        d.tail_tiles, d.tail_split = pl.tail_tiles, pl.tail_split
        self.bn, self.tail_tiles, self.tail_split = pl.bn, pl.tail_tiles, pl.tail_split
        d.c_off = c_off if self.store_all else 0
        # atomic all-reduce of a short matrix: the kernel clears the output itself (one launch less); a large output
        # is cleared faster by a launch of its own than by CTAs that should already be loading operands
        out_bytes = self.out[0].shape[0] * self.out[0].stride(0) * self.out[0].element_size()
        self._zero_in_kernel = (mode == "reduce" and self.store_all and out is None
                                and self.out[0].is_contiguous() and out_bytes <= ZERO_IN_KERNEL_MAX_BYTES)
        d.zero_bytes = out_bytes if self._zero_in_kernel else 0
        # two-shot on a heap bound to an NVLS multicast object: the switch sums and broadcasts
        mc = int(getattr(c0, "mc_base", 0) or 0)
        self.nvls = (bool(mc) and (mode == "two_shot" or pl.bcast) and self.num_local == 1 and out is None
                     and nvls is not False)
        if nvls and not self.nvls:
            raise RuntimeError("nvls=True needs heap_mode='vmm' with IRIS_NVLS=1, a two-shot variant, one process per GPU")
        # all-scatter pushes: which instructions carry a finished tile to the other ranks
        pk = DEFAULT_PUSH_KIND if push_kind is None else push_kind
        if pk not in PUSH_KINDS:
            raise ValueError(f"push_kind must be one of {sorted(PUSH_KINDS)}")
        if pk == "multimem" and not (mc and self.num_local == 1):
            if push_kind is not None:
                raise RuntimeError("push_kind='multimem' needs heap_mode='vmm' with IRIS_NVLS=1, one process per GPU")
            pk = "tma"
        if not (self.store_all and mode in ("store", "reduce")) or (mode == "reduce" and pk == "stores"):
            if push_kind is not None and pk != "tma":
                raise ValueError(f"push_kind={pk!r} does not apply to mode={mode!r}")
            pk = "tma"
        self.push_kind = pk
        d.push_kind = PUSH_KINDS[pk]
        d.mc_base = mc if (self.nvls or pk == "multimem") else 0
        self.ag_slices = int(ag_slices)
        lib = _lib()
        self._plan = lib.iris_gemm_plan_create(ctypes.byref(d))
        if not self._plan:
            raise RuntimeError("fused GEMM plan: " + lib.iris_gemm_last_error().decode())
        self.ctas_per_rank = lib.iris_gemm_plan_ctas_per_rank(self._plan)  # what fits on the device
        self.calls = 0
        self.launches = 0
        # Construction is collective.  The flags were zeroed on this rank's stream just now; a peer that is already
        # past its own constructor must not launch (and bump this rank's counters) before that has happened.
        if self.num_local == 1 and self.world > 1:
            c0.barrier()

    # every rank of a real multi-process world must call this the same number of times
    def __call__(self, stream=None) -> List[torch.Tensor]:
        c0 = self.ctxs[0]
        st = torch.cuda.current_stream(c0.device).cuda_stream if stream is None else stream
        if self.mode == "reduce" and not self._zero_in_kernel:
            for o in self.out[:self.num_local]:
                o.zero_()  # partial sums are added into the output: it has to start at zero
            self.launches += self.num_local
        # No per-call argument: the kernel keeps the call number (entry-flag value, flag targets, partial-buffer parity)
        # in device memory, so this launch may be recorded by a stream capture and replayed from a CUDA graph.
        self.calls += 1
        rc = _lib().iris_gemm_plan_launch(self._plan, ctypes.c_void_p(st))
        if rc != 0:
            raise RuntimeError("fused GEMM launch: " + _lib().iris_gemm_last_error().decode())
        self.launches += 1
        return self.out

    def trace_records(self, local: int = 0):
        """Per-tile timestamps of the last call in microseconds relative to the earliest one: a list of dicts with
        ``mma_begin, mma_end, epi_begin, epi_end, wait_begin, wait_end, pull_end`` and, in the record of the first
        tile a CTA handles, ``cta_begin, cta_end`` (set-up done / leaving) (the reference's per-tile trace
        JSON, ``examples/common/utils.py:66-128``).  Needs ``trace=True`` at construction."""
        if self.trace is None:
            raise RuntimeError("construct the op with trace=True")
        torch.cuda.synchronize(self.ctxs[0].device)
        t = self.trace[local].cpu()
        names = ["mma_begin", "mma_end", "epi_begin", "epi_end", "wait_begin", "wait_end", "pull_end", "cta_begin",
                 "cta_end"]
        nz = t[t > 0]
        t0 = int(nz.min()) if nz.numel() else 0
        recs = []
        for i in range(t.shape[0]):
            rec = {"record": i, "tile_id": i // self.cta_group, "cta_in_pair": i % self.cta_group}
            for j, nm in enumerate(names):
                v = int(t[i, j])
                rec[nm] = (v - t0) / 1e3 if v else None
            recs.append(rec)
        return recs

    def chrome_trace(self, path: str, local: int = 0) -> None:
        """Write the per-tile timestamps of the last call as a Chrome / Perfetto trace file."""
        import json
        from ..utils.results import tile_trace_to_chrome
        with open(path, "w") as f:
            json.dump(tile_trace_to_chrome(self.trace_records(local), self.rank0 + local), f)

    def resources(self) -> dict:
        """Registers, spill bytes and static shared memory of the kernel this op launches, as reported by ptxas when
        the library was built (the reference records ``n_regs`` / ``n_spills`` of its Triton kernel,
        ``examples/07_gemm_all_scatter/matmul_wrapper.py:152-155``).  Empty when the build record is missing."""
        from .. import _build
        pull = self.mode in ("one_shot", "two_shot")
        want = (f"fused_gemm_kernel<{self.cta_group}, {'true' if pull else 'false'}, "
                f"{DTYPES[_TORCH_DTYPES[self.dtype]]}>")
        for name, res in _build.kernel_resources().items():
            if want in name:
                return dict(res, kernel=want)
        return {}

    def check(self) -> None:
        """Synchronise and raise if a bounded wait of the last calls expired."""
        torch.cuda.synchronize(self.ctxs[0].device)
        for c in self.ctxs:
            c.check_status()

    def close(self) -> None:
        if getattr(self, "_plan", None):
            _lib().iris_gemm_plan_destroy(self._plan)
            self._plan = None

    def rebuild(self) -> "FusedGemm":
        """Recovery after :class:`~iris_b200.context.IrisTimeoutError`.  The flags of an op are cumulative counters
        driven to per-call targets that every rank computes from its own call count; when a bounded wait expired on
        some rank, that rank's kernel left the call half-way and the counters of the ranks no longer agree, so the op
        must not be called again.  Every rank (collectively, like construction) calls ``rebuild()``: the old plan is
        closed and a new op with the same arguments is returned, with fresh, zeroed flags and buffers and a call count
        of zero; its constructor ends in a barrier, after which all ranks may call it.  With ``ag=True`` the rows in
        ``a_full`` have to be written again.  The heap space of the old op is not reused (reset the heap to a mark
        taken before the first construction to get it back)."""
        ctxs, a, bt, mode, kw = self._ctor
        self.close()
        return FusedGemm(ctxs, a, bt, mode, **kw)

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# --------------------------------------------------------------------------------------------------
# convenience constructors for the named workloads
# --------------------------------------------------------------------------------------------------
def gemm_all_scatter(ctxs, a, bt, **kw) -> FusedGemm:
    """``C[M, world * N] = A @ [B_0 | B_1 | ...]``: every rank computes its column block and pushes each
    finished tile into the C of every rank (``examples/07_gemm_all_scatter``)."""
    lst = [ctxs] if isinstance(ctxs, Iris) else list(ctxs)
    world = lst[0].get_num_ranks()
    n = as_kmajor_bt(bt[0]).shape[0]
    return FusedGemm(ctxs, a, bt, "store", store_all=True, c_cols=world * n, col_off_per_rank=n, **kw)


def world_of(ctxs) -> int:
    return (ctxs if isinstance(ctxs, Iris) else list(ctxs)[0]).get_num_ranks()


def auto_all_reduce_variant(m: int, world: int):
    """``(variant, keyword arguments)`` that was fastest for a GEMM + all-reduce with ``m`` rows on ``world`` B200s
    (N = 4096, K = 11008 sharded; 2 and 8 GPUs measured, 4 interpolated):

    * up to 256 rows the time is fixed latencies (launch, one link round trip for the data, one for the arrival
      count): the atomic form has the fewest steps.  A single row block leaves most SMs idle, so narrow tiles
      (``bn``) or, while the tile is only a few rows, K pieces (``ksplit``: every piece adds a full tile into every
      rank, so it multiplies the traffic by ``ksplit`` and only pays for the shortest matrices);
    * taller matrices are bound by the link: on 2 GPUs all forms move the same bytes and one-shot has the fewest
      steps; on more GPUs only the two-shot form has the traffic of a library all-reduce, 2 (W - 1) / W partials.
    """
    if m <= 256:
        if world <= 2:
            return "atomic", dict(bn=256, ksplit=8 if m <= 64 else 4)
        return ("atomic", dict(bn=128, ksplit=4)) if m <= 64 else ("atomic", dict(bn=64))
    return ("one_shot", {}) if world <= 2 else ("two_shot", {})


def gemm_all_reduce(ctxs, a, bt, variant: str = "one_shot", **kw) -> FusedGemm:
    """``C[M, N] = sum over ranks of A_r @ B_r`` (K sharded).  ``variant``: ``"atomic"``
    (``examples/08_gemm_atomics_all_reduce``), ``"one_shot"`` (``examples/09_gemm_one_shot_all_reduce``),
    ``"two_shot"`` (each tile summed by one owner rank, which fetches the partials and pushes the result: the traffic
    of a library all-reduce) or ``"two_shot_push"`` (the same traffic made of one-way pushes only: partial tiles are
    pushed to the rank that keeps their rows, as in :func:`gemm_reduce_scatter`, and the keeper writes the summed rows
    to every rank; needs ``M`` to be a multiple of ``world x 128``)."""
    if variant == "auto":
        variant, auto_kw = auto_all_reduce_variant(a[0].shape[0], world_of(ctxs))
        kw = dict(auto_kw, **kw)
    if variant == "atomic":
        return FusedGemm(ctxs, a, bt, "reduce", store_all=True, **kw)
    if variant in ("one_shot", "two_shot"):
        return FusedGemm(ctxs, a, bt, variant, **kw)
    if variant == "two_shot_push":
        return FusedGemm(ctxs, a, bt, "one_shot", reduce_scatter=True, bcast=True, **kw)
    raise ValueError("variant must be 'auto', 'atomic', 'one_shot', 'two_shot' or 'two_shot_push'")


def gemm_reduce_scatter(ctxs, a, bt, **kw) -> FusedGemm:
    """``C_r[M / world, N] = rows r of (sum over ranks of A_q @ B_q)`` (K sharded): the row-parallel projection of a
    sequence-parallel layer, where every rank goes on with its own token rows only.  Each partial tile crosses the
    link once, to the rank that keeps its rows, in an order that gives every keeper one sender at a time; the keeper
    sums the ``world`` slots from local memory in fp32.  ``op.out[l]`` is the kept ``[M / world, N]`` block.  (The
    reference stops at all-reduce, ``examples/08_gemm_atomics_all_reduce`` and ``09_gemm_one_shot_all_reduce``; its
    baseline of this collective is ``examples/benchmark/reference/reduce_scatter.py``.)"""
    return FusedGemm(ctxs, a, bt, "one_shot", reduce_scatter=True, **kw)


def all_gather_gemm(ctxs, M: int, bt, **kw) -> FusedGemm:
    """``C_r[M, N_r] = all_gather(A rows) @ B_r``: peers' rows are pushed into ``op.a_full`` by the kernel's
    communication warps while the tiles of rows already present are computed (no counterpart in the reference)."""
    return FusedGemm(ctxs, None, bt, "store", M=M, ag=True, **kw)


_private_ctx = {}


def gemm(a: torch.Tensor, bt: torch.Tensor, out: Optional[torch.Tensor] = None,
         cta_group: Optional[int] = None, bn: Optional[int] = None, tail_split: Optional[bool] = None) -> torch.Tensor:
    """Single-GPU ``a @ bt.T`` on the tcgen05 kernel (world of one, no communication): bf16, fp16, float32 (as tf32)
    or int8 (the low 8 bits of the integer sums)."""
    dev = a.device
    ctx = _private_ctx.get(dev)
    if ctx is None:
        with torch.cuda.device(dev):
            ctx = Iris.local_world(1, heap_size=64 << 20, backend="cuda", device=dev.index)[0]
        _private_ctx[dev] = ctx
    n = as_kmajor_bt(bt).shape[0]
    if out is None:
        out = torch.empty((a.shape[0], n), dtype=a.dtype, device=dev)
    mark = ctx.mark()
    op = FusedGemm(ctx, [a], [bt], "store", out=[out], cta_group=cta_group, bn=bn, tail_split=tail_split)
    op()
    op.close()
    torch.cuda.current_stream(dev).synchronize()  # the plan's flags and workspace are released just below
    ctx.reset(mark)
    return out


# Names of the fused algorithms (the reference keeps them as Triton constexprs, examples/common/utils.py:13-19).
ALGORITHMS = ("all_scatter", "all_gather", "atomic", "one_shot", "two_shot", "reduce_scatter")


class matmul(torch.autograd.Function):
    """``matmul.apply(op)``: run a prepared :class:`FusedGemm` as an autograd Function (forward only), the calling
    convention of the reference's wrappers (``examples/07_gemm_all_scatter/matmul_wrapper.py:161-219``).
    ``matmul.set_debug(True)`` prints the schedule the way the reference prints its Stream-K bookkeeping (:94-103)."""

    _debug = False

    @staticmethod
    def set_debug(debug: bool) -> None:
        matmul._debug = bool(debug)

    @staticmethod
    def forward(ctx, op: "FusedGemm", stream=None):
        if matmul._debug:
            print(f"[iris_b200.matmul] mode={op.mode} M={op.M} N={op.N} K={op.K} world={op.world} "
                  f"cta_group={op.cta_group} ctas/rank={op.ctas_per_rank} tiles={op.total_tiles} "
                  f"whole_tiles={op.dp_tiles} stream_k_units={op.sk_units} ksplit={op.ksplit} push={op.push} "
                  f"tile={BM * op.cta_group}x{op.bn} tail={op.tail_tiles}x{op.tail_split} push_kind={op.push_kind}")
        out = op(stream)
        return out[0] if len(out) == 1 else tuple(out)

    @staticmethod
    def backward(ctx, *grads):
        raise NotImplementedError("the fused GEMM + collective operators are forward-only, as in the reference")
