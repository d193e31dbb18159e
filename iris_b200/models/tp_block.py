"""Tensor-parallel Llama-style decoder stack built on the fused GEMM + collective kernels.

Per layer, on every rank (W ranks, tokens T = batch x seq, hidden H, SwiGLU width I):

    x_shard [T/W, H]   (the residual stream is token-sharded between blocks)
      RMSNorm -> written straight into this rank's rows of the gathered activation matrix
      all-gather -> GEMM   qkv   = gather(xn) [T, H]   @ Wqkv_r^T [H, 3H/W]       (column-parallel, fused)
      causal attention over this rank's H/W / head_dim heads
      GEMM -> all-reduce   o     = attn [T, H/W]       @ Wo_r^T   [H/W, H]        (row-parallel, fused)
      x_shard += o[own rows]
      RMSNorm -> gathered matrix; all-gather -> GEMM  gate|up = gather(xn) @ Wgu_r^T [H, 2I/W]
      SwiGLU; GEMM -> all-reduce  down = h [T, I/W] @ Wd_r^T [I/W, H];  x_shard += down[own rows]

The reference has no model code; its fused kernels are the ingredients (``docs/FINEGRAINED_OVERLAP.md:23-31``
describes the row-parallel and column-parallel splits).  ``TPDecoderBaseline`` is the same network with cuBLAS GEMMs
and NCCL ``all_gather_into_tensor`` / ``all_reduce``; ``reference_forward`` is the unsharded fp32 oracle.
The attention core of the fused stack is this repository's tcgen05 kernel (``iris_b200/ops/attention.py``) whenever
the head dimension is 128 and the sequence length a multiple of 128; the baseline stack (and the fused one for other
shapes, or with ``attention="sdpa"``) calls ``torch.nn.functional.scaled_dot_product_attention``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Union

import torch
import torch.nn.functional as F

from ..context import Iris
from ..ops import attention as A
from ..ops import elementwise as E
from ..ops import gemm as G


@dataclass
class TPConfig:
    hidden: int = 4096
    n_heads: int = 32
    head_dim: int = 128
    intermediate: int = 11008
    eps: float = 1e-6
    n_layers: int = 4
    batch: int = 8
    seq: int = 2048
    seed: int = 4
    std: float = 0.02

    @property
    def tokens(self) -> int:
        return self.batch * self.seq


def layer_weights(cfg: TPConfig, layer: int, device) -> dict:
    """Full (unsharded) bf16 weights of one layer, identical on every rank: N(0, std) from ``seed + layer``."""
    g = torch.Generator(device=device).manual_seed(cfg.seed * 1000 + layer)
    H, I = cfg.hidden, cfg.intermediate

    def w(rows, cols):
        return (torch.randn((rows, cols), generator=g, device=device) * cfg.std).to(torch.bfloat16)
    return {"wq": w(H, H), "wk": w(H, H), "wv": w(H, H), "wo": w(H, H), "wg": w(I, H), "wu": w(I, H), "wd": w(H, I),
            "norm1": torch.ones(H, device=device, dtype=torch.bfloat16),
            "norm2": torch.ones(H, device=device, dtype=torch.bfloat16)}


def shard_weights(full: dict, cfg: TPConfig, rank: int, world: int) -> dict:
    H, I = cfg.hidden, cfg.intermediate
    hs, is_ = H // world, I // world
    r0, r1 = rank * hs, (rank + 1) * hs
    i0, i1 = rank * is_, (rank + 1) * is_
    return {
        "wqkv": torch.cat([full["wq"][r0:r1], full["wk"][r0:r1], full["wv"][r0:r1]], 0).contiguous(),  # [3H/W, H]
        "wo": full["wo"][:, r0:r1].contiguous(),                                                     # [H, H/W]
        "wgu": torch.cat([full["wg"][i0:i1], full["wu"][i0:i1]], 0).contiguous(),                      # [2I/W, H]
        "wd": full["wd"][:, i0:i1].contiguous(),                                                     # [H, I/W]
        "norm1": full["norm1"], "norm2": full["norm2"]}


def attention(qkv: torch.Tensor, cfg: TPConfig, heads_local: int, out: torch.Tensor) -> torch.Tensor:
    """Causal self-attention over the local heads.  qkv: [T, 3 * heads_local * d]; out: [T, heads_local * d]."""
    B, S, d = cfg.batch, cfg.seq, cfg.head_dim
    hl = heads_local * d
    q = qkv[:, :hl].view(B, S, heads_local, d).transpose(1, 2)
    k = qkv[:, hl:2 * hl].view(B, S, heads_local, d).transpose(1, 2)
    v = qkv[:, 2 * hl:].view(B, S, heads_local, d).transpose(1, 2)
    o = F.scaled_dot_product_attention(q, k, v, is_causal=True)
    out.view(B, S, heads_local, d).copy_(o.transpose(1, 2))
    return out


def attention_iris(qkv: torch.Tensor, cfg: TPConfig, heads_local: int, out: torch.Tensor, status=None) -> torch.Tensor:
    """The same on the tcgen05 kernel: reads Q, K, V straight out of the projection's output, writes ``out`` in place
    (no transposes, no copies)."""
    return A.attention_fwd(qkv, out, cfg.batch, cfg.seq, heads_local, causal=True, status=status)


class TPDecoder:
    """Fused implementation.  ``ctxs``: one ``Iris`` (one process per GPU) or all members of ``Iris.local_world``.
    ``variant``: how the row-parallel projections reduce (an all-reduce variant of ``gemm_all_reduce``, ``"auto"``, or
    ``"reduce_scatter"``); ``attention``: ``"iris"`` (own kernel, when the shape allows) or ``"sdpa"``."""

    def __init__(self, ctxs: Union[Iris, Sequence[Iris]], cfg: TPConfig, variant: str = "two_shot", ag_slices: int = 8,
                 attention: str = "iris"):
        self.ctxs: List[Iris] = [ctxs] if isinstance(ctxs, Iris) else list(ctxs)
        self.cfg = cfg
        c0 = self.ctxs[0]
        self.world = c0.get_num_ranks()
        self.ranks = [c.get_rank() for c in self.ctxs]
        dev = c0.device
        W, T, H, I = self.world, cfg.tokens, cfg.hidden, cfg.intermediate
        if cfg.n_heads % W or I % W or T % W or (I // W) % 8:
            raise ValueError("heads, intermediate size and tokens must divide by the number of ranks")
        # "reduce_scatter": the row-parallel projections deliver only this rank's token rows (all the layer uses)
        self.scatter = variant == "reduce_scatter"

        def row_parallel(a, bt):
            if self.scatter:
                return G.gemm_reduce_scatter(self.ctxs, a, bt)
            return G.gemm_all_reduce(self.ctxs, a, bt, variant=variant)
        self.heads_local = cfg.n_heads // W
        self.own_attention = attention == "iris" and cfg.head_dim == A.HEAD_DIM and cfg.seq % 128 == 0
        self.ts = T // W
        nl = len(self.ctxs)
        self.attn = [torch.empty((T, H // W), dtype=torch.bfloat16, device=dev) for _ in range(nl)]
        self.h = [torch.empty((T, I // W), dtype=torch.bfloat16, device=dev) for _ in range(nl)]
        self.layers = []
        for layer in range(cfg.n_layers):
            full = layer_weights(cfg, layer, dev)
            sh = [shard_weights(full, cfg, r, W) for r in self.ranks]
            del full
            ops = {
                "w": sh,
                "qkv": G.all_gather_gemm(self.ctxs, T, [s["wqkv"] for s in sh], ag_slices=ag_slices),
                "o": row_parallel(self.attn, [s["wo"] for s in sh]),
                "gu": G.all_gather_gemm(self.ctxs, T, [s["wgu"] for s in sh], ag_slices=ag_slices),
                "down": row_parallel(self.h, [s["wd"] for s in sh]),
            }
            self.layers.append(ops)
        self.kernel_launches = 0

    def rows(self, local: int) -> slice:
        r = self.ranks[local]
        return slice(r * self.ts, (r + 1) * self.ts)

    def forward(self, x_shards: Sequence[torch.Tensor], timers=None) -> Sequence[torch.Tensor]:
        """``x_shards[l]``: [T/W, H] bf16 of local rank l; updated in place and returned.  ``timers``: optional
        callable ``timers(name)`` invoked before every phase (per-phase breakdowns with CUDA events)."""
        cfg, nl = self.cfg, len(self.ctxs)
        n = 0
        tick = timers if timers is not None else (lambda name: None)
        pending = None   # output of the previous layer's down projection, not yet added to the residual stream
        for ops in self.layers:
            tick("norm")
            for l in range(nl):
                dst = ops["qkv"].a_full[l][self.rows(l)]
                if pending is None:
                    E.rmsnorm(x_shards[l], ops["w"][l]["norm1"], dst, cfg.eps)
                else:   # the previous layer's residual add rides along with this layer's first norm
                    E.add_rmsnorm(x_shards[l], pending[l], ops["w"][l]["norm1"], dst, cfg.eps)
            tick("qkv_ag_gemm")
            qkv = ops["qkv"]()
            tick("attention")
            for l in range(nl):
                if self.own_attention:
                    attention_iris(qkv[l], cfg, self.heads_local, self.attn[l], status=self.ctxs[l].status)
                else:
                    attention(qkv[l], cfg, self.heads_local, self.attn[l])
            tick("o_gemm_ar")
            o = ops["o"]()
            tick("norm")
            for l in range(nl):   # residual add and the next norm in one pass, written into the gathered matrix
                E.add_rmsnorm(x_shards[l], o[l] if self.scatter else o[l][self.rows(l)], ops["w"][l]["norm2"],
                              ops["gu"].a_full[l][self.rows(l)], cfg.eps)
            tick("gu_ag_gemm")
            gu = ops["gu"]()
            tick("swiglu")
            for l in range(nl):
                E.swiglu(gu[l], self.h[l])
            tick("down_gemm_ar")
            d = ops["down"]()
            pending = [d[l] if self.scatter else d[l][self.rows(l)] for l in range(nl)]
            n += 4 + 4 * nl     # 4 fused GEMMs; per rank: norm, attention, add+norm, SwiGLU
        tick("norm")
        for l in range(nl):
            E.residual_add(x_shards[l], pending[l])
        n += nl
        tick("end")
        self.kernel_launches += n
        return x_shards

    def capture(self, x_shards: Sequence[torch.Tensor]) -> "torch.cuda.CUDAGraph":
        """Record one forward pass over ``x_shards`` (updated in place, as ``forward`` does) into a CUDA graph and
        return it; ``graph.replay()`` then runs the whole pass, all ranks' collectives included, with one submission
        instead of one launch per kernel.  Every rank captures and replays the same number of times.  The fused
        kernels keep their call numbers (flag targets, buffer parity) in device memory, so a recorded launch is
        valid for every replay and may be mixed with ordinary ``forward`` calls."""
        torch.cuda.synchronize(self.ctxs[0].device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            self.forward(x_shards)
        return graph

    def check(self) -> None:
        torch.cuda.synchronize(self.ctxs[0].device)
        for c in self.ctxs:
            c.check_status()

    def close(self) -> None:
        for ops in self.layers:
            for k in ("qkv", "o", "gu", "down"):
                ops[k].close()


class TPDecoderBaseline:
    """Same network, one process per GPU: cuBLAS GEMMs + NCCL all_gather_into_tensor / all_reduce."""

    def __init__(self, cfg: TPConfig, rank: int, world: int, device, scatter: bool = False):
        self.cfg, self.rank, self.world = cfg, rank, world
        self.scatter = bool(scatter) and world > 1   # reduce_scatter_tensor instead of all_reduce
        T, H, I = cfg.tokens, cfg.hidden, cfg.intermediate
        self.heads_local = cfg.n_heads // world
        self.ts = T // world
        self.w = []
        for layer in range(cfg.n_layers):
            full = layer_weights(cfg, layer, device)
            self.w.append(shard_weights(full, cfg, rank, world))
            del full
        bf = dict(dtype=torch.bfloat16, device=device)
        self.xn = torch.empty((self.ts, H), **bf)
        self.full = torch.empty((T, H), **bf)
        self.qkv = torch.empty((T, 3 * H // world), **bf)
        self.attn = torch.empty((T, H // world), **bf)
        self.part = torch.empty((T, H), **bf)
        self.kept = torch.empty((self.ts, H), **bf)
        self.gu = torch.empty((T, 2 * I // world), **bf)
        self.h = torch.empty((T, I // world), **bf)

    def forward(self, x_shard: torch.Tensor, timers=None) -> torch.Tensor:
        import torch.distributed as dist
        cfg = self.cfg
        tick = timers if timers is not None else (lambda name: None)
        rows = slice(self.rank * self.ts, (self.rank + 1) * self.ts)

        def gather(t):
            if self.world > 1:
                dist.all_gather_into_tensor(self.full, t)
            else:
                self.full.copy_(t)

        def reduce(t):
            """Sum over ranks; returns this rank's token rows of the sum."""
            if self.scatter:
                dist.reduce_scatter_tensor(self.kept, t)
                return self.kept
            if self.world > 1:
                dist.all_reduce(t)
            return t[rows]
        for w in self.w:
            tick("norm")
            E.rmsnorm(x_shard, w["norm1"], self.xn, cfg.eps)
            tick("qkv_ag_gemm")
            gather(self.xn)
            torch.matmul(self.full, w["wqkv"].t(), out=self.qkv)
            tick("attention")
            attention(self.qkv, cfg, self.heads_local, self.attn)
            tick("o_gemm_ar")
            torch.matmul(self.attn, w["wo"].t(), out=self.part)
            kept = reduce(self.part)
            tick("norm")
            E.residual_add(x_shard, kept)
            E.rmsnorm(x_shard, w["norm2"], self.xn, cfg.eps)
            tick("gu_ag_gemm")
            gather(self.xn)
            torch.matmul(self.full, w["wgu"].t(), out=self.gu)
            tick("swiglu")
            E.swiglu(self.gu, self.h)
            tick("down_gemm_ar")
            torch.matmul(self.h, w["wd"].t(), out=self.part)
            kept = reduce(self.part)
            tick("norm")
            E.residual_add(x_shard, kept)
        tick("end")
        return x_shard


def reference_forward(x: torch.Tensor, cfg: TPConfig) -> torch.Tensor:
    """Unsharded fp32 oracle: x [T, H] (any float dtype) -> [T, H] fp32, with the same bf16 weights."""
    dev = x.device
    x = x.float().clone()
    B, S, nh, d = cfg.batch, cfg.seq, cfg.n_heads, cfg.head_dim

    def norm(t, w):
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + cfg.eps) * w.float()
    for layer in range(cfg.n_layers):
        w = layer_weights(cfg, layer, dev)
        xn = norm(x, w["norm1"])
        q = (xn @ w["wq"].float().t()).view(B, S, nh, d).transpose(1, 2)
        k = (xn @ w["wk"].float().t()).view(B, S, nh, d).transpose(1, 2)
        v = (xn @ w["wv"].float().t()).view(B, S, nh, d).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B * S, nh * d)
        x = x + a @ w["wo"].float().t()
        xn = norm(x, w["norm2"])
        hidden = F.silu(xn @ w["wg"].float().t()) * (xn @ w["wu"].float().t())
        x = x + hidden @ w["wd"].float().t()
    return x
