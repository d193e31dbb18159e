"""Host-side control plane: rank discovery, all-gather of small byte strings, scalar broadcast, barrier.

Role in the reference: ``iris/_mpi_helpers.py:8-51`` (mpi4py: ``init_mpi``, ``mpi_allgather``,
``mpi_broadcast_scalar``, ``world_barrier``).  Neither ``mpirun`` nor ``mpi4py`` is assumed here: ranks are
ordinary processes started by ``torchrun`` or by :mod:`iris_b200.launch`, and they meet through a
``torch.distributed`` *gloo* group (TCP on 127.0.0.1).  Data never moves through this plane; it only carries
handles, base addresses and barriers.
"""
from __future__ import annotations

import datetime
import os
import pickle
from typing import Any, List, Optional

import torch
import torch.distributed as dist


class BootstrapError(RuntimeError):
    pass


class Bootstrap:
    """Interface of a control-plane back end."""

    rank: int = 0
    world: int = 1

    def allgather_bytes(self, payload: bytes) -> List[bytes]:
        raise NotImplementedError

    def broadcast_object(self, obj: Any, root: int) -> Any:
        raise NotImplementedError

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        raise NotImplementedError

    def local_rank(self) -> int:
        return int(os.environ.get("LOCAL_RANK", self.rank))

    def shutdown(self) -> None:
        """Release what the back end created (a process group it initialised itself)."""


class SingleBootstrap(Bootstrap):
    """World of one process (no launcher)."""

    def allgather_bytes(self, payload: bytes) -> List[bytes]:
        return [bytes(payload)]

    def broadcast_object(self, obj: Any, root: int) -> Any:
        if root != 0:
            raise BootstrapError(f"root {root} does not exist in a world of 1")
        return obj

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        return None


class TorchDistBootstrap(Bootstrap):
    """Control plane over a gloo process group.

    When the default group is NCCL-only a gloo group over the same ranks is created once, so that
    handle exchange and host barriers never touch the GPUs.
    """

    def __init__(self, timeout_s: float = 120.0, owns_process_group: bool = False):
        self.owns_process_group = owns_process_group
        if not dist.is_initialized():
            raise BootstrapError("torch.distributed is not initialised")
        self.rank = dist.get_rank()
        self.world = dist.get_world_size()
        self._timeout = datetime.timedelta(seconds=timeout_s)
        if str(dist.get_backend()) == "gloo":
            self._group = dist.group.WORLD
        else:
            # NCCL-only or mixed default group: keep the control plane off the GPUs
            self._group = dist.new_group(backend="gloo", timeout=self._timeout)

    def allgather_bytes(self, payload: bytes) -> List[bytes]:
        out: List[Any] = [None] * self.world
        dist.all_gather_object(out, bytes(payload), group=self._group)
        return out

    def broadcast_object(self, obj: Any, root: int) -> Any:
        if not 0 <= root < self.world:
            raise BootstrapError(f"root {root} outside world of {self.world}")
        box = [obj if self.rank == root else None]
        dist.broadcast_object_list(box, src=root, group=self._group)
        return box[0]

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        if timeout_s is None:
            dist.barrier(group=self._group)
            return
        try:
            dist.monitored_barrier(group=self._group, timeout=datetime.timedelta(seconds=timeout_s))
        except RuntimeError as e:  # a rank did not arrive in time
            raise BootstrapError(f"barrier timed out after {timeout_s} s on rank {self.rank}: {e}") from e


class MpiBootstrap(Bootstrap):
    """Control plane over mpi4py, for launches under ``mpirun`` (the reference's only back end,
    ``iris/_mpi_helpers.py:8-51``).  Used when ``IRIS_BOOTSTRAP=mpi`` and mpi4py is importable."""

    def __init__(self):
        from mpi4py import MPI  # noqa: WPS433 (optional dependency)
        self._mpi = MPI
        self._comm = MPI.COMM_WORLD
        self.rank = self._comm.Get_rank()
        self.world = self._comm.Get_size()

    def allgather_bytes(self, payload: bytes) -> List[bytes]:
        return list(self._comm.allgather(bytes(payload)))

    def broadcast_object(self, obj: Any, root: int) -> Any:
        if not 0 <= root < self.world:
            raise BootstrapError(f"root {root} outside world of {self.world}")
        return self._comm.bcast(obj, root=root)

    def barrier(self, timeout_s: Optional[float] = None) -> None:
        if timeout_s is None:
            self._comm.Barrier()
            return
        import time
        req = self._comm.Ibarrier()
        t0 = time.monotonic()
        while not req.Test():
            if time.monotonic() - t0 > timeout_s:
                raise BootstrapError(f"barrier timed out after {timeout_s} s on rank {self.rank}")
            time.sleep(0.001)

    def local_rank(self) -> int:
        return self._comm.Split_type(self._mpi.COMM_TYPE_SHARED).Get_rank()


def _shutdown_torchdist(self) -> None:
    if self.owns_process_group and dist.is_initialized():
        try:
            dist.destroy_process_group()
        except Exception:
            pass
        self.owns_process_group = False


TorchDistBootstrap.shutdown = _shutdown_torchdist


def init_from_env(timeout_s: float = 120.0) -> Bootstrap:
    """Pick the back end from the environment.

    * ``IRIS_BOOTSTRAP=mpi`` → mpi4py (``mpirun`` launches).
    * ``torch.distributed`` already initialised → use it.
    * ``RANK`` and ``WORLD_SIZE`` set (torchrun / iris_b200.launch) → initialise a process group
      (gloo for CPU tensors, NCCL for CUDA tensors when a GPU is present) on ``MASTER_ADDR`` (default
      127.0.0.1) and use it.
    * otherwise → a world of one.
    """
    if os.environ.get("IRIS_BOOTSTRAP", "").lower() == "mpi":
        try:
            return MpiBootstrap()
        except ImportError as e:
            raise BootstrapError("IRIS_BOOTSTRAP=mpi needs mpi4py") from e
    if dist.is_available() and dist.is_initialized():
        return TorchDistBootstrap(timeout_s)
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        backend = "cpu:gloo,cuda:nccl" if torch.cuda.is_available() else "gloo"
        dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))
        return TorchDistBootstrap(timeout_s, owns_process_group=True)
    return SingleBootstrap()


def dumps(obj: Any) -> bytes:
    return pickle.dumps(obj, protocol=4)


def loads(b: bytes) -> Any:
    return pickle.loads(b)
