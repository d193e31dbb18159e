"""See the package docstring.  Only what MpiBootstrap uses: COMM_WORLD.{Get_rank, Get_size, allgather, bcast, Barrier,
Ibarrier, Split_type} and COMM_TYPE_SHARED."""
import datetime
import os
import pickle
import tempfile

from torch.distributed import FileStore

COMM_TYPE_SHARED = 1


class _Request:
    def __init__(self, comm, key):
        self._comm, self._key = comm, key

    def Test(self):
        return int(self._comm._store.add(self._key, 0)) >= self._comm._size


class _Comm:
    def __init__(self):
        self._rank = int(os.environ.get("RANK", "0"))
        self._size = int(os.environ.get("WORLD_SIZE", "1"))
        # a file store named after the launcher (parent process) and its rendezvous port: no second port to collide on
        path = os.path.join(tempfile.gettempdir(),
                            f"iris_fake_mpi_{os.getppid()}_{os.environ.get('MASTER_PORT', '0')}")
        self._store = FileStore(path, self._size)
        self._store.set_timeout(datetime.timedelta(seconds=60))
        self._seq = 0

    def _next(self, what):
        self._seq += 1
        return f"{what}/{self._seq}"

    def Get_rank(self):
        return self._rank

    def Get_size(self):
        return self._size

    def allgather(self, obj):
        key = self._next("allgather")
        self._store.set(f"{key}/{self._rank}", pickle.dumps(obj))
        return [pickle.loads(self._store.get(f"{key}/{r}")) for r in range(self._size)]

    def bcast(self, obj, root=0):
        key = self._next("bcast")
        if self._rank == root:
            self._store.set(key, pickle.dumps(obj))
            return obj
        return pickle.loads(self._store.get(key))

    def Ibarrier(self):
        key = self._next("barrier")
        self._store.add(key, 1)
        return _Request(self, key)

    def Barrier(self):
        import time
        req = self.Ibarrier()
        while not req.Test():
            time.sleep(0.0005)

    def Split_type(self, kind):
        assert kind == COMM_TYPE_SHARED
        return self   # all ranks of these tests share one node


class _Lazy:
    """COMM_WORLD connects on first use, as MPI initialises on import of the real module."""
    _comm = None

    def __getattr__(self, name):
        if _Lazy._comm is None:
            _Lazy._comm = _Comm()
        return getattr(_Lazy._comm, name)


COMM_WORLD = _Lazy()
