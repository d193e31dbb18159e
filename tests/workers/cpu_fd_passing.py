"""Worker: the native file-descriptor exchange (SCM_RIGHTS over abstract Unix sockets, csrc/runtime/iris_runtime.cpp)
that the VMM heap uses to hand allocation handles to the other ranks — exercised here with ordinary files."""
import ctypes
import os
import sys
import tempfile

from iris_b200 import _native
from iris_b200.parallel import bootstrap


def main():
    comm = bootstrap.init_from_env()
    rank, world = comm.rank, comm.world
    rt = _native.runtime()
    token = comm.broadcast_object(f"t{os.getpid()}", 0)
    f = tempfile.TemporaryFile()
    f.write(f"hello from {rank}".encode())
    f.flush()
    sock = rt.iris_rt_fd_listen(f"iris_b200_test_{token}_{rank}".encode())
    assert sock >= 0, rt.iris_rt_last_error()
    comm.barrier()
    for peer in range(world):
        if peer != rank:
            assert rt.iris_rt_fd_send(f"iris_b200_test_{token}_{peer}".encode(), f.fileno(), rank) == 0
    got = {}
    for _ in range(world - 1):
        tag = ctypes.c_int(-1)
        fd = rt.iris_rt_fd_recv(sock, 10000, ctypes.byref(tag))
        assert fd >= 0, rt.iris_rt_last_error()
        # the received descriptor shares the sender's open file (and its offset, also with the other receivers):
        # read by position
        got[tag.value] = os.pread(fd, 100, 0).decode()
        os.close(fd)
    rt.iris_rt_fd_close(sock)
    assert got == {p: f"hello from {p}" for p in range(world) if p != rank}, got
    # nothing arrives any more: the receive must time out, not block
    sock2 = rt.iris_rt_fd_listen(f"iris_b200_test_{token}_late_{rank}".encode())
    assert rt.iris_rt_fd_recv(sock2, 300, None) < 0
    rt.iris_rt_fd_close(sock2)
    # a peer that never opened its socket: the send is refused with an error code, nothing blocks
    assert rt.iris_rt_fd_send(f"iris_b200_test_{token}_nobody".encode(), f.fileno(), rank) != 0
    assert rt.iris_rt_last_error()
    comm.barrier()
    comm.shutdown()
    print(f"rank {rank}: OK")


if __name__ == "__main__":
    main()
    sys.exit(0)
