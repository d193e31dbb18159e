"""Start N ranks of a script on this machine: ``python -m iris_b200.launch -np N script.py [args...]``.

Role in the reference: ``mpirun -np N python script.py`` (``README.md:93-100``); neither ``mpirun`` nor
``mpi4py`` is needed here.  Each rank is a child process with ``RANK``, ``LOCAL_RANK``, ``WORLD_SIZE``,
``MASTER_ADDR=127.0.0.1`` and ``MASTER_PORT`` set — the same variables ``torchrun`` sets, so scripts work
under either launcher.  If a rank fails, the others get a grace period to leave on their own (their waits are
bounded); ranks still running after it, or after the time limit, are terminated by process id, and the launcher exits
non-zero.
"""
from __future__ import annotations

import argparse
import os
import socket
import subprocess
import sys
import threading
import time
from typing import List, Optional, Sequence


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(nprocs: int, argv: Sequence[str], timeout_s: Optional[float] = None, env_extra: Optional[dict] = None,
           module: bool = False, capture: bool = False, grace_s: float = 20.0):
    """Run ``python argv...`` as ``nprocs`` ranks.  Returns (exit_code, [per-rank output or None]).

    When a rank fails, the others are given ``grace_s`` seconds to end on their own: every device wait and every
    ``barrier(timeout_s)`` of the package is bounded, so they notice the missing rank and leave with no kernel in
    flight (a rank killed in the middle of a kernel, or while its heap is bound to an NVLink multicast object, can
    disturb the GPUs of the others).  Only ranks still running after that, or after ``timeout_s``, are terminated, by
    process id.  With ``capture`` the ranks' output is drained by reader threads while they run, so a talkative rank
    never blocks on a full pipe."""
    port = free_port()
    procs: List[subprocess.Popen] = []
    chunks: List[List[str]] = [[] for _ in range(nprocs)]
    readers: List[threading.Thread] = []
    for r in range(nprocs):
        env = dict(os.environ)
        env.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(nprocs), LOCAL_WORLD_SIZE=str(nprocs),
                   MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        if env_extra:
            env.update({k: str(v) for k, v in env_extra.items()})
        cmd = [sys.executable] + (["-m"] if module else []) + list(argv)
        p = subprocess.Popen(cmd, env=env, stdout=subprocess.PIPE if capture else None,
                             stderr=subprocess.STDOUT if capture else None, text=capture)
        procs.append(p)
        if capture:
            def pump(stream=p.stdout, sink=chunks[r]):
                for line in stream:
                    sink.append(line)
            t = threading.Thread(target=pump, daemon=True)
            t.start()
            readers.append(t)
    deadline = None if timeout_s is None else time.monotonic() + timeout_s
    code = 0
    grace_end = None
    pending = set(range(nprocs))
    while pending:
        for r in list(pending):
            rc = procs[r].poll()
            if rc is not None:
                pending.discard(r)
                if rc != 0 and code == 0:
                    code = rc
                    grace_end = time.monotonic() + grace_s
        now = time.monotonic()
        timed_out = deadline is not None and now > deadline
        if pending and (timed_out or (grace_end is not None and now > grace_end)):
            if code == 0:
                code = 124  # time limit, as coreutils timeout
            for r in pending:
                procs[r].terminate()
            t_end = time.monotonic() + 5
            for r in pending:
                try:
                    procs[r].wait(max(0.1, t_end - time.monotonic()))
                except subprocess.TimeoutExpired:
                    procs[r].kill()
            break
        time.sleep(0.02)
    for p in procs:
        try:
            p.wait(5)
        except subprocess.TimeoutExpired:
            pass
    for t in readers:
        t.join(5)
    outs = ["".join(c) if capture else None for c in chunks]
    return code, outs


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m iris_b200.launch", description=__doc__.splitlines()[0])
    ap.add_argument("-np", "--nprocs", type=int, default=2)
    ap.add_argument("--timeout", type=float, default=None, help="seconds before all ranks are terminated")
    ap.add_argument("-m", dest="module", action="store_true", help="treat the target as a module name")
    ap.add_argument("target", nargs=argparse.REMAINDER)
    a = ap.parse_args(argv)
    if not a.target:
        ap.error("no script given")
    code, _ = launch(a.nprocs, a.target, timeout_s=a.timeout, module=a.module)
    return code


if __name__ == "__main__":
    sys.exit(main())
