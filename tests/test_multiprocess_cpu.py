"""Multi-process CPU tests: ranks are child processes meeting over gloo on 127.0.0.1; heaps are POSIX shared
memory mapped by every rank.  These stand in for ``mpirun -np N pytest tests/unittests`` of the reference."""
import os

import pytest

from conftest import run_ranks

W = os.path.join(os.path.dirname(__file__), "workers")


def _ok(code, outs):
    assert code == 0, "\n".join(o or "" for o in outs)


def test_cpu_plumbing_two_ranks():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_plumbing.py")])
    _ok(code, outs)
    assert all("OK" in o for o in outs)


@pytest.mark.parametrize("world", [2, 3])
def test_cpu_plumbing_over_the_mpi_bootstrap(world):
    """``IRIS_BOOTSTRAP=mpi``: the same worker with the control plane on mpi4py's interface (the reference's only
    back end, iris/_mpi_helpers.py:8-51).  mpi4py is not installed here; tests/fakes/mpi4py implements the calls the
    bootstrap makes over a file store, so that its MPI code path runs as real processes."""
    fakes = os.path.join(os.path.dirname(__file__), "fakes")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code, outs = run_ranks(world, [os.path.join(W, "cpu_plumbing.py"), "--expect-bootstrap", "MpiBootstrap"],
                           env={"IRIS_BOOTSTRAP": "mpi", "PYTHONPATH": fakes + os.pathsep + root})
    _ok(code, outs)
    assert all("OK" in o for o in outs)


def test_missing_rank_times_out_over_the_mpi_bootstrap():
    """The timed barrier of the MPI back end (a non-blocking barrier polled against a deadline) reports a rank
    that never arrives."""
    fakes = os.path.join(os.path.dirname(__file__), "fakes")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "missing_rank_at_barrier"], timeout_s=60,
                           env={"IRIS_BOOTSTRAP": "mpi", "PYTHONPATH": fakes + os.pathsep + root})
    _ok(code, outs)
    assert "BootstrapError" in outs[0]


@pytest.mark.parametrize("world", [2, 4])
def test_unit_semantics_all_ranks(world):
    code, outs = run_ranks(world, [os.path.join(W, "cpu_unit_all_ranks.py")], timeout_s=180)
    _ok(code, outs)


def test_message_passing_release_acquire():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "message_passing"])
    _ok(code, outs)


def test_heap_size_mismatch_detected():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "heap_size_mismatch"])
    _ok(code, outs)
    assert all("ValueError" in o for o in outs)


def test_missing_rank_times_out_instead_of_hanging():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "missing_rank_at_barrier"], timeout_s=60)
    _ok(code, outs)
    assert "BootstrapError" in outs[0]


def test_debug_heap_reports_divergent_allocations():
    code, outs = run_ranks(3, [os.path.join(W, "cpu_faults.py"), "divergent_allocation"])
    _ok(code, outs)
    assert all("IrisDivergenceError" in o and "differ across ranks" in o for o in outs)


def test_debug_heap_reports_an_overrun_by_a_peer():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "remote_overrun"])
    _ok(code, outs)
    assert "allocation #2 (1000 bytes of torch.uint8" in outs[1] and "byte 8 past its end is 0x11" in outs[1], outs[1]
    assert "overwritten on rank(s) [1]" in outs[0], outs[0]


def test_a_rank_that_dies_is_noticed_at_the_next_barrier():
    code, outs = run_ranks(3, [os.path.join(W, "cpu_faults.py"), "rank_dies"], timeout_s=60)
    assert code != 0                    # the launcher reports the dead rank's exit code and stops the other ranks
    assert "peer loss detected" in outs[0], outs      # rank 0 (root of the monitored barrier) had time to notice


def test_heap_exhaustion_is_symmetric():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "heap_exhaustion"])
    _ok(code, outs)
    offs = {o.strip().split()[-1] for o in outs}
    assert len(offs) == 1 and all("MemoryError" in o for o in outs), outs


def test_flag_never_set_returns_status():
    code, outs = run_ranks(2, [os.path.join(W, "cpu_faults.py"), "flag_never_set"])
    _ok(code, outs)
    assert all("IrisTimeoutError" in o for o in outs)


def test_launcher_propagates_failure(tmp_path):
    bad = tmp_path / "bad.py"
    bad.write_text("import os, sys, time\nif os.environ['RANK'] == '1':\n    sys.exit(3)\ntime.sleep(30)\n")
    code, _ = run_ranks(2, [str(bad)], timeout_s=20)
    assert code == 3


@pytest.mark.parametrize("world", [2, 3])
def test_native_fd_passing(world):
    """SCM_RIGHTS descriptor exchange of the native runtime (what the VMM heap uses for allocation handles)."""
    code, outs = run_ranks(world, [os.path.join(W, "cpu_fd_passing.py")])
    _ok(code, outs)
