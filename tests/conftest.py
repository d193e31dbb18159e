"""Shared test set-up.

Markers: ``gpu`` — needs a CUDA device (run with ``-m gpu`` on a B200); everything else runs on CPU, with
multi-process cases started through ``iris_b200.launch`` over gloo on 127.0.0.1.
"""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (sm_100a)")
    config.addinivalue_line("markers", "multigpu: test needs at least 2 CUDA devices")


@pytest.fixture(scope="session", autouse=True)
def _native_libs():
    """Build the native libraries once per session (a no-op when they are up to date)."""
    from iris_b200 import _build
    _build.build_all()
    yield


def run_ranks(nprocs, script_args, timeout_s=120, env=None):
    """Run ``python <script_args>`` as ``nprocs`` ranks; returns (exit code, per-rank output)."""
    from iris_b200.launch import launch
    env = dict(env or {})
    env.setdefault("PYTHONPATH", ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    return launch(nprocs, script_args, timeout_s=timeout_s, env_extra=env, capture=True)
