"""The CPU back end of the symmetric heap under the thread sanitizer and under the address + undefined-behaviour
sanitizers.  The program (tests/native/cpu_backend_stress.cpp) is compiled together with the back end's source, so
that every access of the back end is instrumented.  The reference has no sanitizer runs at all; these stand where a
device-side race detector would (none is available for the GPU kernels here)."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = [os.path.join(ROOT, "tests", "native", "cpu_backend_stress.cpp"),
       os.path.join(ROOT, "iris_b200", "csrc", "cpu", "iris_cpu_backend.cpp")]
INC = os.path.join(ROOT, "iris_b200", "include")
CSRC = os.path.join(ROOT, "iris_b200", "csrc")   # the schedule arithmetic shared with the kernels


@pytest.mark.parametrize("name,flags,env", [
    ("thread", ["-fsanitize=thread"], {"TSAN_OPTIONS": "halt_on_error=1 exitcode=66"}),
    ("address", ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"],
     {"ASAN_OPTIONS": "detect_leaks=1 exitcode=66", "UBSAN_OPTIONS": "print_stacktrace=1"}),
])
def test_cpu_backend_is_clean_under(name, flags, env, tmp_path):
    cxx = shutil.which("g++")
    if cxx is None:
        pytest.skip("no g++")
    exe = str(tmp_path / f"stress_{name}")
    build = subprocess.run([cxx, "-std=c++17", "-O1", "-g", *flags, "-I", INC, "-I", CSRC, *SRC, "-o", exe, "-pthread",
                            "-lrt"],
                           capture_output=True, text=True, timeout=300)
    if build.returncode != 0 and ("cannot find" in build.stderr or "unrecognized" in build.stderr):
        pytest.skip(f"{name} sanitizer runtime is not installed: {build.stderr.strip().splitlines()[-1]}")
    assert build.returncode == 0, build.stderr
    run = subprocess.run([exe], capture_output=True, text=True, timeout=300, env={**os.environ, **env})
    assert run.returncode == 0, run.stdout + run.stderr
    assert "stress OK" in run.stdout
    assert "WARNING: ThreadSanitizer" not in run.stderr and "ERROR: AddressSanitizer" not in run.stderr, run.stderr
    assert "runtime error" not in run.stderr, run.stderr
