"""Real multi-GPU runs (one process per GPU over CUDA IPC / NVLink).  Skipped when fewer than 2 GPUs are visible;
the same protocols are covered on one GPU by the single-launch rank emulation in test_gpu_gemm.py."""
import os

import pytest
import torch

from conftest import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
    pytest.skip("needs at least 2 CUDA devices", allow_module_level=True)

W = os.path.join(os.path.dirname(__file__), "workers")


@pytest.mark.parametrize("world", [2, 4, 8])
def test_real_ranks(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    code, outs = run_ranks(world, [os.path.join(W, "gpu_multi.py")], timeout_s=300,
                           env={"NCCL_NVLS_ENABLE": "0"})
    assert code == 0, "\n".join(o or "" for o in outs)
    assert all("OK" in (o or "") for o in outs)


@pytest.mark.parametrize("nvls", ["0", "1"])
def test_vmm_heap(nvls):
    """Heap on CUDA virtual memory management (descriptor passing, contiguous mapping); with nvls=1 also the
    NVLink-switch multicast path when the machine offers it.  Every rank exits normally, between steps."""
    world = min(4, torch.cuda.device_count())
    code, outs = run_ranks(world, [os.path.join(W, "gpu_vmm_nvls.py")], timeout_s=240,
                           env={"IRIS_NVLS": nvls, "NCCL_NVLS_ENABLE": "0"})
    assert code == 0, "\n".join(o or "" for o in outs)
    assert all("VMM OK" in (o or "") for o in outs)


EX = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples")


@pytest.mark.parametrize("script,args", [
    ("00_load/load_bench.py", ["-z", str(1 << 22), "-n", "2", "-d"]),
    ("01_store/store_bench.py", ["-z", str(1 << 22), "-n", "2", "-d"]),
    ("02_all_load/all_load_bench.py", ["-m", str(1 << 20), "-M", str(1 << 22), "-x", "2", "-d", "-p", str(1 << 28)]),
    ("03_all_store/all_store_bench.py", ["-m", str(1 << 20), "-M", str(1 << 22), "-x", "2", "-d", "-p", str(1 << 28)]),
    ("04_atomic_add/atomic_add_bench.py", ["-z", str(1 << 20), "-x", "2", "-w", "1", "-d"]),
    ("04_atomic_add/atomic_add_bench.py", ["-t", "fp16", "-z", str(1 << 20), "-x", "2", "-w", "1", "-d"]),
    ("04_atomic_add/atomic_add_bench.py", ["-t", "bf16", "-z", str(1 << 20), "-x", "2", "-w", "1", "-d"]),
    ("04_atomic_add/atomic_add_bench.py", ["-t", "int32", "-z", str(1 << 20), "-x", "2", "-w", "1", "-d"]),
    ("05_atomic_xchg/atomic_xchg_bench.py", ["-z", str(1 << 20), "-x", "2", "-w", "1", "-d"]),
    ("06_message_passing/message_passing_put.py", ["-n", "3"]),
    ("06_message_passing/message_passing_load_store.py", ["-n", "3"]),
    ("07_gemm_all_scatter/benchmark.py", ["-m", "1024", "-n", "2048", "-k", "512", "-v", "-b", "--num_experiments", "3",
                                          "--num_warmup", "1", "--heap_size", str(1 << 28)]),
    ("07_gemm_all_scatter/benchmark.py", ["-m", "1024", "-n", "2048", "-k", "512", "-v", "-b", "--num_experiments", "3",
                                          "--num_warmup", "1", "--heap_size", str(1 << 28), "--datatype", "fp16",
                                          "--BLK_M", "128", "--BLK_N", "128", "--push_kind", "stores", "--all_gather"]),
    ("07_gemm_all_scatter/benchmark.py", ["-m", "1024", "-n", "2048", "-k", "512", "-v", "-b", "--num_experiments", "3",
                                          "--num_warmup", "1", "--heap_size", str(1 << 28), "--datatype", "fp32"]),
    ("07_gemm_all_scatter/benchmark.py", ["-m", "1024", "-n", "2048", "-k", "512", "-v", "-b", "--num_experiments", "3",
                                          "--num_warmup", "1", "--heap_size", str(1 << 28), "--datatype", "int8",
                                          "--all_gather"]),
    ("08_gemm_atomics_all_reduce/benchmark.py", ["-m", "1024", "-n", "1024", "-k", "1024", "-v", "--heap_size", str(1 << 28)]),
    ("08_gemm_atomics_all_reduce/benchmark.py", ["-m", "128", "-n", "1024", "-k", "2048", "-v", "-b", "--num_experiments", "3",
                                                 "--num_warmup", "1", "--BLK_N", "64", "--ksplit", "2",
                                                 "--heap_size", str(1 << 28)]),
    ("09_gemm_one_shot_all_reduce/benchmark.py", ["-m", "1024", "-n", "1024", "-k", "1024", "-v", "--variant", "two_shot_push",
                                                  "--heap_size", str(1 << 28)]),
    ("09_gemm_one_shot_all_reduce/benchmark.py", ["-m", "64", "-n", "1024", "-k", "1024", "-v", "--variant", "auto",
                                                  "--heap_size", str(1 << 28)]),
    ("09_gemm_one_shot_all_reduce/benchmark.py", ["-m", "128", "-n", "1024", "-k", "1024", "-v", "--heap_size", str(1 << 28)]),
    ("10_tp_block/tp_block.py", ["-v", "--hidden", "512", "--heads", "4", "--intermediate", "1024", "--batch", "2",
                                 "--seq", "512", "--layers", "1", "--heap_size", str(1 << 29)]),
    ("10_tp_block/tp_block.py", ["-v", "--variant", "reduce_scatter", "--hidden", "512", "--heads", "4",
                                 "--intermediate", "1024", "--batch", "2", "--seq", "512", "--layers", "1",
                                 "--heap_size", str(1 << 29)]),
    ("11_gemm_reduce_scatter/benchmark.py", ["-m", "1024", "-n", "1024", "-k", "1024", "-v", "-b", "--num_experiments", "3",
                                             "--num_warmup", "1", "--heap_size", str(1 << 28)]),
])
def test_examples_run_on_two_gpus(script, args):
    """Every example script runs end to end on two ranks with its validation switched on (the reference's example
    test only checks that ``00_load`` does not crash, tests/examples/test_load_bench.py:23-60)."""
    code, outs = run_ranks(2, [os.path.join(EX, script)] + args, timeout_s=240, env={"NCCL_NVLS_ENABLE": "0"})
    text = "\n".join(o or "" for o in outs)
    assert code == 0, text
    assert "FAILED" not in text, text


def test_rank_leaving_between_steps_is_detected_on_the_host():
    """A rank leaves between steps; the survivors notice at the next host barrier (short time limit) and do not
    launch the step that would wait for it.  NVLS is off and the heap is plain CUDA IPC memory."""
    world = min(2, torch.cuda.device_count())
    code, outs = run_ranks(world, [os.path.join(W, "gpu_rank_leaves.py")], timeout_s=120,
                           env={"NCCL_NVLS_ENABLE": "0", "IRIS_NVLS": "0"})
    text = "\n".join(o or "" for o in outs)
    assert code == 0, text
    assert "leaving after step 1" in text and "step 2 not launched" in text, text
