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
