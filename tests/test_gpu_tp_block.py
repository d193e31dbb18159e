"""Tensor-parallel decoder stack (fused all-gather->GEMM and GEMM->all-reduce) against the unsharded fp32 oracle,
with the ranks simulated on one GPU; and the element-wise kernels against PyTorch."""
import pytest
import torch

import iris_b200 as iris
from iris_b200.models.tp_block import TPConfig, TPDecoder, reference_forward
from iris_b200.ops import elementwise as E

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)


def test_elementwise_kernels():
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((300, 1024), generator=g, device="cuda").to(torch.bfloat16)
    w = (1 + 0.1 * torch.randn(1024, generator=g, device="cuda")).to(torch.bfloat16)
    big = torch.zeros((600, 1024), dtype=torch.bfloat16, device="cuda")
    out = E.rmsnorm(x, w, big[100:400], 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (out.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    assert float(big[:100].abs().sum()) == 0 and float(big[400:].abs().sum()) == 0
    gu = torch.randn((300, 2 * 1376), generator=g, device="cuda").to(torch.bfloat16)
    h = torch.empty((300, 1376), dtype=torch.bfloat16, device="cuda")
    E.swiglu(gu, h)
    ref = torch.nn.functional.silu(gu[:, :1376].float()) * gu[:, 1376:].float()
    assert (h.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item() + 1e-3
    y = torch.randn((300, 1024), generator=g, device="cuda").to(torch.bfloat16)
    x2 = x.clone()
    E.residual_add(x2, y)
    assert torch.equal(x2, (x.float() + y.float()).to(torch.bfloat16))


@pytest.mark.parametrize("variant", ["one_shot", "two_shot", "atomic", "reduce_scatter"])
@pytest.mark.parametrize("world", [2, 4])
def test_tp_decoder_emulated(world, variant):
    cfg = TPConfig(hidden=512, n_heads=4, head_dim=128, intermediate=1024, n_layers=2, batch=2, seq=512, seed=4)
    ranks = iris.Iris.local_world(world, heap_size=192 << 20)
    model = TPDecoder(ranks, cfg, variant=variant, ag_slices=4)
    g = torch.Generator(device="cuda").manual_seed(7)
    x = torch.randn((cfg.tokens, cfg.hidden), generator=g, device="cuda").to(torch.bfloat16)
    ts = cfg.tokens // world
    for rep in range(2):  # the second pass reuses every flag and buffer
        shards = [x[r * ts:(r + 1) * ts].clone() for r in range(world)]
        model.forward(shards)
        model.check()
        got = torch.cat(shards, 0).float()
        ref = reference_forward(x, cfg)
        err = (got - ref).abs()
        assert err.mean().item() < 2e-2 and err.max().item() < 0.25, (rep, err.mean().item(), err.max().item())
    model.close()
    ranks[0].close()
