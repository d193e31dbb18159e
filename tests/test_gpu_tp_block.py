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


@pytest.mark.parametrize("cols", [8, 1024, 1376, 4096, 8192, 16384])
def test_rmsnorm_every_row_length(cols):
    """Row lengths that take each of the kernel's forms (row kept in registers with 1, 2 or 4 vectors per thread; the
    two-pass form for longer rows), with a strided input view and a strided output view."""
    g = torch.Generator(device="cuda").manual_seed(cols)
    wide = torch.randn((70, cols + 64), generator=g, device="cuda").to(torch.bfloat16)
    x = wide[:, 32:32 + cols]
    w = (1 + 0.1 * torch.randn(cols, generator=g, device="cuda")).to(torch.bfloat16)
    out = torch.zeros((70, cols + 8), dtype=torch.bfloat16, device="cuda")
    E.rmsnorm(x, w, out[:, :cols], 1e-6)
    xf = x.float()
    ref = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (out[:, :cols].float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    assert float(out[:, cols:].abs().sum()) == 0


@pytest.mark.parametrize("cols", [8, 1024, 4096, 8192, 16384])
def test_add_rmsnorm_matches_the_two_kernels(cols):
    """Residual add fused with the following norm: the residual stream gets the bf16-rounded sum and the norm is
    taken of that rounded value, exactly what residual_add followed by rmsnorm produce (16384 columns: the fall-back
    to the two kernels)."""
    g = torch.Generator(device="cuda").manual_seed(cols + 1)
    x = torch.randn((70, cols), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.randn((90, cols + 16), generator=g, device="cuda").to(torch.bfloat16)[10:80, 8:8 + cols]
    w = (1 + 0.1 * torch.randn(cols, generator=g, device="cuda")).to(torch.bfloat16)
    x_two, out_two = x.clone(), torch.zeros((70, cols), dtype=torch.bfloat16, device="cuda")
    E.residual_add(x_two, y)
    E.rmsnorm(x_two, w, out_two, 1e-6)
    x_one, big = x.clone(), torch.zeros((100, cols + 8), dtype=torch.bfloat16, device="cuda")
    out_one = E.add_rmsnorm(x_one, y, w, big[20:90, :cols], 1e-6)
    assert torch.equal(x_one, x_two)
    sf = x_two.float()
    ref = sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert (out_one.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    assert (out_one.float() - out_two.float()).abs().max().item() <= 2 ** -7 * ref.abs().max().item()
    assert float(big[:20].abs().sum()) == 0 and float(big[90:].abs().sum()) == 0 and float(big[:, cols:].abs().sum()) == 0


def test_swiglu_extreme_inputs():
    """The sigmoid is computed with ex2 / rcp approximations: large negative gates give 0, large positive ones the
    gate itself, and nothing turns into NaN."""
    gate = torch.tensor([-300.0, -100.0, -88.0, -20.0, -1.0, 0.0, 1.0, 20.0, 100.0, 300.0, 3.0e38, -3.0e38] * 2,
                        device="cuda")[:24]
    up = torch.full((24,), 1.5, device="cuda")
    gu = torch.cat([gate, up]).to(torch.bfloat16).view(1, 48).repeat(5, 1).contiguous()
    h = torch.empty((5, 24), dtype=torch.bfloat16, device="cuda")
    E.swiglu(gu, h)
    gf = gu[:, :24].float()
    ref = torch.nn.functional.silu(gf) * gu[:, 24:].float()
    assert not torch.isnan(h.float()).any()
    fin = torch.isfinite(ref.to(torch.bfloat16).float())
    assert torch.equal(torch.isfinite(h.float()), fin)
    assert torch.allclose(h.float()[fin], ref[fin], rtol=2 ** -7, atol=1e-30)


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
