"""The tcgen05 attention kernel against a plain PyTorch fp32 softmax(Q K^T / sqrt(d)) V of the same inputs."""
import pytest
import torch

from iris_b200.ops.attention import attention_fwd

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)


def _reference(qkv, batch, seq, heads, causal):
    d = 128
    hl = heads * d
    q = qkv[:, :hl].float().view(batch, seq, heads, d).transpose(1, 2)
    k = qkv[:, hl:2 * hl].float().view(batch, seq, heads, d).transpose(1, 2)
    v = qkv[:, 2 * hl:].float().view(batch, seq, heads, d).transpose(1, 2)
    s = q @ k.transpose(-1, -2) / d ** 0.5
    if causal:
        mask = torch.ones((seq, seq), dtype=torch.bool, device=qkv.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ v
    return o.transpose(1, 2).reshape(batch * seq, hl)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("batch,seq,heads", [(1, 128, 1), (2, 256, 3), (1, 1024, 2), (3, 384, 4)])
def test_attention_matches_fp32_softmax(batch, seq, heads, causal, dtype):
    g = torch.Generator(device="cuda").manual_seed(batch * 1000 + seq + heads)
    wide = torch.randn((batch * seq, 3 * heads * 128 + 64), generator=g, device="cuda").to(dtype)
    qkv = wide[:, 32:32 + 3 * heads * 128]           # a strided view: row pitch larger than the row
    out_full = torch.full((batch * seq, heads * 128 + 8), float("nan"), dtype=dtype, device="cuda")
    out = out_full[:, :heads * 128]
    status = torch.zeros(16, dtype=torch.int32, device="cuda")
    attention_fwd(qkv, out, batch, seq, heads, causal=causal, status=status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, f"a wait of the kernel ran out: {status[:8].tolist()}"
    ref = _reference(qkv, batch, seq, heads, causal)
    # P is rounded to 16 bits before the second product and so is the output: a few 2^-8 of the largest |v| average
    tol = 3 * 2.0 ** -8 * ref.abs().max().item() + 1e-3
    err = (out.float() - ref).abs().max().item()
    assert err <= tol, f"max err {err} > {tol}"
    assert bool(torch.isnan(out_full[:, heads * 128:].float()).all()), "wrote past the row"


def test_attention_large_logits_and_rejects_bad_shapes():
    """Scores far from zero (the running maximum moves from tile to tile) and argument checks."""
    g = torch.Generator(device="cuda").manual_seed(7)
    batch, seq, heads = 1, 512, 2
    qkv = (torch.randn((batch * seq, 3 * heads * 128), generator=g, device="cuda") * 3.0).to(torch.bfloat16)
    out = torch.empty((batch * seq, heads * 128), dtype=torch.bfloat16, device="cuda")
    attention_fwd(qkv, out, batch, seq, heads)
    torch.cuda.synchronize()
    ref = _reference(qkv, batch, seq, heads, True)
    assert (out.float() - ref).abs().max().item() <= 4 * 2.0 ** -8 * ref.abs().max().item() + 1e-3
    with pytest.raises((RuntimeError, ValueError)):
        attention_fwd(qkv[:500], out[:500], 1, 500, heads)       # seq not a multiple of 128
    with pytest.raises(TypeError):
        attention_fwd(qkv.float(), out, batch, seq, heads)
