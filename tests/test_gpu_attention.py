"""tcgen05 causal attention against an fp32 PyTorch reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ref(qkv, B, S, nH, hd):
    H = nH * hd
    q, k, v = (qkv[:, i * H:(i + 1) * H].float().view(B, S, nH, hd).transpose(1, 2) for i in range(3))
    s = (q @ k.transpose(-1, -2)) / math.sqrt(hd)
    mask = torch.ones(S, S, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.softmax(s, dim=-1) @ v
    return o.transpose(1, 2).reshape(B * S, H), lse


@pytest.mark.parametrize("B,S,nH", [(1, 128, 1), (2, 256, 2), (1, 1024, 4), (2, 384, 3), (1, 200, 2)])
def test_attention_fwd_matches_fp32(B, S, nH):
    from matrix_fsdp_b200.ops import attention as A
    from matrix_fsdp_b200.ops import kernels as K

    assert A.fwd_available(), "attention kernel missing from the kernel library"
    torch.manual_seed(0)
    hd = 128
    qkv = torch.randn(B * S, 3 * nH * hd, device="cuda", dtype=torch.bfloat16)
    out, lse = A.attention_fwd(qkv, B, S, nH, hd)
    torch.cuda.synchronize()
    K.check_status()
    ref_o, ref_lse = _ref(qkv, B, S, nH, hd)
    assert torch.isfinite(out).all()
    assert (out.float() - ref_o).abs().max().item() < 3e-2
    assert (lse - ref_lse).abs().max().item() < 2e-3


def test_attention_fwd_large_scores_rescale():
    """Scores that grow along the key axis force the lazy O rescale to fire."""
    from matrix_fsdp_b200.ops import attention as A
    from matrix_fsdp_b200.ops import kernels as K

    torch.manual_seed(1)
    B, S, nH, hd = 1, 512, 2, 128
    qkv = torch.randn(B * S, 3 * nH * hd, device="cuda", dtype=torch.bfloat16)
    ramp = torch.linspace(0.2, 3.0, S, device="cuda").repeat(B)[:, None]
    qkv[:, nH * hd:2 * nH * hd] = (qkv[:, nH * hd:2 * nH * hd].float() * ramp).bfloat16()
    out, lse = A.attention_fwd(qkv, B, S, nH, hd)
    torch.cuda.synchronize()
    K.check_status()
    ref_o, ref_lse = _ref(qkv, B, S, nH, hd)
    assert (out.float() - ref_o).abs().max().item() < 4e-2
    assert (lse - ref_lse).abs().max().item() < 5e-3


@pytest.mark.parametrize("B,S,nH", [(1, 128, 1), (2, 256, 2), (1, 1024, 2), (2, 384, 3), (1, 200, 2), (2, 130, 1)])
def test_attention_bwd_matches_fp32(B, S, nH):
    from matrix_fsdp_b200.ops import attention as A
    from matrix_fsdp_b200.ops import kernels as K

    assert A.bwd_available(), "attention backward kernel missing from the kernel library"
    torch.manual_seed(2)
    hd = 128
    qkv = torch.randn(B * S, 3 * nH * hd, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(B * S, nH * hd, device="cuda", dtype=torch.bfloat16)
    out, lse = A.attention_fwd(qkv, B, S, nH, hd)
    dqkv = A.attention_bwd(dout, qkv, out, lse, B, S, nH, hd)
    torch.cuda.synchronize()
    K.check_status()
    ref_in = qkv.float().requires_grad_(True)
    ref_o, _ = _ref(ref_in, B, S, nH, hd)
    (ref_g,) = torch.autograd.grad(ref_o, ref_in, dout.float())
    assert torch.isfinite(dqkv).all()
    err = (dqkv.float() - ref_g).abs().max().item()
    assert err < 6e-2 * max(1.0, ref_g.abs().max().item() / 4), err
    rel = (dqkv.float() - ref_g).norm() / ref_g.norm()
    assert rel.item() < 2e-2, rel.item()
