"""Muon on the tcgen05 path: Newton-Schulz and a full optimizer step against torch's implementation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("shape", [(512, 512), (256, 1024), (1408, 512)])
def test_newton_schulz_matches_reference(shape):
    from matrix_fsdp_b200.ops import kernels as K
    from matrix_fsdp_b200.optim.muon import newton_schulz_reference, newton_schulz_sm100

    torch.manual_seed(0)
    g = torch.randn(*shape, device="cuda")
    ref = newton_schulz_reference(g, steps=5)
    x = (g / g.norm()).bfloat16().contiguous()
    out = newton_schulz_sm100(x, steps=5)
    K.check_status()
    assert out.shape == ref.shape
    assert _rel(out, ref) < 5e-2
    # Newton-Schulz pushes the singular values towards 1 (the input's were ~1/sqrt(n))
    s = torch.linalg.svdvals(out.float())
    assert s.max() < 1.6 and s.median() > 0.5


def test_matrix_muon_step_matches_torch_muon():
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    torch.manual_seed(1)
    p0 = torch.randn(512, 1024, device="cuda") * 0.02
    p = torch.nn.Parameter(p0.clone())
    q = torch.nn.Parameter(p0.clone())
    ours = MatrixMuon([p], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5, adjust_lr_fn="original")
    ref = torch.optim.Muon([q], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5, adjust_lr_fn="original")
    for _ in range(3):
        g = torch.randn_like(p0)
        p.grad, q.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    assert _rel(p.detach() - p0, q.detach() - p0) < 5e-2
    assert torch.allclose(ours.state[p]["momentum_buffer"], ref.state[q]["momentum_buffer"], atol=1e-5)
