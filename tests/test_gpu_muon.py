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


@pytest.mark.parametrize("shape", [(512, 512), (256, 1024), (1408, 512)])
def test_batched_newton_schulz_matches_per_matrix(shape):
    """Several matrices of one shape through the grouped GEMMs give what each gives alone."""
    from matrix_fsdp_b200.ops import kernels as K
    from matrix_fsdp_b200.optim.muon import (can_batch_newton_schulz, newton_schulz_reference, newton_schulz_sm100,
                                             newton_schulz_sm100_batched)

    if not can_batch_newton_schulz(shape):
        pytest.skip("shape needs 128-row tiles per matrix")
    torch.manual_seed(0)
    g = torch.randn(3, *shape, device="cuda")
    x = torch.stack([(m / m.norm()).bfloat16() for m in g]).contiguous()
    out = newton_schulz_sm100_batched(x.clone(), steps=5)
    K.check_status()
    for i in range(3):
        alone = newton_schulz_sm100(x[i].contiguous(), steps=5)
        assert _rel(out[i], alone) < 1e-2, i
        assert _rel(out[i], newton_schulz_reference(g[i], steps=5)) < 5e-2, i


def test_matrix_muon_batches_same_shape_parameters():
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    torch.manual_seed(2)
    p0s = [torch.randn(256, 512, device="cuda") * 0.02 for _ in range(3)] + [torch.randn(384, 128, device="cuda") * 0.02]
    ps = [torch.nn.Parameter(t.clone()) for t in p0s]
    qs = [torch.nn.Parameter(t.clone()) for t in p0s]
    ours = MatrixMuon(ps, lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5, adjust_lr_fn="original")
    ref = torch.optim.Muon(qs, lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5, adjust_lr_fn="original")
    for _ in range(2):
        for p, q in zip(ps, qs):
            g = torch.randn_like(p)
            p.grad, q.grad = g.clone(), g.clone()
        ours.step()
        ref.step()
    for p, q, p0 in zip(ps, qs, p0s):
        assert _rel(p.detach() - p0, q.detach() - p0) < 5e-2
        assert torch.allclose(ours.state[p]["momentum_buffer"], ref.state[q]["momentum_buffer"], atol=1e-5)
