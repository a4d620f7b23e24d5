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


@pytest.mark.parametrize("n,k", [(128, 256), (384, 512), (1280, 192), (2048, 1024)])
def test_symmetric_gemm_matches_fp32(n, k):
    """Products known to be symmetric compute the upper tiles only and mirror: the full matrix must still
    match an fp32 reference, single and grouped, with and without the ``beta * C`` epilogue."""
    from matrix_fsdp_b200.ops import kernels as K

    torch.manual_seed(n + k)
    x = (torch.randn(n, k, device="cuda") / k ** 0.5).bfloat16()
    ref = x.float() @ x.float().T
    out = torch.full((n, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.gemm(x, x, out=out, symmetric=True)                                      # X Xᵀ
    K.check_status()
    assert torch.isfinite(out.float()).all() and _rel(out, ref) < 1e-2
    assert torch.equal(out.tril(-64), out.T.tril(-64))                         # mirrored part is an exact transpose
    for force_bn in (128, 256):
        o2 = torch.full_like(out, float("nan"))
        K.gemm(x, x, out=o2, symmetric=True, force_bn=force_bn)
        assert _rel(o2, ref) < 1e-2
    gram = out.clone()
    poly = torch.full_like(out, float("nan"))
    K.gemm(gram, gram, out=poly, cin=gram, alpha=2.0, beta=-4.0, symmetric=True)   # bA + cAA
    assert _rel(poly, 2.0 * gram.float() @ gram.float() - 4.0 * gram.float()) < 1e-2
    xt = x.T.contiguous()                                                      # tall orientation: XᵀX from [k, n]
    o3 = torch.full_like(out, float("nan"))
    K.gemm(xt, xt, a_mn_major=True, b_mn_major=True, out=o3, symmetric=True)
    assert _rel(o3, ref) < 1e-2
    K.check_status()


@pytest.mark.parametrize("n,k,G", [(256, 384, 3), (640, 128, 2)])
def test_symmetric_grouped_gemms_match_fp32(n, k, G):
    from matrix_fsdp_b200.ops import kernels as K
    from matrix_fsdp_b200.optim.muon import _tile_groups

    torch.manual_seed(G)
    x = (torch.randn(G, n, k, device="cuda") / k ** 0.5).bfloat16()
    ref = torch.bmm(x.float(), x.float().transpose(1, 2))
    out = torch.full((G * n, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.grouped_gemm_m(x.view(G * n, k), x, _tile_groups(G, n, x.device), out=out, symmetric=True)
    K.check_status()
    assert torch.isfinite(out.float()).all() and _rel(out.view(G, n, n), ref) < 1e-2
    # K-grouped (tall operands stacked along the reduce dimension): out[g] = a_gᵀ a_g
    kk = 192
    a = (torch.randn(G * kk, n, device="cuda") / kk ** 0.5).bfloat16()
    offsets = torch.arange(G + 1, dtype=torch.int32, device="cuda") * kk
    o2 = torch.full((G, n, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    K.grouped_gemm_k(a, a, offsets, G, out=o2, symmetric=True)
    K.check_status()
    a3 = a.view(G, kk, n).float()
    assert torch.isfinite(o2.float()).all() and _rel(o2, torch.bmm(a3.transpose(1, 2), a3)) < 1e-2


def test_newton_schulz_symmetric_products_match_full_products(monkeypatch):
    from matrix_fsdp_b200.optim import muon

    torch.manual_seed(5)
    for shape in ((512, 512), (256, 1024), (1408, 512)):
        g = torch.randn(*shape, device="cuda")
        x = (g / g.norm()).bfloat16().contiguous()
        monkeypatch.setattr(muon, "_symmetric_pays", lambda n, g: True)      # also for these small matrices
        a = muon.newton_schulz_sm100(x.clone(), steps=5)
        ab = muon.newton_schulz_sm100_batched(torch.stack([x, x]), steps=5) if muon.can_batch_newton_schulz(shape) else None
        monkeypatch.setattr(muon, "_symmetric_pays", lambda n, g: False)
        b = muon.newton_schulz_sm100(x.clone(), steps=5)
        assert _rel(a, b) < 2e-2
        if ab is not None:
            assert _rel(ab[0], b) < 2e-2 and _rel(ab[1], b) < 2e-2
