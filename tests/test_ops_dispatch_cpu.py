"""Dispatch and fallbacks of the op layer without a GPU: PyTorch paths for CPU tensors, environment switch,
library loading and signature registration, reference Newton-Schulz, rope tables."""
import math

import pytest
import torch
import torch.nn.functional as F

from matrix_fsdp_b200.ops import functional as OF
from matrix_fsdp_b200.ops import lib


def test_library_loads_and_binds_every_registered_entry_point():
    import matrix_fsdp_b200.ops.attention  # noqa: F401
    import matrix_fsdp_b200.ops.moe_kernels  # noqa: F401
    import matrix_fsdp_b200.parallel.peer  # noqa: F401

    handle = lib.load()
    if handle is None:
        pytest.skip("kernel library not built in this checkout")
    missing = [n for n in lib._SIGNATURES if not hasattr(handle, n)]
    assert missing == []
    assert lib.launch_count() >= 0


def test_env_switch_disables_native_kernels(monkeypatch):
    monkeypatch.setenv("MFSDP_DISABLE_NATIVE_KERNELS", "1")
    assert lib.disabled_by_env()
    from matrix_fsdp_b200.ops import attention

    assert not attention.available()
    monkeypatch.setenv("MFSDP_DISABLE_NATIVE_KERNELS", "0")
    assert not lib.disabled_by_env()


def test_cpu_tensors_take_the_pytorch_paths():
    torch.manual_seed(0)
    x = torch.randn(5, 16, requires_grad=True)
    w = torch.randn(8, 16, requires_grad=True)
    assert not OF.use_native(x)
    y = OF.linear(x, w)
    assert torch.allclose(y, F.linear(x, w))
    g = torch.randn(16)
    n = OF.rms_norm(x, g, 1e-5)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * g
    assert torch.allclose(n, ref, atol=1e-6)
    gu = torch.randn(5, 12)
    assert torch.allclose(OF.swiglu(gu), F.silu(gu[:, :6]) * gu[:, 6:], atol=1e-6)
    logits = torch.randn(7, 11, requires_grad=True)
    target = torch.randint(0, 11, (7,))
    loss = OF.fused_cross_entropy(logits, target)
    assert torch.allclose(loss, F.cross_entropy(logits, target), atol=1e-6)
    loss.backward()
    assert logits.grad is not None
    target[0] = -100
    assert torch.allclose(OF.fused_cross_entropy(logits, target, ignore_index=-100),
                          F.cross_entropy(logits, target, ignore_index=-100), atol=1e-6)


def test_rope_reference_is_a_rotation_and_tables_are_cached():
    cos, sin = OF.rope_tables(9, 8, 10000.0, "cpu")
    assert cos.shape == (9, 4) and OF.rope_tables(9, 8, 10000.0, "cpu")[0] is cos
    x = torch.randn(2, 9, 3, 8)
    y = OF.apply_rope_reference(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)         # rotations keep lengths
    assert torch.allclose(y[:, 0], x[:, 0], atol=1e-6)                        # position 0 is the identity
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 9, 1, 8), torch.randn(1, 9, 1, 8)
    q[:, :] = q[:, :1]
    k[:, :] = k[:, :1]
    rq, rk = OF.apply_rope_reference(q, cos, sin), OF.apply_rope_reference(k, cos, sin)
    d1 = (rq[0, 3, 0] * rk[0, 1, 0]).sum()
    d2 = (rq[0, 7, 0] * rk[0, 5, 0]).sum()
    assert torch.allclose(d1, d2, atol=1e-5)


def test_causal_attention_reference_is_causal():
    torch.manual_seed(0)
    B, S, nH, hd = 1, 6, 2, 4
    qkv = torch.randn(B * S, 3 * nH * hd)
    out = OF.causal_attention_reference(qkv, B, S, nH, hd)
    qkv2 = qkv.clone()
    qkv2[4:] += 1.0                                   # changing later tokens must not move earlier outputs
    out2 = OF.causal_attention_reference(qkv2, B, S, nH, hd)
    assert torch.allclose(out[:4], out2[:4], atol=1e-6) and not torch.allclose(out[4:], out2[4:])


def test_reference_newton_schulz_orthogonalises():
    from matrix_fsdp_b200.optim.muon import adjust_lr, newton_schulz_reference

    torch.manual_seed(0)
    for shape in ((16, 32), (32, 16)):
        g = torch.randn(*shape)
        o = newton_schulz_reference(g, steps=5).float()
        s = torch.linalg.svdvals(o)
        assert s.max() < 1.6 and s.min() > 0.3                 # singular values pulled towards 1
    assert adjust_lr(0.02, None, (8, 4)) == adjust_lr(0.02, "original", (8, 4))      # torch's default
    assert adjust_lr(0.02, "original", (4, 8)) == 0.02
    assert adjust_lr(0.02, "original", (8, 4)) == pytest.approx(0.02 * math.sqrt(2.0))
    assert adjust_lr(0.02, "match_rms_adamw", (8, 4)) == pytest.approx(0.2 * 0.02 * math.sqrt(8))


def test_muon_step_matches_torch_muon_on_cpu():
    if not hasattr(torch.optim, "Muon"):
        pytest.skip("torch.optim.Muon not available")
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    torch.manual_seed(0)
    w1 = torch.nn.Parameter(torch.randn(12, 20))
    w2 = torch.nn.Parameter(w1.detach().clone())
    ours = MatrixMuon([w1], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5)
    theirs = torch.optim.Muon([w2], lr=0.02, momentum=0.95, weight_decay=0.1, ns_steps=5)
    for s in range(3):
        g = torch.randn(12, 20, generator=torch.Generator().manual_seed(s))
        w1.grad, w2.grad = g.clone(), g.clone()
        ours.step()
        theirs.step()
    assert torch.allclose(w1, w2, atol=2e-3), (w1 - w2).abs().max()
    with pytest.raises(ValueError, match="2D"):
        bad = MatrixMuon([torch.nn.Parameter(torch.randn(4))], lr=0.02)
        bad.param_groups[0]["params"][0].grad = torch.randn(4)
        bad.step()


def test_fused_weight_needs_one_storage_not_adjacent_addresses():
    """Row blocks are stacked into one matrix only when they are consecutive views of one storage."""
    buf = torch.arange(6 * 4, dtype=torch.float32)
    a, b = buf[:8].view(2, 4), buf[8:24].view(4, 4)
    fused = OF._fused_weight([a, b])
    assert fused is not None and fused.shape == (6, 4)
    assert torch.equal(fused, buf.view(6, 4))
    # a gap, a swapped order, or a different width break the stacking
    assert OF._fused_weight([b, a]) is None
    assert OF._fused_weight([buf[:8].view(2, 4), buf[12:24].view(3, 4)]) is None
    assert OF._fused_weight([buf[:8].view(2, 4), buf[8:24].view(2, 8)]) is None
    # two separate allocations never fuse, wherever the allocator put them
    x, y = torch.zeros(2, 4), torch.zeros(4, 4)
    assert OF._fused_weight([x, y]) is None

    class FakeAdjacent(torch.Tensor):
        """Second allocation that reports the address right behind the first one."""
        @staticmethod
        def __new__(cls, t, ptr):
            r = torch.Tensor._make_subclass(cls, t)
            r._ptr = ptr
            return r

        def data_ptr(self):
            return self._ptr

    fake = FakeAdjacent(y, x.data_ptr() + x.numel() * 4)
    assert OF._fused_weight([x, fake]) is None


def test_embedding_falls_back_to_torch_off_gpu_and_token_embedding_keeps_the_parameter_name():
    import torch
    from torch import nn

    from matrix_fsdp_b200.models.llama import TokenEmbedding
    from matrix_fsdp_b200.ops import functional as OF

    torch.manual_seed(0)
    emb = TokenEmbedding(50, 16)
    assert isinstance(emb, nn.Embedding) and [n for n, _ in emb.named_parameters()] == ["weight"]
    ids = torch.randint(0, 50, (3, 7))
    out = emb(ids)
    assert torch.equal(out, torch.nn.functional.embedding(ids, emb.weight))
    out.sum().backward()
    ref = torch.zeros(50, 16).index_add_(0, ids.reshape(-1), torch.ones(21, 16))
    assert torch.allclose(emb.weight.grad, ref)
    assert torch.equal(OF.embedding(ids, emb.weight.detach()), out.detach())


def test_newton_schulz_shares_are_balanced_and_deterministic():
    from matrix_fsdp_b200.optim.muon import assign_to_replicas, ns_flops

    shapes = [(4096, 4096)] * 4 + [(11008, 4096)] * 3 + [(256, 256)]
    owner = assign_to_replicas(shapes, 2, 5)
    assert owner == assign_to_replicas(list(shapes), 2, 5) and set(owner) == {0, 1}
    load = [sum(ns_flops(s, 5) for s, o in zip(shapes, owner) if o == r) for r in (0, 1)]
    assert max(load) / min(load) < 1.35
    assert assign_to_replicas(shapes, 1, 5) == [0] * len(shapes)
    # more replicas than matrices: every matrix still has exactly one owner
    assert sorted(assign_to_replicas([(8, 8), (16, 8)], 4, 5)) == [0, 1]
