"""MoE routing / dispatch / combine kernels and the expert-parallel FFN node against the plain
PyTorch implementation of the same layer (fp32 reference of bf16 inputs)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def test_router_topk_and_slots():
    from matrix_fsdp_b200.ops import moe_kernels as MK

    torch.manual_seed(0)
    T, E, K = 777, 64, 6
    logits = torch.randn(T, E, device="cuda").bfloat16()
    psum = torch.zeros(E, device="cuda")
    probs, idx, w = MK.router_topk(logits, K, psum)
    ref = torch.softmax(logits.float(), -1)
    rw, ri = ref.topk(K, -1)
    assert torch.allclose(probs, ref, atol=1e-5)
    assert torch.allclose(w, rw, atol=1e-5)
    assert torch.allclose(psum, ref.sum(0), rtol=1e-4)
    assert torch.equal(torch.gather(ref, 1, idx.long()), torch.gather(ref, 1, ri))   # same set up to ties
    slot, counts = MK.assign_slots(idx, E)
    flat = idx.reshape(-1).long()
    assert torch.equal(counts.long(), torch.bincount(flat, minlength=E))
    for e in (0, 17, 63):
        got = slot[flat == e].long()
        assert torch.equal(got, torch.arange(got.numel(), device="cuda"))


def _ffn_case(T, H, E, Fd, K, seed=0):
    torch.manual_seed(seed)
    x = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
    res = (torch.randn(T, H, device="cuda") * 0.5).bfloat16()
    wr = (torch.randn(E, H, device="cuda") * 0.1).bfloat16()
    wgu = (torch.randn(E, 2 * Fd, H, device="cuda") * 0.05).bfloat16()
    wd = (torch.randn(E, H, Fd, device="cuda") * 0.05).bfloat16()
    return x, res, wr, wgu, wd


@pytest.mark.parametrize("T,H,E,Fd,K", [(300, 256, 8, 128, 2), (1024, 512, 64, 192, 6)])
def test_moe_ffn_single_rank_matches_reference(T, H, E, Fd, K):
    from matrix_fsdp_b200.ops import kernels as Kn
    from matrix_fsdp_b200.ops import moe_functional as MF
    from matrix_fsdp_b200.parallel.expert_parallel import ExpertParallelContext

    x, res, wr, wgu, wd = _ffn_case(T, H, E, Fd, K)
    leaves = [t.clone().requires_grad_(True) for t in (x, res, wr, wgu, wd)]
    ep = ExpertParallelContext.get(None, x.device, H, E, K, T)
    y, aux = MF.moe_ffn(leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], ep, K, 0.01)
    dy = (torch.randn(T, H, device="cuda") * 0.1).bfloat16()
    (y.float() * dy.float()).sum().add(aux * 3.0).backward()
    torch.cuda.synchronize()
    Kn.check_status()
    assert int(ep.last_stats[1]) == 0
    refs = [t.float().clone().requires_grad_(True) for t in (x, res, wr, wgu, wd)]
    # route with the kernel's (bf16-logit) choice so both sides use the same experts
    yr, auxr = MF.moe_ffn_reference(refs[0], refs[1], refs[2], refs[3], refs[4], K, 0.01)
    (yr * dy.float()).sum().add(auxr * 3.0).backward()
    assert torch.allclose(aux, auxr, rtol=2e-2, atol=1e-4)
    err = (y.float() - yr).abs()
    # a token whose k-th and (k+1)-th probabilities are within bf16 rounding may pick another expert
    assert (err > 3e-2).float().mean().item() < 0.02, err.max().item()
    for got, ref, name in zip(leaves, refs, ("x", "res", "router", "w_gu", "w_down")):
        rel = (got.grad.float() - ref.grad).norm() / ref.grad.norm().clamp_min(1e-6)
        assert rel.item() < 0.08, (name, rel.item())


def _ep_worker(rank, world):
    import torch.distributed as dist

    from matrix_fsdp_b200.ops import kernels as Kn
    from matrix_fsdp_b200.ops import moe_functional as MF
    from matrix_fsdp_b200.parallel.expert_parallel import ExpertParallelContext

    T, H, E, Fd, K = 512, 256, 8, 128, 2
    x, res, wr, wgu, wd = _ffn_case(T * world, H, E, Fd, K)          # same on every rank
    el = E // world
    mine = slice(rank * T, (rank + 1) * T)
    leaves = [x[mine].clone().requires_grad_(True), res[mine].clone().requires_grad_(True),
              wr.clone().requires_grad_(True), wgu[rank * el:(rank + 1) * el].clone().requires_grad_(True),
              wd[rank * el:(rank + 1) * el].clone().requires_grad_(True)]
    ep = ExpertParallelContext.get(dist.group.WORLD, x.device, H, E, K, T, capacity_factor=float(world))
    torch.manual_seed(5)
    dy = (torch.randn(T * world, H, device="cuda") * 0.1).bfloat16()
    for _ in range(2):                                               # second pass reuses the buffers
        for t in leaves:
            t.grad = None
        y, aux = MF.moe_ffn(*leaves, ep, K, 0.01)
        (y.float() * dy[mine].float()).sum().backward()
    torch.cuda.synchronize()
    Kn.check_status()
    # single-rank run of the whole batch with all experts local
    ep1 = ExpertParallelContext.get(None, x.device, H, E, K, T * world)
    full = [t.clone().requires_grad_(True) for t in (x, res, wr, wgu, wd)]
    yf, _ = MF.moe_ffn(*full, ep1, K, 0.01)
    (yf.float() * dy.float()).sum().backward()
    torch.cuda.synchronize()
    assert torch.allclose(y.float(), yf[mine].float(), atol=2e-2)
    assert torch.allclose(leaves[0].grad.float(), full[0].grad[mine].float(), atol=2e-2)
    for i in (3, 4):
        ref = full[i].grad[rank * el:(rank + 1) * el].float()
        rel = (leaves[i].grad.float() - ref).norm() / ref.norm()
        assert rel.item() < 2e-2, (i, rel.item())


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_moe_ffn_expert_parallel_two_gpus():
    from test_gpu_multi import _run

    _run(_ep_worker, 2)


def test_moe_model_trains_single_gpu():
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from matrix_fsdp_b200.models.moe import MoEConfig, MoEModel, configure_moe_optimizer, shard_moe
    from matrix_fsdp_b200.ops import kernels as Kn

    torch.manual_seed(0)
    cfg = MoEConfig.tiny()
    model = MoEModel(cfg, ep_group=False, dtype=torch.bfloat16).cuda()
    for p in model.expert_parameters():
        assert p.dtype == torch.bfloat16
    shard_moe(model, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32),
              optimizer_policy="mixed_muon_adamw")
    opt = configure_moe_optimizer(model, "mixed_muon_adamw", lr=1e-3, muon_lr=0.02)
    toks = torch.randint(0, cfg.vocab_size, (2, 129), device="cuda")
    losses = []
    for _ in range(6):
        loss = model(toks[:, :-1], toks[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        losses.append(float(loss))
    Kn.check_status()
    assert all(l == l for l in losses)
    assert losses[-1] < losses[0] - 0.1, losses
