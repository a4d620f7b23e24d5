"""MoE decoder on CPU: expert parallelism over gloo (gather + sum exchange) must reproduce the
single-process model in which every expert is local."""
import torch
import torch.distributed as dist

from dist_utils import run_ranks


def _cfg():
    from matrix_fsdp_b200.models.moe import MoEConfig

    return MoEConfig(vocab_size=128, hidden=64, n_layers=2, n_heads=2, head_dim=32, n_experts=4, expert_ffn=48,
                     top_k=2, max_seq_len=32)


def _tokens():
    g = torch.Generator().manual_seed(0)
    return torch.randint(0, 128, (2, 17), generator=g)


def test_moe_reference_matches_dense_loop():
    from matrix_fsdp_b200.ops.moe_functional import moe_ffn_reference

    torch.manual_seed(0)
    T, H, E, Fd, K = 12, 16, 4, 8, 2
    x = torch.randn(T, H, requires_grad=True)
    wr, wgu, wd = torch.randn(E, H) * 0.3, torch.randn(E, 2 * Fd, H) * 0.2, torch.randn(E, H, Fd) * 0.2
    y, aux = moe_ffn_reference(x, None, wr, wgu, wd, K, 0.01)
    probs = torch.softmax(x @ wr.t(), -1)
    w, idx = probs.topk(K, -1)
    exp = torch.zeros(T, H)
    for t in range(T):
        for k in range(K):
            e = idx[t, k]
            gu = wgu[e] @ x[t]
            exp[t] += w[t, k] * (wd[e] @ (torch.nn.functional.silu(gu[:Fd]) * gu[Fd:]))
    assert torch.allclose(y, exp, atol=1e-5)
    frac = torch.bincount(idx.reshape(-1), minlength=E).float() / (T * K)
    assert torch.allclose(aux, 0.01 * E * (frac * probs.mean(0)).sum(), atol=1e-6)


def _ep_worker(rank, world):
    from matrix_fsdp_b200.models.moe import MoEModel, configure_moe_optimizer, shard_moe

    cfg = _cfg()
    torch.manual_seed(0)
    model = MoEModel(cfg)                       # experts split over the two ranks
    torch.manual_seed(0)
    ref = MoEModel(cfg, ep_group=False)         # every expert local
    assert model.layers[0].experts.w_down.shape[0] == cfg.n_experts // world
    el = cfg.n_experts // world
    for a, b in zip(model.layers, ref.layers):
        assert torch.equal(a.experts.w_gate_up, b.experts.w_gate_up[rank * el:(rank + 1) * el])
    shard_moe(model)
    opt = configure_moe_optimizer(model, "adamw", lr=1e-2, betas=(0.9, 0.95))
    dense_ref = [p for n, p in ref.named_parameters() if ".experts." not in n]
    ropt = torch.optim.AdamW(dense_ref + ref.expert_parameters(), lr=1e-2, weight_decay=0.0, betas=(0.9, 0.95))
    toks = _tokens()
    for step in range(3):
        mine = toks[rank:rank + 1]
        loss = model(mine[:, :-1], mine[:, 1:])
        loss.backward()
        # reference: the two sequences are two data-parallel micro-batches (aux loss is per rank)
        losses = []
        for r in range(world):
            lr_ = ref(toks[r:r + 1, :-1], toks[r:r + 1, 1:])
            (lr_ / world).backward()
            losses.append(lr_.detach())
        assert torch.allclose(loss.detach(), losses[rank], atol=1e-5), (step, loss, losses)
        # expert grads: the EP model sums both ranks' tokens; data-parallel mean needs 1/world
        for p in model.expert_parameters():
            p.grad.div_(world)
        opt.step()
        opt.zero_grad()
        ropt.step()
        ropt.zero_grad()
    for a, b in zip(model.layers, ref.layers):
        assert torch.allclose(a.experts.w_down, b.experts.w_down[rank * el:(rank + 1) * el], atol=2e-5)
        assert torch.allclose(a.experts.w_gate_up, b.experts.w_gate_up[rank * el:(rank + 1) * el], atol=2e-5)
    dist.barrier()


def test_moe_ep_gloo_matches_single_process():
    run_ranks(_ep_worker, 2)


def test_moe_checkpoint_roundtrip_single_process(tmp_path):
    from matrix_fsdp_b200.models.moe import (MoEModel, configure_moe_optimizer, load_moe_checkpoint, save_moe_checkpoint,
                                             shard_moe)

    cfg = _cfg()
    toks = _tokens()

    def make():
        torch.manual_seed(0)
        m = MoEModel(cfg, ep_group=False)
        shard_moe(m)
        return m, configure_moe_optimizer(m, "adamw", lr=1e-2, betas=(0.9, 0.95))

    model, opt = make()
    for _ in range(2):
        model(toks[:, :-1], toks[:, 1:]).backward()
        opt.step()
        opt.zero_grad()
    save_moe_checkpoint(model, str(tmp_path), optimizer=opt)
    model(toks[:, :-1], toks[:, 1:]).backward()
    opt.step()
    opt.zero_grad()
    expect = model(toks[:, :-1], toks[:, 1:]).item()

    model2, opt2 = make()
    load_moe_checkpoint(model2, str(tmp_path), optimizer=opt2)
    model2(toks[:, :-1], toks[:, 1:]).backward()
    opt2.step()
    opt2.zero_grad()
    got = model2(toks[:, :-1], toks[:, 1:]).item()
    assert abs(got - expect) < 1e-5, (got, expect)
