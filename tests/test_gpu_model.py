"""Fused decoder-block node and the sharded Llama step on a GPU, against plain PyTorch math."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("recompute", [False, True])
def test_decoder_block_matches_reference(recompute):
    from matrix_fsdp_b200.models.llama import LlamaBlock, LlamaConfig

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=256, hidden=512, n_layers=1, n_heads=4, head_dim=128, ffn=1408,
                      activation_checkpointing=recompute)
    blk = LlamaBlock(cfg).cuda().bfloat16()
    ref = copy.deepcopy(blk).float()
    x = (torch.randn(2, 256, 512, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    xr = x.detach().float().requires_grad_(True)
    y = blk(x)
    from matrix_fsdp_b200.ops import functional as OF

    cos, sin = OF.rope_tables(256, 128, cfg.rope_theta, x.device)
    yr = ref._forward_reference(xr, cos, sin)
    assert _rel(y, yr) < 2e-2
    g = torch.randn_like(y)
    y.backward(g)
    yr.backward(g.float())
    assert _rel(x.grad, xr.grad) < 3e-2
    for (n, p), (_, pr) in zip(blk.named_parameters(), ref.named_parameters()):
        assert p.grad is not None, n
        assert _rel(p.grad, pr.grad) < 4e-2, n
    from matrix_fsdp_b200.ops import kernels as K

    K.check_status()


@pytest.mark.parametrize("fused_update", [False, True])
def test_sharded_llama_step_world1_direct_grads_and_fused_adamw(fused_update):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from matrix_fsdp_b200.models.llama import LlamaConfig, LlamaModel, shard_llama
    from matrix_fsdp_b200.ops import kernels as K
    from matrix_fsdp_b200.optim import configure_optimizer

    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=1024, hidden=256, n_layers=2, n_heads=2, head_dim=128, ffn=688)
    model = LlamaModel(cfg).cuda()
    ref = copy.deepcopy(model)
    shard_llama(model, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16))
    # fused_update: each unit's AdamW runs on a side stream right after that unit's backward
    opt = configure_optimizer(model, "adamw", lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1,
                              fused_reduce_update=fused_update)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    before = K.launch_count()
    losses, rlosses = [], []
    tok = torch.randint(0, 1024, (2, 129), device="cuda")
    for step in range(4):
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        opt.step()
        opt.zero_grad()
        with torch.autocast("cuda", dtype=torch.bfloat16):
            rl = ref(tok[:, :-1], tok[:, 1:])
        rl.backward()
        ropt.step()
        ropt.zero_grad()
        losses.append(loss.item())
        rlosses.append(rl.item())
    K.check_status()
    assert K.launch_count() - before > 50, "native kernels did not run"
    for a, b in zip(losses, rlosses):
        assert abs(a - b) < 0.05 * abs(b), (losses, rlosses)
    assert losses[-1] < losses[0]
    # sharded fp32 masters track the eager model
    for (n, p), (_, pr) in zip(model.named_parameters(), ref.named_parameters()):
        assert _rel(p, pr) < 2e-2, n
    if fused_update:
        from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

        impls = {e.collective_impl for u in collect_param_groups(model) for e in u.runtime_events if e.collective_impl}
        assert "local_adamw" in impls, impls
