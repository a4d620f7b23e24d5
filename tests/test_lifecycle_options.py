"""World-size-1 lifecycle under the less common options: keeping parameters unsharded, evaluation forwards,
saved-tensor hooks, zero-copy gradient bucket, ignored / tied parameters, input gradients, LR schedulers."""
import copy

import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import FSDPLifecycleState, configure_optimizer, fully_shard, matrix_fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


def _mlp(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(6, 10), nn.Tanh(), nn.Linear(10, 4))


def _x(seed=1, n=3):
    return torch.randn(n, 6, generator=torch.Generator().manual_seed(seed))


def _train_pair(model, ref, opt, ropt, steps=3):
    for s in range(steps):
        x = _x(s)
        model(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()


def _assert_same(model, ref, atol=1e-6):
    for u in collect_param_groups(model):
        u.unshard("check")
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p.detach().float(), q.detach(), atol=atol), n
    for u in collect_param_groups(model):
        u.reshard("check")


def test_reshard_after_forward_false_keeps_parameters_until_backward_ends():
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    fully_shard(model, reshard_after_forward=False)
    unit = model._matrix_fsdp_param_group
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    out = model(_x())
    assert unit.state == FSDPLifecycleState.UNSHARDED
    out2 = model(_x(2))                                   # a second forward before backward is legal here
    (out.sum() + out2.sum()).backward()
    assert unit.state == FSDPLifecycleState.SHARDED
    (ref(_x()).sum() + ref(_x(2)).sum()).backward()
    opt.step(), ropt.step()
    _assert_same(model, ref)


def test_no_grad_forward_leaves_no_hooks_and_reshards():
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    fully_shard(model)
    unit = model._matrix_fsdp_param_group
    with torch.no_grad():
        y = model(_x())
    assert torch.allclose(y, ref(_x()), atol=1e-6)
    assert unit.state == FSDPLifecycleState.SHARDED and unit.full_param_storage_nbytes() == 0
    model.eval()
    y2 = model(_x(3))                                      # grad mode on, but nothing downstream needs it
    assert torch.allclose(y2, ref(_x(3)), atol=1e-6)
    y2.sum().backward()
    assert unit.state == FSDPLifecycleState.SHARDED


@pytest.mark.parametrize("option", ["use_saved_tensor_hooks", "use_zero_copy_grad_bucket"])
def test_runtime_options_do_not_change_the_math(option):
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    matrix_fully_shard(model, **{option: True})
    opt = configure_optimizer(model, "adamw", lr=1e-2, weight_decay=0.0)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    _train_pair(model, ref, opt, ropt)
    _assert_same(model, ref, atol=1e-5)


def test_input_gradients_match_eager():
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    fully_shard(model)
    x1, x2 = _x().requires_grad_(True), _x().requires_grad_(True)
    model(x1).pow(2).sum().backward()
    ref(x2).pow(2).sum().backward()
    assert torch.allclose(x1.grad, x2.grad, atol=1e-6)


def test_ignored_parameters_stay_ordinary_and_may_be_frozen():
    reset_shared_owner_planners()
    model = _mlp()
    model[2].bias.requires_grad_(False)
    ref = copy.deepcopy(model)
    fully_shard(model, ignored_params={model[2].bias, model[2].weight})
    unit = model._matrix_fsdp_param_group
    assert [mp.fqn for mp in unit.registry] == ["0.weight", "0.bias"]
    assert not hasattr(model[2].weight, "_mfsdp_unit_ref")
    opt = configure_optimizer(model, "sgd", lr=0.1)
    extra = torch.optim.SGD([model[2].weight], lr=0.1)      # the upper stack's own optimizer
    ropt = torch.optim.SGD([p for p in ref.parameters() if p.requires_grad], lr=0.1)
    for s in range(2):
        x = _x(s)
        model(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        opt.step(), extra.step(), ropt.step()
        opt.zero_grad(), extra.zero_grad(), ropt.zero_grad()
    _assert_same(model, ref)


def test_tied_parameters_need_an_explicit_opt_in():
    class Tied(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.embed = nn.Embedding(12, 6)
            self.head = nn.Linear(6, 12, bias=False)
            self.head.weight = self.embed.weight

        def forward(self, t):
            return self.head(self.embed(t))

    reset_shared_owner_planners()
    with pytest.raises(NotImplementedError, match="shared parameters"):
        fully_shard(Tied())
    model, ref = Tied(), Tied()
    matrix_fully_shard(model, allow_shared_params=True)
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    t = torch.randint(0, 12, (5,), generator=torch.Generator().manual_seed(0))
    for _ in range(2):
        model(t).pow(2).mean().backward()
        ref(t).pow(2).mean().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    unit = model._matrix_fsdp_param_group
    unit.unshard("check")
    assert model.head.weight.data_ptr() == model.embed.weight.data_ptr()
    assert torch.allclose(model.embed.weight.detach(), ref.embed.weight.detach(), atol=1e-6)
    unit.reshard("check")


def test_lr_scheduler_drives_the_wrapped_optimizer():
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    fully_shard(model)
    opt = configure_optimizer(model, "adamw", lr=1e-2, weight_decay=0.0)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    sched = torch.optim.lr_scheduler.StepLR(opt.optimizer, step_size=1, gamma=0.5)
    rsched = torch.optim.lr_scheduler.StepLR(ropt, step_size=1, gamma=0.5)
    for s in range(3):
        x = _x(s)
        model(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        opt.step(), ropt.step()
        sched.step(), rsched.step()
        opt.zero_grad(), ropt.zero_grad()
    assert opt.param_groups[0]["lr"] == pytest.approx(1e-2 * 0.125)
    _assert_same(model, ref, atol=1e-5)


def test_plain_torch_optimizer_state_dict_round_trip():
    reset_shared_owner_planners()
    model = _mlp()
    fully_shard(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)      # created after sharding: prepared automatically
    for s in range(2):
        model(_x(s)).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    sd = copy.deepcopy(opt.state_dict())
    before = model._matrix_fsdp_param_group.flat_buffer.local_shard.clone()
    model(_x(5)).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()
    opt.load_state_dict(sd)
    assert float(next(iter(opt.state.values()))["step"]) == 2.0
    assert not torch.equal(model._matrix_fsdp_param_group.flat_buffer.local_shard, before)   # weights are not optimizer state


def test_manual_unshard_gives_full_parameters_and_debug_state():
    reset_shared_owner_planners()
    model = _mlp()
    ref = copy.deepcopy(model)
    fully_shard(model)
    unit = model._matrix_fsdp_param_group
    assert model[0].weight.numel() in (0, 60)               # local view while sharded
    unit.unshard()
    assert model[0].weight.shape == (10, 6) and torch.equal(model[0].weight.detach(), ref[0].weight.detach())
    with pytest.raises(RuntimeError):
        unit.assert_optimizer_ready()
    unit.reshard()
    unit.assert_optimizer_ready()
    sd = unit.state_dict()
    assert sd["total_numel"] == sum(p.numel() for p in ref.parameters())
