"""Optimizer state of sharded parameters, one property per test (single rank, CPU): where the flat optimizers keep
their moments, what the state manager reports about them, and which torch.optim behaviours carry over.  The
reference's counterpart is test/fsdp/test_optim_state.py (14 tests)."""
import copy

import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.optim.flat import FlatShardedAdamW, FlatShardedSGD


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2, bias=False))


def _sharded(kind="adamw", policy=None, **kw):
    reset_shared_owner_planners()
    model = _model()
    fully_shard(model, optimizer_policy=policy)
    return model, configure_optimizer(model, kind, **kw)


def _step(model, opt, seed=1):
    model(torch.randn(3, 4, generator=torch.Generator().manual_seed(seed))).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()


def test_configure_optimizer_returns_the_flat_classes_behind_the_lifecycle_wrapper():
    _, adamw = _sharded("adamw", lr=1e-2)
    _, sgd = _sharded("sgd", lr=1e-2)
    assert isinstance(adamw.optimizer, FlatShardedAdamW) and isinstance(sgd.optimizer, FlatShardedSGD)
    assert isinstance(adamw.optimizer, torch.optim.Optimizer)            # schedulers and hooks of torch.optim apply


def test_adamw_moments_of_all_parameters_are_views_of_two_flat_buffers():
    model, opt = _sharded("adamw", lr=1e-2)
    unit = model._matrix_fsdp_param_group
    flat = opt.optimizer.flat_state(unit)
    assert set(flat) == {"exp_avg", "exp_avg_sq"} and all(t.numel() == unit.flat_buffer.local_numel for t in flat.values())
    for name in flat:
        lo = flat[name].data_ptr()
        hi = lo + flat[name].numel() * 4
        for p in model.parameters():
            view = opt.state[p][name]
            assert lo <= view.data_ptr() < hi and tuple(view.shape) == tuple(p.shape)


def test_the_step_count_is_published_to_every_parameter_by_both_flat_optimizers():
    for kind, kw in (("adamw", dict(lr=1e-2)), ("sgd", dict(lr=1e-2, momentum=0.9))):
        model, opt = _sharded(kind, **kw)
        for i in range(3):
            _step(model, opt, seed=i)
        assert opt.optimizer.unit_step_count(model._matrix_fsdp_param_group) == 3
        assert all(float(opt.state[p]["step"]) == 3.0 for p in model.parameters()), kind


def test_loading_a_state_dict_copies_into_the_flat_buffers_and_keeps_the_views():
    model, opt = _sharded("adamw", lr=1e-2)
    _step(model, opt)
    saved = copy.deepcopy(opt.state_dict())
    flat_before = opt.optimizer.flat_state(model._matrix_fsdp_param_group)["exp_avg"]
    ptr = flat_before.data_ptr()
    expect = flat_before.clone()
    _step(model, opt, seed=2)
    opt.load_state_dict(saved)
    flat = opt.optimizer.flat_state(model._matrix_fsdp_param_group)["exp_avg"]
    assert flat.data_ptr() == ptr and torch.equal(flat, expect)
    for p in model.parameters():
        assert opt.state[p]["exp_avg"].untyped_storage().data_ptr() == flat.untyped_storage().data_ptr()
    assert opt.optimizer.unit_step_count(model._matrix_fsdp_param_group) == 1


def test_sgd_momentum_survives_a_state_dict_round_trip():
    model, opt = _sharded("sgd", lr=0.05, momentum=0.9)
    twin, topt = _sharded("sgd", lr=0.05, momentum=0.9)
    for i in range(2):
        _step(model, opt, seed=i)
        _step(twin, topt, seed=i)
    fresh, fopt = _sharded("sgd", lr=0.05, momentum=0.9)
    with torch.no_grad():
        fresh._matrix_fsdp_param_group.flat_buffer.local_shard.copy_(model._matrix_fsdp_param_group.flat_buffer.local_shard)
    fopt.load_state_dict(copy.deepcopy(opt.state_dict()))
    _step(twin, topt, seed=5)
    _step(fresh, fopt, seed=5)
    assert torch.equal(fresh._matrix_fsdp_param_group.flat_buffer.local_shard,
                       twin._matrix_fsdp_param_group.flat_buffer.local_shard)


def test_hyperparameters_are_read_from_the_param_groups_at_every_step():
    model, opt = _sharded("sgd", lr=0.1)
    ref = _model()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    sched = torch.optim.lr_scheduler.StepLR(opt.optimizer, step_size=1, gamma=0.1)
    rsched = torch.optim.lr_scheduler.StepLR(ropt, step_size=1, gamma=0.1)
    for i in range(3):
        _step(model, opt, seed=i)
        _step(ref, ropt, seed=i)
        sched.step()
        rsched.step()
    assert opt.param_groups[0]["lr"] == pytest.approx(1e-4)
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-7)


def test_unsupported_torch_options_are_refused_not_dropped():
    reset_shared_owner_planners()
    model = _model()
    fully_shard(model)
    with pytest.raises(NotImplementedError, match="amsgrad"):
        configure_optimizer(model, "adamw", lr=1e-2, amsgrad=True)
    with pytest.raises(NotImplementedError, match="nesterov"):
        configure_optimizer(model, "sgd", lr=1e-2, momentum=0.9, nesterov=True)
    with pytest.raises(TypeError, match="unexpected"):
        configure_optimizer(model, "adamw", lr=1e-2, warp_speed=9)
    with pytest.raises(ValueError):
        configure_optimizer(model, "adamw", lr=-1.0)


def test_a_gradient_scale_is_applied_on_the_fly():
    model, opt = _sharded("sgd", lr=0.1)
    ref = _model()
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    opt.optimizer.grad_scale = 0.5
    model(torch.ones(2, 4)).sum().backward()
    ref(torch.ones(2, 4)).sum().backward()
    for q in ref.parameters():
        q.grad.mul_(0.5)
    opt.step()
    ropt.step()
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-7)


def test_state_manager_lists_every_managed_parameter_with_its_place_in_the_shard():
    model, opt = _sharded("adamw", lr=1e-2)
    infos = [info for _, info in opt.state_manager.iter_param_infos()]
    assert [i.fqn for i in infos] == [n for n, _ in model.named_parameters()]
    assert all(i.component == "optimizer" and i.local_numel == i.param_numel and i.param_start == 0 for i in infos)
    starts = [i.local_start for i in infos]
    assert starts == sorted(starts) and starts[0] == 0


def test_state_tensors_shaped_like_their_parameter_carry_shard_metadata():
    model, opt = _sharded("adamw", lr=1e-2)
    _step(model, opt)
    tensors = list(opt.state_manager.iter_state_tensors())
    shaped = [t for t in tensors if t.sharded is not None]
    scalars = [t for t in tensors if t.sharded is None]
    assert {t.state_name for t in shaped} == {"exp_avg", "exp_avg_sq"} and {t.state_name for t in scalars} == {"step"}
    w = next(t for t in shaped if t.info.fqn == "0.weight" and t.state_name == "exp_avg")
    assert tuple(w.sharded.logical_shape) == (6, 4) and w.sharded.world_size == 1 and w.sharded.name == "0.weight.exp_avg"


def test_summary_counts_tensors_and_bytes_per_component():
    model, opt = _sharded("adamw", lr=1e-2)
    _step(model, opt)
    s = opt.local_state_summary()
    n = sum(p.numel() for p in model.parameters())
    assert s.num_params == 3 and s.num_state_tensors == 9                 # 3 x (exp_avg, exp_avg_sq, step)
    assert s.local_state_numel == 2 * n + 3 and s.by_component == {"optimizer": 2 * n + 3}
    assert s.local_state_bytes == 4 * (2 * n + 3)


def test_mixed_optimizer_keeps_muon_state_on_matrices_and_adamw_state_on_the_rest():
    model, opt = _sharded("mixed_muon_adamw", policy="mixed_muon_adamw", lr=1e-2)
    _step(model, opt)
    by_comp = {}
    for t in opt.state_manager.iter_state_tensors():
        by_comp.setdefault(t.info.component, set()).add((t.info.fqn, t.state_name))
    assert {f for f, _ in by_comp["muon"]} == {"0.weight", "1.weight"}
    assert {n for _, n in by_comp["muon"]} == {"momentum_buffer"}
    assert {f for f, _ in by_comp["adamw"]} == {"0.bias"}
    assert set(opt.local_state_summary().by_component) == {"muon", "adamw"}
    groups = opt.optimizer_group_summary()
    assert {g.optimizer_type for g in groups} == {"muon", "adamw"}


def test_units_whose_parameters_sit_in_different_param_groups_fall_back_to_per_parameter_updates():
    reset_shared_owner_planners()
    model, ref = _model(), _model()
    fully_shard(model)
    decay, no_decay = [model[0].weight, model[1].weight], [model[0].bias]
    inner = FlatShardedAdamW([dict(params=decay, weight_decay=0.1), dict(params=no_decay, weight_decay=0.0)],
                             units=model, lr=1e-2)
    assert inner.flat_state(model._matrix_fsdp_param_group) is None       # no single hyper-parameter set for the unit
    from matrix_fsdp_b200.optim.wrapper import MatrixFSDPOptimizer

    opt = MatrixFSDPOptimizer(inner, model)
    ropt = torch.optim.AdamW([dict(params=[ref[0].weight, ref[1].weight], weight_decay=0.1),
                              dict(params=[ref[0].bias], weight_decay=0.0)], lr=1e-2)
    for i in range(3):
        _step(model, opt, seed=i)
        _step(ref, ropt, seed=i)
    for p, q in zip(model.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-6)
