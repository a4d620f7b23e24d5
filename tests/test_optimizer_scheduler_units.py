"""Optimizer wrappers and the scheduler at world size 1 (no process group): option routing, lifecycle guards,
summaries, prefetch counters and caps, SGD / Muon parity with the eager optimizers."""
import copy

import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard, matrix_fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.scheduler import MatrixFSDPScheduler, MatrixFSDPSchedulerConfig
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


def _stack(n=3, seed=0, width=8):
    torch.manual_seed(seed)
    return nn.Sequential(*[nn.Sequential(nn.Linear(width, width), nn.Tanh()) for _ in range(n)])


def _shard_blocks(model, **kw):
    reset_shared_owner_planners()
    for block in model:
        fully_shard(block, **kw)
    return model


def _batch(seed=1, width=8):
    return torch.randn(4, width, generator=torch.Generator().manual_seed(seed))


# ------------------------------------------------------------------------------------ config
def test_scheduler_config_validation():
    MatrixFSDPSchedulerConfig(backward_prefetch_timing="post_reshard", prefetch_policy="adaptive")
    with pytest.raises(ValueError):
        MatrixFSDPSchedulerConfig(max_unsharded_prefetch_units=-1)
    with pytest.raises(ValueError):
        MatrixFSDPSchedulerConfig(backward_prefetch_timing="sometimes")
    with pytest.raises(ValueError):
        MatrixFSDPSchedulerConfig(prefetch_policy="psychic")
    with pytest.raises(ValueError):
        MatrixFSDPSchedulerConfig(max_pending_backward_reduces=-2)
    model = _shard_blocks(_stack())
    with pytest.raises(TypeError, match="Unknown scheduler option"):
        MatrixFSDPScheduler(collect_param_groups(model), bogus=1)


def test_scheduler_kwargs_are_split_from_optimizer_kwargs():
    model = _shard_blocks(_stack())
    opt = configure_optimizer(model, "adamw", lr=1e-2, weight_decay=0.0, max_unsharded_prefetch_units=2,
                              max_pending_backward_reduces=2, backward_prefetch_timing="post_reshard")
    cfg = opt.scheduler.config
    assert cfg.max_unsharded_prefetch_units == 2 and cfg.max_pending_backward_reduces == 2
    assert cfg.backward_prefetch_timing == "post_reshard"
    assert opt.param_groups[0]["lr"] == 1e-2 and "max_unsharded_prefetch_units" not in opt.param_groups[0]
    with pytest.raises(TypeError):
        configure_optimizer(_shard_blocks(_stack()), "adamw", lr=1e-2, not_an_option=3)
    with pytest.raises(ValueError, match="optimizer must be one of"):
        configure_optimizer(_shard_blocks(_stack()), "lion")


# ------------------------------------------------------------------------------------ prefetch behaviour
def test_prefetch_counters_and_recorded_order():
    model = _shard_blocks(_stack(4))
    opt = configure_optimizer(model, "sgd", lr=0.1)
    sched = opt.scheduler
    model(_batch()).sum().backward()
    opt.step()
    opt.zero_grad()
    c = sched.counters.as_dict()
    assert c["forward_prefetch_issued"] == 3 and c["backward_prefetch_issued"] == 3     # every unit but the first
    assert c["high_water_active_full_param_buffers"] <= 2                               # window of one unit ahead
    assert c["iterations"] == 1
    units = collect_param_groups(model)
    assert [u.name for u in sched.forward_order] == [u.name for u in units]
    assert all(u.state.value == "sharded" for u in units)


def test_prefetch_can_be_switched_off_and_capped():
    model = _shard_blocks(_stack(4))
    opt = configure_optimizer(model, "sgd", lr=0.1, max_unsharded_prefetch_units=0)
    model(_batch()).sum().backward()
    opt.step()
    c = opt.scheduler.counters.as_dict()
    assert c["forward_prefetch_issued"] == 0 and c["backward_prefetch_issued"] == 0
    assert c["high_water_active_full_param_buffers"] == 1
    capped = _shard_blocks(_stack(4))
    opt2 = configure_optimizer(capped, "sgd", lr=0.1, max_unsharded_prefetch_units=3, max_active_full_param_buffers=2)
    capped(_batch()).sum().backward()
    opt2.step()
    c2 = opt2.scheduler.counters.as_dict()
    assert c2["high_water_active_full_param_buffers"] <= 2 and c2["prefetch_blocked_by_caps"] > 0


# ------------------------------------------------------------------------------------ lifecycle guards
def test_no_sync_guards_and_closures():
    model = _shard_blocks(_stack(2))
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    with opt.no_sync():
        model(_batch()).sum().backward()
        with pytest.raises(RuntimeError, match="no_sync"):
            opt.step()
        with pytest.raises(RuntimeError, match="no_sync"):
            opt.zero_grad()
    model(_batch(2)).sum().backward()
    opt.step()
    opt.zero_grad()
    with pytest.raises(NotImplementedError, match="closure"):
        opt.step(lambda: None)


def test_sgd_and_muon_match_eager_optimizers():
    for kind, make_ref, kw in (
            ("sgd", lambda ps: torch.optim.SGD(ps, lr=0.1, momentum=0.9, weight_decay=0.01),
             dict(lr=0.1, momentum=0.9, weight_decay=0.01)),
            ("adamw", lambda ps: torch.optim.AdamW(ps, lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1),
             dict(lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1))):
        model = _stack(2, seed=3)
        ref = copy.deepcopy(model)
        _shard_blocks(model)
        opt, ropt = configure_optimizer(model, kind, **kw), make_ref(ref.parameters())
        for s in range(3):
            x = _batch(s)
            model(x).pow(2).mean().backward()
            ref(x).pow(2).mean().backward()
            opt.step(), ropt.step()
            opt.zero_grad(), ropt.zero_grad()
        for u, block in zip(collect_param_groups(model), ref):
            full = torch.cat([p.detach().reshape(-1) for p in block.parameters()])
            assert torch.allclose(u.flat_buffer.local_shard, full, atol=1e-6), kind


def test_mixed_optimizer_surface_and_classification():
    from matrix_fsdp_b200.optim.wrapper import classify_matrix_optimizer_params

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(8, 8), nn.LayerNorm(8), nn.Linear(8, 4, bias=False))
    fully_shard(model, optimizer_policy="mixed_muon_adamw")
    cls = classify_matrix_optimizer_params(model)
    muon_fqns = {getattr(p, "_matrix_fsdp_fqn") for p in cls.muon_params}
    adamw_fqns = {getattr(p, "_matrix_fsdp_fqn") for p in cls.adamw_params}
    assert muon_fqns == {"0.weight", "2.weight"} and adamw_fqns == {"0.bias", "1.weight", "1.bias"}
    opt = configure_optimizer(model, "mixed_muon_adamw", lr=1e-2, muon_lr=0.02)
    names = [n for n, _ in opt.iter_named_optimizers()]
    assert names == ["muon", "adamw"]
    # defaults of the mixed optimizer follow the reference: momentum 0.5, 2 Newton-Schulz steps, match_rms_adamw
    g = opt.muon.param_groups[0]
    assert g["momentum"] == 0.5 and g["ns_steps"] == 2 and g["adjust_lr_fn"] == "match_rms_adamw"
    model(_batch()).sum().backward()
    opt.step()
    opt.zero_grad()
    summary = opt.optimizer_group_summary()
    assert {s.optimizer_type for s in summary} == {"muon", "adamw"}
    assert sum(s.param_numel for s in summary) == sum(p.numel() for p in model.parameters())
    st = opt.local_state_summary()
    assert st.num_state_tensors > 0 if hasattr(st, "num_state_tensors") else st is not None
    with pytest.raises(TypeError, match="Unknown mixed optimizer options"):
        configure_optimizer(model, "mixed_muon_adamw", lr=1e-2, muon_nonsense=1)
    with pytest.raises(ValueError, match="component"):
        opt.load_state_dict({"muon": opt.muon.state_dict()})


def test_muon_rejects_non_matrix_parameters():
    reset_shared_owner_planners()
    model = nn.Sequential(nn.Linear(4, 4))          # has a bias
    fully_shard(model)
    with pytest.raises(ValueError, match="2D"):
        configure_optimizer(model, "muon", lr=0.02)
    reset_shared_owner_planners()
    ok = nn.Sequential(nn.Linear(4, 4, bias=False))
    fully_shard(ok, optimizer_policy="muon")
    opt = configure_optimizer(ok, "muon", lr=0.02)
    ok(_batch(width=4)).sum().backward()
    opt.step()


def test_matrix_fully_shard_installs_a_scheduler_and_wrap_policy():
    from matrix_fsdp_b200.policy.wrap import module_type_policy

    reset_shared_owner_planners()
    model = _stack(3)
    matrix_fully_shard(model, wrap_policy=module_type_policy(nn.Sequential))
    units = collect_param_groups(model)
    assert len(units) >= 3 and all(u.scheduler is units[0].scheduler and u.scheduler is not None for u in units)
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    assert opt.scheduler is units[0].scheduler
    model(_batch()).sum().backward()
    opt.step()
