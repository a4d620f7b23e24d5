"""Scheduler behaviour, one rule per test (single rank, CPU): prefetch budgets, caps, timing of the backward
prefetch, configuration objects, order tracking.  The reference keeps the same rules in
test/fsdp/test_matrix_fsdp_e2e.py (scheduler section)."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.scheduler import MatrixFSDPSchedulerConfig


def _stack(n=4):
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(*[nn.Linear(8, 8) for _ in range(n)])
    for blk in model:
        fully_shard(blk)
    return model


def _step(model, opt):
    model(torch.randn(2, 8)).sum().backward()
    opt.step()
    opt.zero_grad()


def _sched(model):
    return model[0]._matrix_fsdp_param_group.scheduler


def _names(unit):
    return [e.name for e in unit.runtime_events]


def test_one_scheduler_is_shared_by_all_units_of_the_optimizer():
    model = _stack()
    configure_optimizer(model, "sgd", lr=0.1)
    scheds = {id(b._matrix_fsdp_param_group.scheduler) for b in model}
    assert len(scheds) == 1 and _sched(model) is not None
    assert len(_sched(model).units) == 4


def test_default_budget_prefetches_one_unit_ahead_in_both_directions():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1)
    _step(model, opt)
    c = _sched(model).counters
    assert c.forward_prefetch_issued == 3 and c.backward_prefetch_issued == 3       # every unit but the first / last
    assert c.prefetch_blocked_by_caps == 0 and c.high_water_active_full_param_buffers <= 2


def test_backward_prefetch_can_be_switched_off_alone():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_backward_prefetch_units=0)
    _step(model, opt)
    c = _sched(model).counters
    assert c.forward_prefetch_issued == 3 and c.backward_prefetch_issued == 0


def test_forward_budget_does_not_limit_the_backward_prefetch():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_forward_prefetch_units=0)
    _step(model, opt)
    c = _sched(model).counters
    assert c.forward_prefetch_issued == 0 and c.backward_prefetch_issued == 3


def test_zero_unsharded_budget_means_no_prefetch_at_all():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_unsharded_prefetch_units=0)
    _step(model, opt)
    c = _sched(model).counters
    assert c.forward_prefetch_issued == 0 and c.backward_prefetch_issued == 0
    assert not any(e.prefetched for b in model for e in b._matrix_fsdp_param_group.runtime_events if e.name == "unshard")


def test_active_buffer_cap_blocks_prefetch_and_is_counted():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_active_full_param_buffers=1)
    _step(model, opt)
    c = _sched(model).counters
    assert c.forward_prefetch_issued == 0 and c.prefetch_blocked_by_caps > 0
    assert c.high_water_active_full_param_buffers == 1


def test_backward_prefetch_timing_before_or_after_the_current_units_reshard():
    for timing, tag in (("pre_backward", "backward_prefetch"), ("post_reshard", "post_reshard_prefetch")):
        model = _stack()
        opt = configure_optimizer(model, "sgd", lr=0.1, backward_prefetch_timing=timing)
        _step(model, opt)
        ev = _names(model[2]._matrix_fsdp_param_group)
        assert f"start_unshard:{tag}" in ev, (timing, ev)
        # either way the gather was issued before the unit's own backward needed it
        assert ev.index(f"start_unshard:{tag}") < ev.index("pre_backward_unshard")


def test_scheduler_config_object_is_accepted_and_exclusive_with_keywords():
    model = _stack()
    configure_optimizer(model, "sgd", lr=0.1, scheduler_config=MatrixFSDPSchedulerConfig(max_unsharded_prefetch_units=2))
    assert _sched(model).config.max_unsharded_prefetch_units == 2
    with pytest.raises(ValueError, match="either scheduler_config or explicit"):
        configure_optimizer(_stack(), "sgd", lr=0.1, scheduler_config=MatrixFSDPSchedulerConfig(),
                            max_unsharded_prefetch_units=1)


def test_forward_order_is_recorded_as_run_not_as_registered():
    model = _stack(3)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    x = torch.randn(2, 8)
    model[0](model[1](model[2](x))).sum().backward()          # 2 -> 1 -> 0
    opt.step()
    assert [u.module for u in _sched(model).forward_order] == [model[2], model[1], model[0]]
    opt.zero_grad()
    _step(model, opt)                                          # the usual order replaces it in the next iteration
    assert [u.module for u in _sched(model).forward_order] == list(model)


def test_iterations_and_waits_are_counted():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1)
    for _ in range(3):
        _step(model, opt)
    c = _sched(model).counters
    assert c.iterations == 3 and c.unshard_waits >= 3 * 4 and c.reduce_waits >= 3


def test_two_pending_reduces_are_allowed_when_configured():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_pending_backward_reduces=2)
    _step(model, opt)
    assert _sched(model).config.max_pending_backward_reduces == 2
    assert all(b._matrix_fsdp_param_group.flat_buffer.pending_reduce is None for b in model)


def test_next_step_prefetch_is_off_on_cpu_and_can_be_requested():
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1)
    _step(model, opt)
    assert _sched(model).counters.next_step_prefetch_issued == 0
    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, prefetch_first_unit_after_step=True)
    _step(model, opt)
    assert _sched(model).counters.next_step_prefetch_issued == 1
    first = model[0]._matrix_fsdp_param_group
    assert first.flat_buffer.pending_gather is not None or first.state.value == "unsharded"
    _step(model, opt)                                          # the prefetched unit is consumed normally
    assert _sched(model).counters.next_step_prefetch_issued == 2


def test_summary_reports_policy_depths_and_counters():
    from matrix_fsdp_b200 import summarize_scheduler

    model = _stack()
    opt = configure_optimizer(model, "sgd", lr=0.1, max_unsharded_prefetch_units=2)
    _step(model, opt)
    s = summarize_scheduler(model)
    assert s["prefetch_policy"] == "static" and s["forward_prefetch_depth"] == 2 and s["backward_prefetch_depth"] == 2
    assert s["counters"]["forward_prefetch_issued"] >= 3 and s["num_units"] == 4
