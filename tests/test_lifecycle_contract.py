"""Small single-rank checks of the unit lifecycle contract, one behaviour per test (the reference keeps the same
contract in test/fsdp/test_matrix_fsdp_e2e.py).  Everything runs on CPU with the local transport."""
import copy

import pytest
import torch
from torch import nn
from torch.distributed.fsdp import MixedPrecisionPolicy
from torch.utils.checkpoint import checkpoint

from matrix_fsdp_b200 import (FSDPLifecycleState, configure_optimizer, fully_shard, matrix_fully_shard, module_type_policy,
                              summarize_param_groups)
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


class Blk(nn.Module):
    def __init__(self, d=8):
        super().__init__()
        self.a = nn.Linear(d, 2 * d)
        self.b = nn.Linear(2 * d, d)

    def forward(self, x):
        return x + self.b(torch.relu(self.a(x)))


def _stack(n=3, d=8, seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(*[Blk(d) for _ in range(n)])


def _pair(n=3, **shard_kw):
    """A sharded stack (one unit per block) and its eager twin."""
    reset_shared_owner_planners()
    model = _stack(n)
    ref = copy.deepcopy(model)
    for b in model:
        fully_shard(b, **shard_kw)
    return model, ref


def _same_params(model, ref, tol=1e-6):
    got = {n: p for n, p in model.named_parameters()}
    for n, p in ref.named_parameters():
        full = got[n].full_tensor() if hasattr(got[n], "full_tensor") else got[n]
        assert torch.allclose(full.detach().float().reshape(p.shape), p.detach().float(), atol=tol), n


def _train(model, opt, ref, ropt, steps=2, fn=None, seed=3):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        x = torch.randn(4, 8, generator=g)
        for m, o in ((model, opt), (ref, ropt)):
            out = fn(m, x) if fn is not None else m(x)
            out.pow(2).mean().backward()
            o.step()
            o.zero_grad()


# ------------------------------------------------------------------------------------------ numerics vs eager
@pytest.mark.parametrize("reshard", [True, False])
def test_multi_unit_step_matches_eager(reshard):
    model, ref = _pair(reshard_after_forward=reshard)
    _train(model, configure_optimizer(model, "adamw", lr=1e-2), ref, torch.optim.AdamW(ref.parameters(), lr=1e-2))
    _same_params(model, ref)


def test_root_unit_step_matches_eager():
    reset_shared_owner_planners()
    model = _stack(2)
    ref = copy.deepcopy(model)
    fully_shard(model)
    _train(model, configure_optimizer(model, "sgd", lr=0.05), ref, torch.optim.SGD(ref.parameters(), lr=0.05))
    _same_params(model, ref)


def test_multiple_forwards_single_backward_matches_eager():
    model, ref = _pair(reshard_after_forward=False)

    def twice(m, x):
        return m(x) + m(x * 0.5)

    _train(model, configure_optimizer(model, "sgd", lr=0.05), ref, torch.optim.SGD(ref.parameters(), lr=0.05), fn=twice)
    _same_params(model, ref)


def test_parallel_branches_match_eager():
    model, ref = _pair()

    def branches(m, x):
        return m[0](x) + m[1](x) + m[2](x)

    _train(model, configure_optimizer(model, "adamw", lr=1e-2), ref, torch.optim.AdamW(ref.parameters(), lr=1e-2), fn=branches)
    _same_params(model, ref)


@pytest.mark.parametrize("reentrant", [False, True])
def test_activation_checkpoint_around_units_matches_eager(reentrant):
    model, ref = _pair()

    def ckpt(m, x):
        x = x.clone().requires_grad_(True)       # the re-entrant form needs an input that carries a gradient
        for blk in m:
            x = checkpoint(blk, x, use_reentrant=reentrant)
        return x

    _train(model, configure_optimizer(model, "adamw", lr=1e-2), ref, torch.optim.AdamW(ref.parameters(), lr=1e-2), fn=ckpt)
    _same_params(model, ref)


def test_activation_checkpoint_of_the_root_unit_matches_eager():
    reset_shared_owner_planners()
    model = _stack(2)
    ref = copy.deepcopy(model)
    fully_shard(model)
    fn = lambda m, x: checkpoint(m, x, use_reentrant=False)      # noqa: E731
    _train(model, configure_optimizer(model, "sgd", lr=0.05), ref, torch.optim.SGD(ref.parameters(), lr=0.05), fn=fn)
    _same_params(model, ref)


def test_plain_torch_optimizer_is_prepared_automatically_and_matches_eager():
    model, ref = _pair()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-2)          # no configure_optimizer: step hooks do the lifecycle
    _train(model, opt, ref, torch.optim.AdamW(ref.parameters(), lr=1e-2), steps=3)
    _same_params(model, ref)


def test_no_sync_accumulation_equals_one_big_batch_gradient():
    model, ref = _pair()
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(4, 8, generator=g) for _ in range(3)]
    with opt.no_sync():
        for x in xs[:-1]:
            model(x).pow(2).mean().backward()
    model(xs[-1]).pow(2).mean().backward()
    for x in xs:
        ref(x).pow(2).mean().backward()
    opt.step(), ropt.step()
    _same_params(model, ref)


@pytest.mark.parametrize("set_to_none", [True, False])
def test_zero_grad_modes_leave_the_next_step_clean(set_to_none):
    model, ref = _pair(2)
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(6)
    for _ in range(2):
        x = torch.randn(4, 8, generator=g)
        model(x).sum().backward(), ref(x).sum().backward()
        opt.step(), ropt.step()
        opt.zero_grad(set_to_none=set_to_none), ropt.zero_grad(set_to_none=set_to_none)
    _same_params(model, ref)


def test_unused_unit_is_left_alone_by_the_step():
    model, ref = _pair()
    opt, ropt = configure_optimizer(model, "adamw", lr=1e-2), torch.optim.AdamW(ref.parameters(), lr=1e-2)
    before = model[2]._matrix_fsdp_param_group.flat_buffer.local_shard.clone()
    x = torch.randn(4, 8)
    model[1](model[0](x)).sum().backward(), ref[1](ref[0](x)).sum().backward()
    opt.step(), ropt.step()
    assert torch.equal(model[2]._matrix_fsdp_param_group.flat_buffer.local_shard, before)
    _same_params(model, ref)


# ------------------------------------------------------------------------------------------ states and views
def test_state_sequence_of_one_training_step():
    model, _ = _pair(2)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    u = model[0]._matrix_fsdp_param_group
    assert u.state == FSDPLifecycleState.SHARDED
    out = model(torch.randn(2, 8))
    assert u.state == FSDPLifecycleState.FORWARD_RESHARDED
    out.sum().backward()
    assert u.state == FSDPLifecycleState.SHARDED and u.finalized_after_backward
    opt.step()
    u.assert_optimizer_ready()
    assert u.state == FSDPLifecycleState.SHARDED


def test_without_reshard_after_forward_the_unit_stays_unsharded_until_backward():
    model, _ = _pair(2, reshard_after_forward=False)
    configure_optimizer(model, "sgd", lr=0.1)
    u = model[0]._matrix_fsdp_param_group
    out = model(torch.randn(2, 8))
    assert u.state == FSDPLifecycleState.UNSHARDED       # (one rank: the full buffer aliases the shard)
    out.sum().backward()
    assert u.state == FSDPLifecycleState.SHARDED


def test_forward_under_no_grad_returns_to_sharded():
    model, _ = _pair(2)
    u = model[1]._matrix_fsdp_param_group
    with torch.no_grad():
        model(torch.randn(2, 8))
    assert u.state == FSDPLifecycleState.SHARDED and u.forward_count_since_backward == 0


def test_unsharded_parameters_are_views_of_the_full_buffer():
    model, _ = _pair(1, reshard_after_forward=False)
    u = model[0]._matrix_fsdp_param_group
    model(torch.randn(2, 8))
    full = u.flat_buffer.full_buffer
    lo, hi = full.data_ptr(), full.data_ptr() + full.numel() * full.element_size()
    for p in model[0].parameters():
        assert lo <= p.data_ptr() < hi
    u.reshard()
    assert u.state != FSDPLifecycleState.UNSHARDED


def test_manual_unshard_and_reshard_round_trip():
    model, ref = _pair(1)
    u = model[0]._matrix_fsdp_param_group
    u.unshard()
    assert u.state == FSDPLifecycleState.UNSHARDED
    for (n, p), (_, q) in zip(model[0].named_parameters(), ref[0].named_parameters()):
        assert torch.equal(p.detach().reshape(q.shape), q.detach()), n
    u.reshard()
    assert u.state == FSDPLifecycleState.SHARDED and u.full_param_storage_nbytes() == 0


def test_unit_names_are_unique_and_collected_in_module_order():
    model, _ = _pair(3)
    units = collect_param_groups(model)
    assert [u.module for u in units] == list(model)
    assert len({u.name for u in units}) == 3 and len({id(u.flat_buffer) for u in units}) == 3
    assert len({u.metadata.runtime_param_group_id for u in units}) == 3 and len({u.metadata.comm_buffer_id for u in units}) == 3


def test_unit_layout_queries_cover_every_parameter_once():
    model, _ = _pair(1)
    u = model[0]._matrix_fsdp_param_group
    fqns = [mp.fqn for mp in u.registry]
    assert sorted(fqns) == ["a.bias", "a.weight", "b.bias", "b.weight"]
    assert sorted(u.params_for_rank(0)) == sorted(fqns) and u.world_size == 1
    for fqn in fqns:
        segs = u.rank_segments_for_param(fqn)
        assert sum(s.numel for s in segs) == dict(model[0].named_parameters())[fqn].numel()
    assert u.owner_ranks("a.weight") == (0,)


def test_scheduler_records_forward_order_and_reverses_it_for_backward():
    model, _ = _pair(3)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    model(torch.randn(2, 8)).sum().backward()
    opt.step()
    sched = model[0]._matrix_fsdp_param_group.scheduler
    assert [u.module for u in sched.forward_order] == list(model)
    assert sched.counters.forward_prefetch_issued >= 2 and sched.counters.backward_prefetch_issued >= 2


def test_summary_rows_describe_every_unit():
    model, _ = _pair(2)
    configure_optimizer(model, "adamw", lr=1e-2)
    rows = summarize_param_groups(model)
    assert len(rows) == 2
    for r in rows:
        assert r["num_params"] == 4 and r["world_size"] == 1 and r["total_numel"] == sum(p.numel() for p in model[0].parameters())


# ------------------------------------------------------------------------------------------ options and rejections
def test_mixed_precision_forward_dtype_and_master_dtype():
    model, _ = _pair(1, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16))
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    u = model[0]._matrix_fsdp_param_group
    seen = []
    model[0].a.register_forward_hook(lambda m, i, o: seen.append(m.weight.dtype))
    model(torch.randn(2, 8).bfloat16()).float().sum().backward()
    opt.step()
    assert seen == [torch.bfloat16] and u.flat_buffer.local_shard.dtype == torch.float32
    assert all(st["exp_avg"].dtype == torch.float32 for st in opt.state.values() if "exp_avg" in st)


def test_frozen_parameters_are_rejected_unless_ignored():
    m = nn.Linear(4, 4)
    m.bias.requires_grad_(False)
    with pytest.raises(ValueError, match="ignored_params"):
        fully_shard(m)
    fully_shard(m, ignored_params={m.bias})
    assert [mp.fqn for mp in m._matrix_fsdp_param_group.registry] == ["weight"]


def test_module_without_parameters_is_rejected():
    with pytest.raises(ValueError, match="at least one parameter"):
        fully_shard(nn.ReLU())


def test_shared_parameter_between_units_is_rejected():
    a, b = nn.Linear(4, 4), nn.Linear(4, 4)
    b.weight = a.weight
    holder = nn.Sequential(a, b)
    fully_shard(a)
    with pytest.raises(ValueError, match="shared"):
        fully_shard(b)
    del holder


def test_integer_reshard_after_forward_is_not_supported():
    with pytest.raises(NotImplementedError):
        fully_shard(nn.Linear(4, 4), reshard_after_forward=2)


def test_unknown_optimizer_policy_and_conflicting_placement_are_rejected():
    from torch.distributed.tensor.placement_types import Shard

    with pytest.raises(ValueError):
        fully_shard(nn.Linear(4, 4), optimizer_policy="adagrad_owner")
    with pytest.raises(ValueError):
        fully_shard(nn.Linear(4, 4), optimizer_policy="mixed_muon_adamw", shard_placement_fn=lambda p: Shard(0))


def test_wrap_policy_makes_one_unit_per_matching_module():
    reset_shared_owner_planners()
    model = _stack(3)
    matrix_fully_shard(model, wrap_policy=module_type_policy(Blk))
    units = collect_param_groups(model)
    assert [u.module for u in units] == list(model)
    with pytest.raises(ValueError):
        matrix_fully_shard(_stack(1), wrap_policy=module_type_policy(nn.Conv2d))


def test_optimizer_step_inside_no_sync_is_rejected():
    model, _ = _pair(1)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    with opt.no_sync():
        model(torch.randn(2, 8)).sum().backward()
        with pytest.raises(RuntimeError):
            opt.step()
    model(torch.randn(2, 8)).sum().backward()
    opt.step()


def test_scheduler_option_validation():
    model, _ = _pair(1)
    with pytest.raises(ValueError):
        configure_optimizer(model, "sgd", lr=0.1, max_unsharded_prefetch_units=-1)
    model, _ = _pair(1)
    with pytest.raises(ValueError):
        configure_optimizer(model, "sgd", lr=0.1, prefetch_policy="psychic")


def test_second_forward_after_the_step_starts_a_fresh_cycle():
    model, ref = _pair(2)
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    _train(model, opt, ref, ropt, steps=1)
    u = model[0]._matrix_fsdp_param_group
    u.clear_runtime_events()
    _train(model, opt, ref, ropt, steps=1, seed=9)
    names = [e.name for e in u.runtime_events]
    assert names.count("pre_forward") == 1 and names.count("finalize_backward") == 1
    _same_params(model, ref)


@pytest.mark.parametrize("reshard", [True, False])
def test_two_losses_over_one_forward_add_their_gradients(reshard):
    """``loss_a.backward(retain_graph=True); loss_b.backward()``: the kept graph is walked twice, every unit gathers
    its parameters again for the second pass and the two reductions add up."""
    model, ref = _pair(reshard_after_forward=reshard)
    opt, ropt = configure_optimizer(model, "sgd", lr=0.05), torch.optim.SGD(ref.parameters(), lr=0.05)
    for seed in range(2):
        x = torch.randn(4, 8, generator=torch.Generator().manual_seed(seed))
        for m in (model, ref):
            y = m(x)
            y.pow(2).mean().backward(retain_graph=True)
            y.abs().mean().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    _same_params(model, ref)
    unit = model[0]._matrix_fsdp_param_group
    names = [e.name for e in unit.runtime_events]
    assert names.count("pre_backward_unshard") == 4 and names.count("start_reduce_scatter") == 4   # 2 steps x 2 passes


class _PassThrough(nn.Module):
    """Two outputs; the second one reaches no parameter of the unit."""

    def __init__(self):
        super().__init__()
        self.lin = nn.Linear(8, 8)

    def forward(self, x):
        return self.lin(x), x * 2.0


@pytest.mark.parametrize("wrapped_torch", [False, True])
def test_an_output_that_reaches_no_parameter_does_not_disturb_the_step(wrapped_torch):
    from matrix_fsdp_b200.optim.wrapper import MatrixFSDPOptimizer

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model, ref = _PassThrough(), None
    ref = copy.deepcopy(model)
    fully_shard(model)
    opt = MatrixFSDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), model) if wrapped_torch \
        else configure_optimizer(model, "sgd", lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    for seed in range(2):
        x = torch.randn(4, 8, generator=torch.Generator().manual_seed(seed)).requires_grad_(True)
        for m in (model, ref):
            a, b = m(x)
            # the pass-through output gets its gradient last: after the unit has seen all of its parameters' gradients
            (a.pow(2).mean() + (b.detach() * 0).sum()).backward(retain_graph=True)
            b.sum().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    _same_params(model, ref)


@pytest.mark.parametrize("wrapped_torch", [False, True])
def test_a_forward_without_backward_after_a_backward_keeps_the_reduced_gradients(wrapped_torch):
    from matrix_fsdp_b200.optim.wrapper import MatrixFSDPOptimizer

    model, ref = _pair()
    opt = MatrixFSDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1), model) if wrapped_torch \
        else configure_optimizer(model, "sgd", lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    x = torch.randn(4, 8)
    model(x).pow(2).mean().backward()
    ref(x).pow(2).mean().backward()
    with torch.no_grad():
        model(x)                                            # e.g. an evaluation batch between backward and step
    model(x)                                                # and a training-mode forward whose loss is never used
    opt.step(), ropt.step()
    _same_params(model, ref)


def test_no_sync_contexts_nest_and_survive_exceptions():
    model, ref = _pair()
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    units = [b._matrix_fsdp_param_group for b in model]
    x = torch.randn(4, 8)

    def both():
        model(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()

    with opt.no_sync():
        with units[0].no_sync():                                                   # one unit, inside the context of all
            both()
        assert all(u.in_no_sync and u.defer_backward_reduce for u in units)      # the outer context is still in force
        both()
        assert all(u.flat_buffer.pending_reduce is None and not u.flat_buffer.local_grad_valid for u in units)
    assert not any(u.in_no_sync or u.defer_backward_reduce for u in units)
    with pytest.raises(KeyboardInterrupt):
        with opt.no_sync():
            both()
            raise KeyboardInterrupt
    assert not any(u.in_no_sync or u.defer_backward_reduce for u in units)       # left cleanly
    both()                                                                        # reduces all four micro-batches
    opt.step(), ropt.step()
    _same_params(model, ref)
