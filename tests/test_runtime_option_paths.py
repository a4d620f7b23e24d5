"""Runtime options that select a different code path must really take it: saved-tensor hooks, zero-copy
gradient bucket, keeping the unsharded storage, gather / reduce strategies, measuring prefetch policies."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import check_case, run_cases
from matrix_fsdp_b200 import configure_optimizer, fully_shard, matrix_fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


class ViewSaver(nn.Module):
    """Uses explicit transposed views of its weights, which autograd saves as views of the full buffer."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(0)
        self.w1 = nn.Parameter(torch.randn(10, 6) * 0.3)
        self.w2 = nn.Parameter(torch.randn(4, 10) * 0.3)

    def forward(self, x):
        return torch.tanh(x @ self.w1.t()) @ self.w2.t()


def _x(seed=1, n=3):
    return torch.randn(n, 6, generator=torch.Generator().manual_seed(seed))


def _full(model):
    units = collect_param_groups(model)
    for u in units:
        u.unshard("check")
    out = {n: p.detach().clone().float() for n, p in model.named_parameters()}
    for u in units:
        u.reshard("check")
    return out


def test_saved_tensor_hooks_replace_saved_views_of_the_full_buffer():
    reset_shared_owner_planners()
    model, ref = ViewSaver(), ViewSaver()
    matrix_fully_shard(model, use_saved_tensor_hooks=True)
    unit = model._matrix_fsdp_param_group
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for s in range(3):
        model(_x(s)).pow(2).mean().backward()
        ref(_x(s)).pow(2).mean().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    assert unit._saved_view_count > 0, "no saved tensor went through the hooks"
    names = [e.name for e in unit.runtime_events]
    assert "enter_saved_tensor_hooks" in names and "exit_saved_tensor_hooks" in names
    for (n, p), (_, q) in zip(_full(model).items(), ref.named_parameters()):
        assert torch.allclose(p, q.detach(), atol=1e-6), n


def test_zero_copy_grad_bucket_lets_autograd_write_the_bucket():
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 10), nn.Tanh(), nn.Linear(10, 4))
    ref = copy.deepcopy(model)
    matrix_fully_shard(model, use_zero_copy_grad_bucket=True)
    unit = model._matrix_fsdp_param_group
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    for s in range(2):
        model(_x(s)).pow(2).mean().backward()
        ref(_x(s)).pow(2).mean().backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    names = [e.name for e in unit.runtime_events]
    assert "attach_zero_copy_grads" in names
    fin = [e for e in unit.runtime_events if e.name == "finalize_backward"]
    assert fin and all(e.extra.get("copy_in") == "direct" for e in fin), [e.extra for e in fin]
    for (n, p), (_, q) in zip(_full(model).items(), ref.named_parameters()):
        assert torch.allclose(p, q.detach(), atol=1e-6), n


def test_zero_copy_grad_bucket_accumulates_under_no_sync():
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 10), nn.Tanh(), nn.Linear(10, 4))
    ref = copy.deepcopy(model)
    matrix_fully_shard(model, use_zero_copy_grad_bucket=True)
    opt, ropt = configure_optimizer(model, "sgd", lr=0.1), torch.optim.SGD(ref.parameters(), lr=0.1)
    with model.no_sync():
        model(_x(0)).pow(2).mean().backward()
    model(_x(1)).pow(2).mean().backward()
    ref(_x(0)).pow(2).mean().backward()
    ref(_x(1)).pow(2).mean().backward()
    opt.step(), ropt.step()
    for (n, p), (_, q) in zip(_full(model).items(), ref.named_parameters()):
        assert torch.allclose(p, q.detach(), atol=1e-6), n


def test_keeping_unsharded_storage_after_backward():
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(6, 10), nn.Tanh(), nn.Linear(10, 4))
    # a planner that splits: world size 1 with an aliasing full buffer has no storage of its own to keep
    from matrix_fsdp_b200.core.layout import ShardPlan

    keep = copy.deepcopy(model)
    matrix_fully_shard(model)
    matrix_fully_shard(keep, shrink_full_param_storage_after_backward=False)
    for m in (model, keep):
        m(_x()).sum().backward()
    a, b = model._matrix_fsdp_param_group, keep._matrix_fsdp_param_group
    assert a.state.value == b.state.value == "sharded"
    if not a.flat_buffer.full_aliases_shard:
        assert a.full_param_storage_nbytes() == 0 and b.full_param_storage_nbytes() > 0
    del ShardPlan


def test_unknown_strategy_names_are_rejected():
    for kw in (dict(param_gather_strategy="nope"), dict(matrix_collective_backend="nope"),
               dict(backward_reduce_strategy="nope")):
        with pytest.raises(ValueError):
            matrix_fully_shard(nn.Linear(4, 4), **kw)


# ----------------------------------------------------------------------------- two ranks (gloo)
def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(8, 12), nn.Tanh(), nn.Linear(12, 8, bias=False))


def _train(model, rank, steps=3, opt_kind="adamw"):
    opt = configure_optimizer(model, opt_kind, lr=1e-2)
    g = torch.Generator().manual_seed(50 + rank)
    for _ in range(steps):
        model(torch.randn(4, 8, generator=g)).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    return torch.cat([u.flat_buffer.local_shard.flatten() for u in collect_param_groups(model)])


def _strategy_body(rank, world, kw, expect_impl_kind, expect_impl):
    reset_shared_owner_planners()
    base = _model()
    matrix_fully_shard(base)
    want = _train(base, rank)
    reset_shared_owner_planners()
    model = _model()
    matrix_fully_shard(model, **kw)
    got = _train(model, rank)
    assert torch.allclose(got, want, atol=1e-6), (got - want).abs().max()
    unit = model._matrix_fsdp_param_group
    impls = {e.collective_impl for e in unit.runtime_events if e.collective_kind == expect_impl_kind}
    assert expect_impl in impls, impls


_STRATEGIES = [
    (dict(backward_reduce_strategy="flat"), "reduce_scatter", "reduce_scatter_tensor"),
    (dict(backward_reduce_strategy="per_param"), "reduce_scatter", "per_param_reduce_scatter"),
    (dict(backward_reduce_strategy="per_param_allreduce"), "all_reduce", "per_param_allreduce"),
    (dict(param_gather_strategy="equal_all_gather"), "all_gather", "all_gather_into_tensor"),
    (dict(param_gather_strategy="matrix_all_gather"), "all_gather", "padded_all_gather"),
    (dict(param_gather_strategy="all_reduce"), "all_gather", "all_reduce_gather"),
    (dict(param_gather_strategy="uneven_all_gather"), "all_gather", "padded_all_gather"),   # gloo: falls back
]


def _strategy_name(kw):
    return "strategy:" + ",".join(f"{k}={v}" for k, v in kw.items())


@pytest.fixture(scope="module")
def two_rank_outcomes():
    """Every two-rank case of this file in one spawn (see ``dist_utils.run_cases``)."""
    cases = [(_strategy_name(kw), _strategy_body, (kw, kind, impl)) for kw, kind, impl in _STRATEGIES]
    cases.append(("owner_broadcast", _owner_broadcast_body, ()))
    cases += [(f"policy:{p}", _policy_body, (p,)) for p in ("adaptive", "profile_guided")]
    cases.append(("pooled", _pooled_body, ()))
    return run_cases(2, cases)


@pytest.mark.parametrize("kw,kind,impl", _STRATEGIES)
def test_strategy_selects_its_collective_and_keeps_the_result(two_rank_outcomes, kw, kind, impl):
    check_case(two_rank_outcomes, _strategy_name(kw))


def _owner_broadcast_body(rank, world):
    reset_shared_owner_planners()
    even = _model()
    matrix_fully_shard(even, param_gather_strategy="owner_broadcast")      # even split: parameters are cut
    with pytest.raises(RuntimeError, match="whole-parameter owner"):
        even(torch.randn(2, 8))
    dist.barrier()
    reset_shared_owner_planners()
    base = _model()
    fully_shard(base, optimizer_policy="mixed_muon_adamw")
    want = _train(base, rank, opt_kind="sgd")
    reset_shared_owner_planners()
    owner = _model()
    matrix_fully_shard(owner, auto_shard_hints=True, auto_planner_policy="muon_shard_aware",
                       owner_assignment="role_greedy", param_gather_strategy="owner_broadcast")
    got = _train(owner, rank, opt_kind="sgd")
    assert torch.allclose(got, want, atol=1e-6)
    impls = {e.collective_impl for e in owner._matrix_fsdp_param_group.runtime_events if e.collective_kind == "all_gather"}
    assert "owner_broadcast" in impls, impls


def test_owner_broadcast_strategy_needs_whole_parameter_owners(two_rank_outcomes):
    check_case(two_rank_outcomes, "owner_broadcast")


def _policy_body(rank, world, policy):
    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(*[nn.Sequential(nn.Linear(8, 8), nn.Tanh()) for _ in range(4)])
    for blk in model:
        fully_shard(blk)
    opt = configure_optimizer(model, "sgd", lr=0.01, prefetch_policy=policy, adaptive_wait_threshold_ms=0.0,
                              profile_iterations=1, max_unsharded_prefetch_units=1)
    sched = model[0]._matrix_fsdp_param_group.scheduler
    assert sched.config.prefetch_policy == policy
    g = torch.Generator().manual_seed(rank)
    for _ in range(6):
        model(torch.randn(4, 8, generator=g)).sum().backward()
        opt.step()
        opt.zero_grad()
    c = sched.counters
    assert c.mean_unshard_wait_us >= 0 and c.iterations == 6
    if policy == "adaptive":
        # every measured wait is above a threshold of 0: the depth grew to the cap and was used
        assert sched._fwd_budget() == 2 and c.policy_adjustments >= 1
    else:
        assert sched._profile["done"] and set(sched._profile["results"]) == {1, 2}
        assert sched._fwd_budget() in (1, 2)


@pytest.mark.parametrize("policy", ["adaptive", "profile_guided"])
def test_measuring_prefetch_policies_change_the_depth_from_measured_waits(two_rank_outcomes, policy):
    check_case(two_rank_outcomes, f"policy:{policy}")


def _pooled_body(rank, world):
    """With saved-tensor hooks the unsharded buffers come from the scheduler's pool and are reused."""
    reset_shared_owner_planners()
    torch.manual_seed(0)
    blocks = [ViewSaver() for _ in range(3)]
    model = nn.Sequential()
    for i, b in enumerate(blocks):
        model.add_module(str(i), nn.Sequential())
    # three same-shaped units chained through a 6 -> 4 -> (pad) projection
    class Chain(nn.Module):
        def __init__(self):
            super().__init__()
            self.blocks = nn.ModuleList(blocks)
            self.up = nn.Linear(4, 6)

        def forward(self, x):
            for b in self.blocks:
                x = self.up(b(x))
            return x

    net, ref = Chain(), None
    ref = copy.deepcopy(net)
    for b in net.blocks:
        matrix_fully_shard(b, use_saved_tensor_hooks=True)
    fully_shard(net)
    opt, ropt = configure_optimizer(net, "sgd", lr=0.05), torch.optim.SGD(ref.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(3 + rank)
    for _ in range(3):
        x = torch.randn(4, 6, generator=g)
        net(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        for p in ref.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    unit = net.blocks[0]._matrix_fsdp_param_group
    pool = unit.scheduler.comm.full_param_pool
    assert unit.flat_buffer.full_pool is pool
    st = pool.stats
    assert st.acquires >= 18 and st.reuses > 0 and st.allocations < st.acquires, st.as_dict()
    assert unit.full_param_storage_nbytes() == 0
    for (n, p), (_, q) in zip(_full(net).items(), ref.named_parameters()):
        assert torch.allclose(p, q.detach(), atol=1e-6), n


def test_saved_tensor_hooks_take_unsharded_buffers_from_the_pool(two_rank_outcomes):
    check_case(two_rank_outcomes, "pooled")
