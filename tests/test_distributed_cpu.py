"""Multi-rank lifecycle on CPU (gloo): sharded training equals the single-process model."""
import copy

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import check_case, run_cases


class Blk(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = nn.Linear(d, 2 * d)
        self.n = nn.LayerNorm(2 * d)
        self.b = nn.Linear(2 * d, d, bias=False)

    def forward(self, x):
        return x + self.b(torch.relu(self.n(self.a(x))))


def _model(d=8, n=3):
    torch.manual_seed(0)
    m = nn.Sequential(*[Blk(d) for _ in range(n)])
    m.add_module("head", nn.Linear(d, d))
    return m


def _allreduce_grads(model, world):
    for p in model.parameters():
        if p.grad is not None:
            dist.all_reduce(p.grad)
            p.grad /= world


def _full_params(model):
    """Gather every unit and return {fqn: full tensor} (debug helper used by the tests)."""
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    out = {}
    units = collect_param_groups(model)
    for u in units:
        u.unshard("test")
    for n, p in model.named_parameters():
        out[n] = p.detach().clone().float()
    for u in units:
        u.reshard("test")
    return out


def _train_compare(rank, world, kind, shard_kwargs, opt_kind, opt_kwargs, steps=3, tol=2e-5):
    from matrix_fsdp_b200.api import fully_shard
    from matrix_fsdp_b200.optim import configure_optimizer

    model = _model()
    ref = copy.deepcopy(model)
    mesh = None
    kw = dict(shard_kwargs)
    if kind == "hsdp":
        from torch.distributed.device_mesh import init_device_mesh
        from matrix_fsdp_b200 import DataParallelMeshDims

        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        kw["dp_mesh_dims"] = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    elif kind == "mesh1d":
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh("cpu", (world,))
    for blk in list(model.children())[:-1]:
        fully_shard(blk, mesh=mesh, **kw)
    fully_shard(model, mesh=mesh, **kw)
    opt = configure_optimizer(model, opt_kind, **opt_kwargs)
    if opt_kind == "adamw":
        ropt = torch.optim.AdamW(ref.parameters(), **opt_kwargs)
    elif opt_kind == "sgd":
        ropt = torch.optim.SGD(ref.parameters(), **opt_kwargs)
    else:
        raise AssertionError(opt_kind)
    g = torch.Generator().manual_seed(100 + rank)
    for _ in range(steps):
        x = torch.randn(4, 8, generator=g)
        loss = model(x).pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad()
        rl = ref(x).pow(2).mean()
        rl.backward()
        _allreduce_grads(ref, world)
        ropt.step()
        ropt.zero_grad()
        assert torch.allclose(loss, rl, atol=1e-5), (loss.item(), rl.item())
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=tol, rtol=1e-4), n
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    for u in collect_param_groups(model):
        assert u.state.value == "sharded"
        assert u.full_param_storage_nbytes() == 0


def _world_dense(rank, world):
    _train_compare(rank, world, "world", {}, "adamw", dict(lr=1e-2, weight_decay=0.1))


def _mesh_rows(rank, world):
    from torch.distributed.tensor.placement_types import Shard

    _train_compare(rank, world, "mesh1d", dict(shard_placement_fn=lambda p: Shard(0)), "sgd",
                   dict(lr=0.1, momentum=0.9))


def _hsdp(rank, world):
    _train_compare(rank, world, "hsdp", {}, "adamw", dict(lr=1e-2, weight_decay=0.0))


@pytest.fixture(scope="module")
def two_rank_outcomes():
    """Every two-rank case of this file in one spawn (see ``dist_utils.run_cases``)."""
    return run_cases(2, [("dense", _world_dense, ()), ("rows", _mesh_rows, ()), ("muon_owner", _muon_owner, ()),
                         ("no_sync", _no_sync_and_accumulation, ())])


def test_two_rank_dense_even_split_adamw(two_rank_outcomes):
    check_case(two_rank_outcomes, "dense")


def test_two_rank_row_sharding_sgd(two_rank_outcomes):
    check_case(two_rank_outcomes, "rows")


def test_four_rank_hsdp_2x2():
    check_case(run_cases(4, [("hsdp", _hsdp, ())]), "hsdp")


def _muon_owner(rank, world):
    from matrix_fsdp_b200.api import fully_shard, reset_shared_owner_planners
    from matrix_fsdp_b200.optim import configure_optimizer

    reset_shared_owner_planners()
    model = _model(d=8, n=2)
    ref = copy.deepcopy(model)
    for blk in list(model.children())[:-1]:
        fully_shard(blk, optimizer_policy="mixed_muon_adamw")
    fully_shard(model, optimizer_policy="mixed_muon_adamw")
    units = [m._matrix_fsdp_param_group for m in model.children() if hasattr(m, "_matrix_fsdp_param_group")]
    assert units[0].planner_result.name == "matrix_owner_tail_role_greedy"
    assert units[0].planner_result.policy == "muon_shard_aware"
    opt = configure_optimizer(model, "mixed_muon_adamw", lr=0.02, muon_momentum=0.95, muon_ns_steps=5,
                              muon_adjust_lr_fn="original", weight_decay=0.0)
    muon_ref = [p for n, p in ref.named_parameters() if p.ndim == 2]
    other_ref = [p for n, p in ref.named_parameters() if p.ndim != 2]
    rm = torch.optim.Muon(muon_ref, lr=0.02, momentum=0.95, ns_steps=5, weight_decay=0.0)
    ra = torch.optim.AdamW(other_ref, lr=0.02, weight_decay=0.0)
    g = torch.Generator().manual_seed(7 + rank)
    for _ in range(2):
        x = torch.randn(4, 8, generator=g)
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        _allreduce_grads(ref, world)
        rm.step(); ra.step(); rm.zero_grad(); ra.zero_grad()
    # only owners hold Muon state
    owned = {id(p) for grp in opt.muon.param_groups for p in grp["params"]}
    for u in units:
        for mp in u.registry:
            if mp.param.ndim == 2 or len(mp.shape) == 2:
                is_owner = u.owner_ranks(mp.fqn) == (u.rank,)
                assert (id(mp.param) in owned) == is_owner
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=2e-2, rtol=2e-2), n


def test_two_rank_matrix_owner_mixed_muon(two_rank_outcomes):
    check_case(two_rank_outcomes, "muon_owner")


def _no_sync_and_accumulation(rank, world):
    from matrix_fsdp_b200.api import fully_shard
    from matrix_fsdp_b200.optim import configure_optimizer

    model = _model()
    ref = copy.deepcopy(model)
    for blk in list(model.children())[:-1]:
        fully_shard(blk)
    fully_shard(model)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(3 + rank)
    xs = [torch.randn(4, 8, generator=g) for _ in range(3)]
    with model.no_sync():
        model(xs[0]).pow(2).mean().backward()
        with pytest.raises(RuntimeError, match="no_sync"):
            opt.step()
    model(xs[1]).pow(2).mean().backward()     # reduces the accumulated bucket
    model(xs[2]).pow(2).mean().backward()     # a third micro-batch without no_sync: accumulates locally
    opt.step()
    opt.zero_grad()
    for x in xs:
        ref(x).pow(2).mean().backward()
    _allreduce_grads(ref, world)
    ropt.step()
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=1e-5), n


def test_two_rank_no_sync_and_grad_accumulation(two_rank_outcomes):
    check_case(two_rank_outcomes, "no_sync")
