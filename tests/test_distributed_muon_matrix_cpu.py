"""Mixed Muon / AdamW on gloo ranks, one (wrapping, owner assignment, Muon option) per case: three steps of the
sharded model equal an unsharded model stepped by the same optimizer classes on the rank-averaged gradients
(so the comparison is tight: the only difference is who owns which matrix).  Each case also checks that Muon state
exists only on the owner of a matrix, that no matrix is split, and that the owners together cover every matrix.

Two ranks (flat) and four ranks (HSDP 2 x 2, with and without the replicas sharing Newton-Schulz); all cases of a
world size share one spawn.  The reference has one such test per world
(test/fsdp/test_matrix_fsdp_distributed.py:2899, 3333)."""
import copy
import json
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks

_MUON = dict(muon_momentum=0.9, muon_ns_steps=3, muon_nesterov=True, muon_adjust_lr_fn="original")

# name -> (how the model is sharded, keyword overrides for the optimizer)
CASES = {
    "policy_api-units": ("fully_shard", "units", None, {}),
    "policy_api-root": ("fully_shard", "root", None, {}),
    "rotate-units": ("matrix", "units", "rotate", {}),
    "rotate-root": ("matrix", "root", "rotate", {}),
    "role_greedy-units": ("matrix", "units", "role_greedy", {}),
    "role_greedy-wrap_policy": ("matrix", "policy", "role_greedy", {}),
    "cost_aware-wrap_policy": ("matrix", "policy", "cost_aware", {}),
    "scope_greedy-wrap_policy": ("matrix", "policy", "scope_greedy", {}),
    "model_wide-wrap_policy": ("matrix", "policy", "model_wide", {}),
    "no_nesterov": ("fully_shard", "units", None, dict(muon_nesterov=False)),
    "match_rms_adamw": ("fully_shard", "units", None, dict(muon_adjust_lr_fn="match_rms_adamw")),
    "no_lr_adjust": ("fully_shard", "units", None, dict(muon_adjust_lr_fn=None)),
    "five_ns_steps": ("fully_shard", "units", None, dict(muon_ns_steps=5)),
    "weight_decay": ("fully_shard", "units", None, dict(weight_decay=0.1)),
    "separate_lrs": ("fully_shard", "units", None, dict(muon_lr=0.03, adamw_lr=0.004)),
    "separate_decays": ("fully_shard", "units", None, dict(muon_weight_decay=0.2, adamw_weight_decay=0.05)),
    "adamw_betas_eps": ("fully_shard", "units", None, dict(adamw_betas=(0.8, 0.9), adamw_eps=1e-6)),
}
HSDP_CASES = {
    "hsdp-shared_ns": ("fully_shard", "units", None, {}),
    "hsdp-own_ns": ("fully_shard", "units", None, dict(muon_share_ns_across_replicas=False)),
    "hsdp-root-shared_ns": ("fully_shard", "root", None, {}),
    "hsdp-role_greedy-wrap_policy": ("matrix", "policy", "role_greedy", {}),
    "hsdp-weight_decay": ("fully_shard", "units", None, dict(weight_decay=0.1)),
}


class Blk(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = nn.Linear(d, 2 * d)
        self.n = nn.LayerNorm(2 * d)
        self.b = nn.Linear(2 * d, d, bias=False)

    def forward(self, x):
        return x + self.b(torch.tanh(self.n(self.a(x))))


def _model():
    torch.manual_seed(0)
    m = nn.Sequential(*[Blk(8) for _ in range(3)])
    m.add_module("head", nn.Linear(8, 8))
    return m


_MESH = {}


def _shard(model, api, wrap, assignment, mesh_kw):
    from matrix_fsdp_b200 import fully_shard, matrix_fully_shard
    from matrix_fsdp_b200.policy.wrap import module_type_policy

    if api == "fully_shard":
        for m in ([] if wrap == "root" else list(model.children())[:-1]) + [model]:
            fully_shard(m, optimizer_policy="mixed_muon_adamw", **mesh_kw)
        return
    kw = dict(auto_planner_policy="muon_shard_aware", owner_assignment=assignment, auto_shard_hints=True, **mesh_kw)
    if wrap == "policy":
        matrix_fully_shard(model, wrap_policy=module_type_policy(Blk), **kw)
        rest = dict(kw, owner_assignment="rotate") if assignment in ("scope_greedy", "cost_aware", "model_wide") else kw
        matrix_fully_shard(model, **rest)                    # the root unit takes what the blocks left (the head)
    else:
        for m in ([] if wrap == "root" else list(model.children())[:-1]) + [model]:
            matrix_fully_shard(m, **kw)


def _reference_optimizers(ref, kw):
    """The same optimizer classes on the unsharded model: Muon on every matrix, AdamW on the rest."""
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    lr, wd = kw.get("lr", 0.02), kw.get("weight_decay", 0.0)
    matrices = [p for p in ref.parameters() if p.ndim == 2]
    others = [p for p in ref.parameters() if p.ndim != 2]
    muon = MatrixMuon(matrices, lr=kw.get("muon_lr", lr), weight_decay=kw.get("muon_weight_decay", wd),
                      momentum=kw["muon_momentum"], nesterov=kw["muon_nesterov"], ns_steps=kw["muon_ns_steps"],
                      adjust_lr_fn=kw["muon_adjust_lr_fn"])
    adamw = torch.optim.AdamW(others, lr=kw.get("adamw_lr", lr), weight_decay=kw.get("adamw_weight_decay", wd),
                              betas=kw.get("adamw_betas", (0.9, 0.999)), eps=kw.get("adamw_eps", 1e-8))
    return muon, adamw


def _full_params(model):
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    units = collect_param_groups(model)
    for u in units:
        u.unshard("test")
    out = {n: p.detach().clone().float() for n, p in model.named_parameters()}
    for u in units:
        u.reshard("test")
    return out


def _run_case(rank, world, name):
    from matrix_fsdp_b200 import configure_optimizer
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    hsdp = name.startswith("hsdp-")
    api, wrap, assignment, overrides = (HSDP_CASES if hsdp else CASES)[name]
    mesh_kw = {}
    if hsdp:
        from torch.distributed.device_mesh import init_device_mesh

        from matrix_fsdp_b200 import DataParallelMeshDims

        if world not in _MESH:
            _MESH[world] = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        mesh_kw = dict(mesh=_MESH[world], dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    reset_shared_owner_planners()
    model = _model()
    ref = copy.deepcopy(model)
    _shard(model, api, wrap, assignment, mesh_kw)
    kw = dict(_MUON, lr=0.02, weight_decay=0.0)
    kw.update(overrides)
    opt = configure_optimizer(model, "mixed_muon_adamw", **kw)
    rmuon, radamw = _reference_optimizers(ref, kw)
    g = torch.Generator().manual_seed(7 + rank)
    for _ in range(3):
        x = torch.randn(4, 8, generator=g)
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        for p in ref.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        rmuon.step(); radamw.step(); rmuon.zero_grad(); radamw.zero_grad()
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=2e-5, rtol=1e-4), (n, float((full[n] - p.detach()).abs().max()))
    # ownership: every matrix whole on exactly one rank of the shard group, Muon state only there
    units = collect_param_groups(model)
    owned = {id(p) for grp in opt.muon.param_groups for p in grp["params"] if p.numel()}
    mine = 0
    for u in units:
        for mp in u.registry:
            if len(mp.shape) != 2:
                continue
            owners = u.owner_ranks(mp.fqn)
            assert len(owners) == 1, (mp.fqn, owners)
            is_owner = owners == (u.rank,)
            assert (id(mp.param) in owned) == is_owner, mp.fqn
            mine += int(is_owner)
    shard_world = units[0].world_size
    counts = [None] * world
    dist.all_gather_object(counts, mine)
    n_matrices = sum(1 for p in ref.parameters() if p.ndim == 2)
    assert sum(counts) == n_matrices * (world // shard_world), counts           # each replica owns every matrix once
    if hsdp and overrides.get("muon_share_ns_across_replicas", True):
        done = [None] * world
        dist.all_gather_object(done, opt.muon.ns_matrices_done if hasattr(opt.muon, "ns_matrices_done") else 0)
        assert sum(done) == n_matrices, done                                     # replicas split the work, no repeats


def _lonely_rank_case(rank, world):
    """One matrix, two ranks: one of them owns no matrix at all.  Its ``opt.muon`` is still a torch optimizer (LR
    schedulers attach on every rank), checkpoints round-trip, and training matches the unsharded optimizers."""
    import tempfile as _tempfile

    from matrix_fsdp_b200 import configure_optimizer, fully_shard, load_matrix_dcp, save_matrix_dcp
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.optim.muon import MatrixMuon

    def build(seed):
        reset_shared_owner_planners()
        torch.manual_seed(seed)
        m = nn.Sequential(nn.Linear(8, 8))
        fully_shard(m, optimizer_policy="mixed_muon_adamw")
        return m, configure_optimizer(m, "mixed_muon_adamw", **dict(_MUON, lr=0.02, weight_decay=0.0))

    model, opt = build(0)
    torch.manual_seed(0)
    ref = nn.Sequential(nn.Linear(8, 8))
    unit = model._matrix_fsdp_param_group
    owners = [None] * world
    dist.all_gather_object(owners, unit.owner_ranks("0.weight") == (rank,))
    assert sum(owners) == 1                                            # exactly one rank owns the matrix
    assert isinstance(opt.muon, torch.optim.Optimizer) and isinstance(opt.adamw, torch.optim.Optimizer)
    scheds = [torch.optim.lr_scheduler.StepLR(o, step_size=1, gamma=0.5) for o in (opt.muon, opt.adamw)]
    rmuon = MatrixMuon([ref[0].weight], lr=0.02, weight_decay=0.0, momentum=_MUON["muon_momentum"], nesterov=True,
                       ns_steps=_MUON["muon_ns_steps"], adjust_lr_fn="original")
    radamw = torch.optim.AdamW([ref[0].bias], lr=0.02, weight_decay=0.0)
    rscheds = [torch.optim.lr_scheduler.StepLR(o, step_size=1, gamma=0.5) for o in (rmuon, radamw)]
    g = torch.Generator().manual_seed(3 + rank)
    for _ in range(3):
        x = torch.randn(4, 8, generator=g)
        model(x).pow(2).mean().backward()
        ref(x).pow(2).mean().backward()
        for p in ref.parameters():
            dist.all_reduce(p.grad)
            p.grad /= world
        opt.step(); rmuon.step(); radamw.step()
        opt.zero_grad(); rmuon.zero_grad(); radamw.zero_grad()
        for s in scheds + rscheds:
            s.step()
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=2e-5), n
    base = [None]
    if rank == 0:
        base[0] = _tempfile.mkdtemp()
    dist.broadcast_object_list(base, src=0)
    save_matrix_dcp(model, base[0], optimizer=opt)
    dist.barrier()
    twin, topt = build(4)
    load_matrix_dcp(twin, base[0], optimizer=topt)
    assert torch.equal(twin._matrix_fsdp_param_group.flat_buffer.local_shard, unit.flat_buffer.local_shard)
    assert [g_["lr"] for g_ in topt.param_groups] == [g_["lr"] for g_ in opt.param_groups]


def _worker(rank, world, out_path, which):
    results = {}
    for name in (HSDP_CASES if which == "hsdp" else list(CASES) + ["lonely_rank"]):
        try:
            if name == "lonely_rank":
                _lonely_rank_case(rank, world)
            else:
                _run_case(rank, world, name)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        results[name] = "\n".join(f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


def _spawn(world, which):
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, world, path, which, timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.fixture(scope="module")
def outcomes():
    return _spawn(2, "flat")


@pytest.fixture(scope="module")
def hsdp_outcomes():
    return _spawn(4, "hsdp")


@pytest.mark.parametrize("case", sorted(CASES))
def test_two_rank_mixed_muon_matches_unsharded_optimizers(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]


@pytest.mark.parametrize("case", sorted(HSDP_CASES))
def test_four_rank_hsdp_mixed_muon_matches_unsharded_optimizers(hsdp_outcomes, case):
    assert case in hsdp_outcomes, "the worker did not reach this case"
    assert not hsdp_outcomes[case], hsdp_outcomes[case]


def test_two_ranks_one_matrix_the_rank_without_it_still_has_a_muon_optimizer(outcomes):
    assert "lonely_rank" in outcomes, "the worker did not reach this case"
    assert not outcomes["lonely_rank"], outcomes["lonely_rank"]
