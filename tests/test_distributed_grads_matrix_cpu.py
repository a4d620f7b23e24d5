"""Reduced gradients on gloo ranks, one (layout, norm) per case: the gradient shards assembled by
``gather_full_grads`` equal the eager model's rank-averaged gradients, the global norm computed from the shards
equals the eager norm, and clipping scales every shard by the same factor.

Two ranks for the flat layouts, four ranks (2 x 2 mesh) for HSDP; all cases of a world size share one spawn.
The reference checks gradient shards per planner in test/fsdp/test_matrix_fsdp_distributed.py:2910-2976."""
import copy
import itertools
import json
import math
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks

LAYOUTS = ("even", "fsdp2_chunks", "parameter_boundaries", "ordered_groups", "rows", "owners", "auto_balanced")
NORMS = ("2", "1", "inf")
CASES = [f"{l}-{n}" for l, n in itertools.product(LAYOUTS, NORMS)]
HSDP_CASES = [f"hsdp_{l}-{n}" for l, n in itertools.product(("even", "parameter_boundaries", "owners"), ("2", "inf"))]


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Sequential(nn.Linear(8, 12), nn.Tanh()), nn.Sequential(nn.LayerNorm(12), nn.Linear(12, 8)),
                         nn.Linear(8, 4, bias=False))


def _shard(model, layout, mesh_kw):
    from torch.distributed.tensor.placement_types import Shard

    from matrix_fsdp_b200 import fully_shard, matrix_fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.planning import planner as P

    reset_shared_owner_planners()
    for m in list(model.children())[:-1] + [model]:
        if layout == "even":
            fully_shard(m, **mesh_kw)
        elif layout == "rows":
            fully_shard(m, shard_placement_fn=lambda p: Shard(0), **mesh_kw)
        elif layout == "owners":
            fully_shard(m, optimizer_policy="mixed_muon_adamw", **mesh_kw)
        elif layout == "auto_balanced":
            matrix_fully_shard(m, auto_planner_policy="balanced", **mesh_kw)
        else:
            planner = {"fsdp2_chunks": P.fsdp2_chunk_plan, "parameter_boundaries": P.parameter_boundary_plan,
                       "ordered_groups": P.ordered_group_plan}[layout]
            matrix_fully_shard(m, group_planner=planner, **mesh_kw)


def _run_case(rank, world, name):
    from matrix_fsdp_b200 import configure_optimizer
    from matrix_fsdp_b200.utils import clip_grad_norm_
    from matrix_fsdp_b200.utils.training import gather_full_grads

    hsdp = name.startswith("hsdp_")
    layout, norm_name = name.removeprefix("hsdp_").split("-")
    norm_type = math.inf if norm_name == "inf" else float(norm_name)
    mesh_kw = {}
    if hsdp:
        from matrix_fsdp_b200 import DataParallelMeshDims

        mesh_kw = dict(mesh=_mesh(world), dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    model = _model()
    ref = copy.deepcopy(model)
    _shard(model, layout, mesh_kw)
    opt = configure_optimizer(model, "mixed_muon_adamw" if layout == "owners" else "sgd", lr=0.1)
    g = torch.Generator().manual_seed(50 + rank)
    x = torch.randn(4, 8, generator=g) * 2
    model(x).pow(2).mean().backward()
    ref(x).pow(2).mean().backward()
    for p in ref.parameters():
        dist.all_reduce(p.grad)
        p.grad /= world
    # 1. the shards are the averaged gradients
    got = gather_full_grads(model)
    assert set(got) == {n for n, _ in ref.named_parameters()}
    for n, p in ref.named_parameters():
        assert torch.allclose(got[n].view(p.shape), p.grad, atol=1e-6), (n, float((got[n].view(p.shape) - p.grad).abs().max()))
    # 2. the norm assembled from the shards is the eager norm
    rtotal = torch.nn.utils.get_total_norm([p.grad for p in ref.parameters()], norm_type)
    max_norm = float(rtotal) * 0.25
    total = clip_grad_norm_(model, max_norm, norm_type)
    assert torch.allclose(total, rtotal, rtol=1e-5), (float(total), float(rtotal))
    # 3. clipping scaled every shard by the same factor
    torch.nn.utils.clip_grad_norm_(ref.parameters(), max_norm, norm_type)
    got = gather_full_grads(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(got[n].view(p.shape), p.grad, atol=1e-6), n
    # 4. a second call is a no-op (already inside the ball) and the step still runs
    again = clip_grad_norm_(model, max_norm * 1.001, norm_type)
    assert float(again) <= max_norm * 1.001
    opt.step()
    opt.zero_grad()


_MESH = {}


def _mesh(world):
    if world not in _MESH:
        from torch.distributed.device_mesh import init_device_mesh

        _MESH[world] = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    return _MESH[world]


def _worker(rank, world, out_path, names):
    results = {}
    for name in names:
        try:
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


def _spawn(world, names):
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, world, path, names, timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.fixture(scope="module")
def outcomes():
    return _spawn(2, CASES)


@pytest.fixture(scope="module")
def hsdp_outcomes():
    return _spawn(4, HSDP_CASES)


@pytest.mark.parametrize("case", CASES)
def test_two_rank_gradient_shards_norm_and_clipping(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]


@pytest.mark.parametrize("case", HSDP_CASES)
def test_four_rank_hsdp_gradient_shards_norm_and_clipping(hsdp_outcomes, case):
    assert case in hsdp_outcomes, "the worker did not reach this case"
    assert not hsdp_outcomes[case], hsdp_outcomes[case]
