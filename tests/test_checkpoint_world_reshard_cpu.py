"""matrix_dcp checkpoints cross world sizes: written by 1 process, 2 and 3 flat gloo ranks, 2 replicas (nothing sharded) and 4 gloo ranks (HSDP 2 x 2),
each read back, re-sharded, by every OTHER arrangement.  Parameters have to arrive bitwise, and one more training
step (optimizer state included) has to land where the writer's own next step landed.  Every rank of every
arrangement trains on the same batch, so the averaged gradient does not depend on the arrangement.

One spawn per arrangement does all of its loads (and, the first time, its saves); each (writer, reader, optimizer)
is reported as its own test.  The reference covers 1 <-> 2 ranks in
test/fsdp/test_matrix_fsdp_distributed.py:3054-3121."""
import json
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks

ARRANGEMENTS = ("w1", "w2", "w2rep", "w3", "w4hsdp")
OPTIMIZERS = ("adamw", "sgd", "mixed_muon_adamw")
CASES = [f"{src}->{dst}:{opt}" for src in ARRANGEMENTS for dst in ARRANGEMENTS if src != dst for opt in OPTIMIZERS]


def _model(seed):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(6, 10), nn.Tanh()), nn.Sequential(nn.LayerNorm(10), nn.Linear(10, 6)),
                         nn.Linear(6, 4))


def _build(seed, opt_kind, arrangement):
    from matrix_fsdp_b200 import configure_optimizer, fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    kw = {}
    if arrangement == "w4hsdp":
        from torch.distributed.device_mesh import init_device_mesh

        from matrix_fsdp_b200 import DataParallelMeshDims

        if "mesh" not in _CACHE:
            _CACHE["mesh"] = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        kw = dict(mesh=_CACHE["mesh"], dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    if arrangement == "w2rep":                                # two replicas, nothing sharded: only one of them writes
        from torch.distributed.device_mesh import init_device_mesh

        from matrix_fsdp_b200 import DataParallelMeshDims

        if "rep" not in _CACHE:
            _CACHE["rep"] = init_device_mesh("cpu", (2, 1), mesh_dim_names=("dp_replicate", "dp_shard"))
        kw = dict(mesh=_CACHE["rep"], dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    model = _model(seed)
    for m in list(model.children())[:-1] + [model]:
        fully_shard(m, optimizer_policy="mixed_muon_adamw" if opt_kind == "mixed_muon_adamw" else None, **kw)
    hyper = {"adamw": dict(lr=1e-2, weight_decay=0.01), "sgd": dict(lr=0.05, momentum=0.9),
             "mixed_muon_adamw": dict(lr=0.01)}[opt_kind]
    return model, configure_optimizer(model, opt_kind, **hyper)


_CACHE = {}


def _step(model, opt, index):
    x = torch.randn(3, 6, generator=torch.Generator().manual_seed(500 + index))     # the same on every rank
    model(x).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()


def _full(model):
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

    return get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))


def _save_all(arrangement, base_dir, rank, no_dist):
    from matrix_fsdp_b200 import save_matrix_dcp

    for opt_kind in OPTIMIZERS:
        model, opt = _build(0, opt_kind, arrangement)
        for i in range(2):
            _step(model, opt, i)
        directory = os.path.join(base_dir, f"{arrangement}-{opt_kind}")
        if rank == 0:
            os.makedirs(directory, exist_ok=True)
        if not no_dist:
            dist.barrier()
        save_matrix_dcp(model, directory, optimizer=opt, no_dist=True if no_dist else None)
        before = _full(model)
        _step(model, opt, 2)
        after = _full(model)
        if rank == 0:
            torch.save({"before": before, "after": after}, os.path.join(directory, "expected.pt"))
        if not no_dist:
            dist.barrier()


def _load_case(src, dst, opt_kind, base_dir, no_dist):
    from matrix_fsdp_b200 import load_matrix_dcp

    directory = os.path.join(base_dir, f"{src}-{opt_kind}")
    expected = torch.load(os.path.join(directory, "expected.pt"))
    model, opt = _build(7, opt_kind, dst)
    load_matrix_dcp(model, directory, optimizer=opt, allow_reshard=True, no_dist=True if no_dist else None)
    got = _full(model)
    for k, v in expected["before"].items():
        assert torch.equal(got[k], v), k
    _step(model, opt, 2)
    got = _full(model)
    tol = 2e-5 if opt_kind == "mixed_muon_adamw" else 2e-6
    for k, v in expected["after"].items():
        assert torch.allclose(got[k], v, atol=tol), (k, float((got[k] - v).abs().max()))


def _stage(arrangement, base_dir, sources, *, save, rank=0, world=1):
    """Everything one arrangement does in one visit: write its own checkpoints (first visit), read the others'."""
    no_dist = arrangement == "w1"
    if save:
        _save_all(arrangement, base_dir, rank, no_dist)
    results = {}
    for src in sources:
        for opt_kind in OPTIMIZERS:
            try:
                _load_case(src, arrangement, opt_kind, base_dir, no_dist)
                mine = ""
            except Exception:
                mine = traceback.format_exc()
            if no_dist:
                results[f"{src}->{arrangement}:{opt_kind}"] = mine
            else:
                gathered = [None] * world
                dist.all_gather_object(gathered, mine)
                results[f"{src}->{arrangement}:{opt_kind}"] = "\n".join(
                    f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    return results


def _worker(rank, world, jobs, base_dir, save, out_path):
    results = {}
    for arrangement, sources in jobs:                       # every arrangement of this world size in one spawn
        results.update(_stage(arrangement, base_dir, sources, save=save, rank=rank, world=world))
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


_WORLD = {"w2": 2, "w2rep": 2, "w3": 3, "w4hsdp": 4}


def _visit(jobs, base_dir, save):
    """``jobs``: [(arrangement, sources), ...] of one world size."""
    if jobs[0][0] == "w1":
        return _stage("w1", base_dir, jobs[0][1], save=save)
    world = _WORLD[jobs[0][0]]
    assert all(_WORLD[a] == world for a, _ in jobs)
    out_path = os.path.join(base_dir, f"outcomes-{world}-{int(save)}.json")
    run_ranks(_worker, world, jobs, base_dir, save, out_path, timeout=600.0)
    with open(out_path) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def outcomes():
    results = {}
    with tempfile.TemporaryDirectory() as tmp:
        results.update(_visit([("w1", ())], tmp, True))
        results.update(_visit([("w2", ("w1",)), ("w2rep", ("w1", "w2"))], tmp, True))
        results.update(_visit([("w3", ("w1", "w2", "w2rep"))], tmp, True))
        results.update(_visit([("w4hsdp", ("w1", "w2", "w2rep", "w3"))], tmp, True))
        results.update(_visit([("w3", ("w4hsdp",))], tmp, False))
        results.update(_visit([("w2rep", ("w3", "w4hsdp")), ("w2", ("w2rep", "w3", "w4hsdp"))], tmp, False))
        results.update(_visit([("w1", ("w2", "w2rep", "w3", "w4hsdp"))], tmp, False))
    return results


@pytest.mark.parametrize("case", CASES)
def test_checkpoint_crosses_world_sizes(outcomes, case):
    assert case in outcomes, "no stage reached this case"
    assert not outcomes[case], outcomes[case]
