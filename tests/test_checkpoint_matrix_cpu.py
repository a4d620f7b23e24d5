"""Resume equivalence on two gloo ranks, one (optimizer, wrapping, route) per case: train two steps, hand the
state to a differently initialised twin through the route, train both one more step on the same data, compare.

Routes: the on-disk matrix_dcp format (same layout, and re-sharded into another planner's layout), the in-memory
sharded state dict, and the get_/set_state_dict facade in its sharded and its gathered form.  All cases run
inside one spawn; each is reported as its own test.  The reference keeps one test per route in
test/fsdp/test_matrix_fsdp_distributed.py:2998-3121 and test/fsdp/test_checkpoint.py."""
import copy
import itertools
import json
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks

OPTIMIZERS = ("adamw", "sgd", "mixed_muon_adamw")
WRAPS = ("root", "units")
ROUTES = ("dcp", "dcp_reshard", "dcp_full_state", "in_memory", "facade_sharded", "facade_full")
CASES = [f"{o}-{w}-{r}" for o, w, r in itertools.product(OPTIMIZERS, WRAPS, ROUTES)]


def _model(seed):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(6, 10), nn.Tanh()), nn.Sequential(nn.LayerNorm(10), nn.Linear(10, 6)),
                         nn.Linear(6, 4))


def _build(seed, opt_kind, wrap, *, other_layout=False):
    from matrix_fsdp_b200 import configure_optimizer, matrix_fully_shard
    from matrix_fsdp_b200.api import fully_shard, reset_shared_owner_planners
    from matrix_fsdp_b200.planning.planner import parameter_boundary_plan

    reset_shared_owner_planners()
    model = _model(seed)
    targets = ([] if wrap == "root" else list(model.children())[:-1]) + [model]
    for m in targets:
        if opt_kind == "mixed_muon_adamw":
            fully_shard(m, optimizer_policy="mixed_muon_adamw")       # whole matrices on one owner
        elif other_layout:
            matrix_fully_shard(m, group_planner=parameter_boundary_plan)
        else:
            fully_shard(m)                                              # even split
    hyper = {"adamw": dict(lr=1e-2, weight_decay=0.01), "sgd": dict(lr=0.05, momentum=0.9),
             "mixed_muon_adamw": dict(lr=0.01)}[opt_kind]
    return model, configure_optimizer(model, opt_kind, **hyper)


def _train(model, opt, seed, steps):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        model(torch.randn(3, 6, generator=g)).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()


def _units(model):
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    return collect_param_groups(model)


def _full(model):
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

    return get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))


def _run_case(rank, world, name, base_dir):
    from matrix_fsdp_b200 import load_matrix_dcp, load_matrix_state_dict, matrix_state_dict, save_matrix_dcp
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_state_dict, set_state_dict

    opt_kind, wrap, route = name.split("-")
    src, src_opt = _build(0, opt_kind, wrap)
    _train(src, src_opt, seed=10 + rank, steps=2)
    reshard = route == "dcp_reshard"
    # the muon layout is already uneven (owners); re-shard it into the even split of plain AdamW-style sharding
    dst, dst_opt = _build(5, opt_kind, wrap, other_layout=reshard)
    if route in ("dcp", "dcp_reshard", "dcp_full_state"):
        directory = os.path.join(base_dir, name)
        if rank == 0:
            os.makedirs(directory, exist_ok=True)
        dist.barrier()
        save_matrix_dcp(src, directory, optimizer=src_opt, full_state=(route == "dcp_full_state"))
        dist.barrier()
        if route == "dcp_full_state":
            # the same files also hold every parameter whole, readable without the model or a process group
            from matrix_fsdp_b200 import load_matrix_dcp_full_state

            whole = load_matrix_dcp_full_state(directory)["params"]
            want = _full(src)
            assert set(whole) == set(want), (sorted(whole), sorted(want))
            for k, v in want.items():
                assert torch.equal(whole[k], v), k
        if reshard and opt_kind != "mixed_muon_adamw":
            with pytest.raises(ValueError):                  # a different layout is refused unless asked for
                load_matrix_dcp(dst, directory, optimizer=dst_opt)
        load_matrix_dcp(dst, directory, optimizer=dst_opt, allow_reshard=reshard)
    elif route == "in_memory":
        load_matrix_state_dict(dst, matrix_state_dict(src))
        for (_, a), (_, b) in zip(_components(src_opt), _components(dst_opt)):
            b.load_state_dict(copy.deepcopy(a.state_dict()))     # state_dict() hands out the live tensors
    else:
        options = MatrixStateDictOptions(full_state_dict=(route == "facade_full"))
        model_sd, optim_sd = get_state_dict(src, src_opt, options=options)
        optim_sd = copy.deepcopy(optim_sd)                   # as a save / load would: no tensor shared with src
        if route == "facade_full":
            assert set(model_sd) == set(_model(0).state_dict())          # plain names, full tensors
        set_state_dict(dst, dst_opt, model_state_dict=model_sd, optim_state_dict=optim_sd, options=options)
    same_layout = not reshard
    if same_layout:
        for a, b in zip(_units(src), _units(dst)):
            assert torch.equal(a.flat_buffer.local_shard, b.flat_buffer.local_shard), a.name
    fa, fb = _full(src), _full(dst)
    for k in fa:
        assert torch.equal(fa[k], fb[k]), k                               # parameters arrive bitwise on every route
    _train(src, src_opt, seed=20 + rank, steps=1)
    _train(dst, dst_opt, seed=20 + rank, steps=1)
    fa, fb = _full(src), _full(dst)
    for k in fa:                                                          # and so did the optimizer state
        if same_layout:
            assert torch.equal(fa[k], fb[k]), k
        else:
            assert torch.allclose(fa[k], fb[k], atol=1e-6), (k, float((fa[k] - fb[k]).abs().max()))


def _components(opt):
    from matrix_fsdp_b200.checkpoint.state_dict import iter_optimizer_components

    return list(iter_optimizer_components(opt))


def _worker(rank, world, out_path, base_dir):
    results = {}
    for name in CASES:
        try:
            _run_case(rank, world, name, base_dir)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        results[name] = "\n".join(f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


@pytest.fixture(scope="module")
def outcomes():
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, 2, path, tmp, timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.mark.parametrize("case", CASES)
def test_two_rank_resume_matches_uninterrupted_training(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]
