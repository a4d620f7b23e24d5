"""Checkpoint contract details: legacy per-rank sidecars, optimizer component checks, HSDP payload keys with
replica de-duplication, expert-owner hints in the metadata, and structural mismatches reported before loading."""
import os
import tempfile

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks
from matrix_fsdp_b200 import configure_optimizer, fully_shard, load_matrix_dcp, save_matrix_dcp
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.checkpoint import read_global_metadata


def _model(seed=0, width=10):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(6, width), nn.LayerNorm(width), nn.Linear(width, 4))


def _step(model, opt, seed=1):
    g = torch.Generator().manual_seed(seed)
    model(torch.randn(3, 6, generator=g)).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()


def test_legacy_per_rank_sidecar_is_accepted_on_load():
    reset_shared_owner_planners()
    model = _model()
    fully_shard(model)
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    _step(model, opt)
    with tempfile.TemporaryDirectory() as d:
        save_matrix_dcp(model, d, optimizer=opt, no_dist=True)
        payload = read_global_metadata(d)
        os.remove(os.path.join(d, "matrix_metadata.pt"))
        torch.save(payload["ranks"][0], os.path.join(d, "matrix_metadata_rank_0.pt"))     # the older layout
        again = read_global_metadata(d)
        assert again["metadata"]["ranks"] == (0,) and again["ranks"][0]["dcp_rank"] == 0
        other = _model(seed=3)
        fully_shard(other)
        opt2 = configure_optimizer(other, "adamw", lr=1e-2)
        load_matrix_dcp(other, d, optimizer=opt2, no_dist=True)
        assert torch.equal(model._matrix_fsdp_param_group.flat_buffer.local_shard,
                           other._matrix_fsdp_param_group.flat_buffer.local_shard)
    with tempfile.TemporaryDirectory() as empty, pytest.raises(FileNotFoundError):
        read_global_metadata(empty)


def test_optimizer_component_and_structure_mismatches_raise():
    reset_shared_owner_planners()
    model = _model()
    fully_shard(model, optimizer_policy="mixed_muon_adamw")
    mixed = configure_optimizer(model, "mixed_muon_adamw", lr=1e-2, muon_lr=1e-2)
    _step(model, mixed)
    with tempfile.TemporaryDirectory() as d:
        save_matrix_dcp(model, d, optimizer=mixed, no_dist=True)
        meta = read_global_metadata(d)["ranks"][0]["optimizer"]
        assert meta["kind"] == "mixed_muon_adamw" and set(meta["components"]) == {"muon", "adamw"}
        # an optimizer with other components cannot take this state
        reset_shared_owner_planners()
        plain = _model(seed=2)
        fully_shard(plain, optimizer_policy="mixed_muon_adamw")
        adamw = configure_optimizer(plain, "adamw", lr=1e-2)
        with pytest.raises(ValueError, match="component"):
            load_matrix_dcp(plain, d, optimizer=adamw, no_dist=True)
        # a model with a different parameter set is refused before any tensor is read
        reset_shared_owner_planners()
        wider = _model(width=12)
        fully_shard(wider, optimizer_policy="mixed_muon_adamw")
        with pytest.raises(ValueError):
            load_matrix_dcp(wider, d, no_dist=True)
    with tempfile.TemporaryDirectory() as d:
        save_matrix_dcp(model, d, no_dist=True)                       # no optimizer saved
        with pytest.raises(ValueError, match="no optimizer state"):
            load_matrix_dcp(model, d, optimizer=mixed, no_dist=True)


def test_expert_owner_hints_survive_in_metadata():
    class Moe(nn.Module):
        def __init__(self):
            super().__init__()
            self.router = nn.Linear(4, 2, bias=False)
            self.experts = nn.ModuleList([nn.Sequential(nn.Linear(4, 8, bias=False), nn.Linear(8, 4, bias=False))
                                          for _ in range(2)])

        def forward(self, x):
            w = torch.softmax(self.router(x), -1)
            return sum(w[:, i:i + 1] * e(x) for i, e in enumerate(self.experts))

    reset_shared_owner_planners()
    torch.manual_seed(0)
    m = Moe()
    fully_shard(m, optimizer_policy="mixed_muon_adamw")
    with tempfile.TemporaryDirectory() as d:
        save_matrix_dcp(m, d, no_dist=True)
        unit = read_global_metadata(d)["ranks"][0]["units"][0]
        hint = unit["params"]["experts.1.0.weight"]["shard_hint"]
        assert hint["runtime_kind"] == "expert_owner" and hint["expert_id"] == 1
        assert unit["params"]["router.weight"]["shard_hint"]["parallel_role"] == "router"


def _hsdp_worker(rank, world, directory):
    from torch.distributed.device_mesh import init_device_mesh

    from matrix_fsdp_b200 import DataParallelMeshDims

    reset_shared_owner_planners()
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    model = _model()
    fully_shard(model, mesh=mesh, dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    _step(model, opt, seed=rank)
    unit = model._matrix_fsdp_param_group
    assert unit.rank == rank % 2 and unit.world_size == 2 and unit.replicate_world_size == 2
    save_matrix_dcp(model, directory, optimizer=opt)
    payload = read_global_metadata(directory)
    assert payload["metadata"]["ranks"] == (0, 1, 2, 3)
    mine = payload["ranks"][rank]
    assert mine["dcp_rank"] == rank
    u0 = mine["units"][0]
    assert u0["dcp_payload_rank"] == f"shard_{rank % 2}" and u0["dcp_dedup_replicates"] is True
    before = unit.flat_buffer.local_shard.clone()
    _step(model, opt, seed=10 + rank)
    load_matrix_dcp(model, directory, optimizer=opt)
    assert torch.equal(unit.flat_buffer.local_shard, before)
    dist.barrier()


def test_hsdp_payload_keys_are_shared_by_replicas():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_hsdp_worker, 4, d)
        files = os.listdir(d)
        assert "matrix_metadata.pt" in files and not [f for f in files if f.startswith("matrix_metadata_rank_")]


# ----------------------------------------------------------------------------- mixed precision through every route
def _bf16_pair(seed, kind, policy):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    reset_shared_owner_planners()
    torch.manual_seed(seed)
    m = nn.Sequential(nn.Linear(4, 6), nn.Tanh(), nn.Linear(6, 4))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16)
    fully_shard(m[0], optimizer_policy=policy, mp_policy=mp)
    fully_shard(m, optimizer_policy=policy, mp_policy=mp)
    return m, configure_optimizer(m, kind, lr=1e-2)


def _bf16_step(m, o, seed):
    x = torch.randn(3, 4, generator=torch.Generator().manual_seed(seed))
    y = m(x.bfloat16())
    y.float().pow(2).mean().backward()
    o.step()
    o.zero_grad()
    return y.detach().float()


@pytest.mark.parametrize("kind,policy", [("adamw", None), ("sgd", None), ("mixed_muon_adamw", "mixed_muon_adamw")])
@pytest.mark.parametrize("route", ["dcp", "in_memory", "facade_sharded", "facade_full"])
def test_bf16_compute_with_fp32_masters_resumes_exactly_through_every_route(route, kind, policy):
    """The masters travel, never their bf16 copies: a twin with a history of its own continues bit for bit, and
    the first forward after the load already runs on the loaded weights."""
    import copy as _copy
    import tempfile as _tempfile

    from matrix_fsdp_b200 import load_matrix_state_dict, matrix_state_dict
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_state_dict, set_state_dict
    from matrix_fsdp_b200.checkpoint.state_dict import iter_optimizer_components

    src, so = _bf16_pair(0, kind, policy)
    _bf16_step(src, so, 1)
    _bf16_step(src, so, 2)
    dst, do = _bf16_pair(7, kind, policy)
    _bf16_step(dst, do, 5)
    if route == "dcp":
        with _tempfile.TemporaryDirectory() as d:
            save_matrix_dcp(src, d, optimizer=so, no_dist=True)
            load_matrix_dcp(dst, d, optimizer=do, no_dist=True)
    elif route == "in_memory":
        load_matrix_state_dict(dst, matrix_state_dict(src))
        for (_, a), (_, b) in zip(iter_optimizer_components(so), iter_optimizer_components(do)):
            b.load_state_dict(_copy.deepcopy(a.state_dict()))
    else:
        options = MatrixStateDictOptions(full_state_dict=(route == "facade_full"))
        model_sd, optim_sd = get_state_dict(src, so, options=options)
        if route == "facade_full":
            assert all(v.dtype == torch.float32 for v in model_sd.values())          # masters, not the compute copy
        set_state_dict(dst, do, model_state_dict=model_sd, optim_state_dict=_copy.deepcopy(optim_sd), options=options)
    for seed in (3, 4):
        assert torch.equal(_bf16_step(src, so, seed), _bf16_step(dst, do, seed)), (route, kind, seed)


def test_full_state_files_of_a_bf16_model_hold_the_fp32_masters():
    from matrix_fsdp_b200 import load_matrix_dcp_full_state
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

    model, opt = _bf16_pair(0, "adamw", None)
    _bf16_step(model, opt, 1)
    with tempfile.TemporaryDirectory() as d:
        save_matrix_dcp(model, d, optimizer=opt, full_state=True, no_dist=True)
        whole = load_matrix_dcp_full_state(d)["params"]
    want = get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    masters = torch.cat([u.flat_buffer.local_shard for u in (model[0]._matrix_fsdp_param_group, model._matrix_fsdp_param_group)])
    assert set(whole) == set(want)
    for k, v in want.items():
        assert whole[k].dtype == torch.float32 and torch.equal(whole[k], v), k
    assert torch.equal(torch.cat([want["0.weight"].flatten(), want["0.bias"].flatten(), want["2.weight"].flatten(),
                                  want["2.bias"].flatten()]), masters)


def test_gathered_state_dict_loading_is_strict_about_names_and_shapes():
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions as O
    from matrix_fsdp_b200.checkpoint import get_model_state_dict, set_model_state_dict

    def build(seed):
        reset_shared_owner_planners()
        torch.manual_seed(seed)
        m = nn.Sequential(nn.Linear(4, 6), nn.BatchNorm1d(6), nn.Linear(6, 4))
        fully_shard(m[0])
        fully_shard(m)
        return m

    full = get_model_state_dict(build(0), options=O(full_state_dict=True))
    assert "1.running_mean" in full and "1.num_batches_tracked" in full                 # buffers travel too
    with pytest.raises(KeyError, match="unexpected"):
        set_model_state_dict(build(1), dict(full, **{"extra.weight": torch.zeros(2)}), options=O(full_state_dict=True))
    set_model_state_dict(build(1), dict(full, **{"extra.weight": torch.zeros(2)}), options=O(full_state_dict=True, strict=False))
    with pytest.raises(KeyError, match="missing key '2.weight'"):
        set_model_state_dict(build(1), {k: v for k, v in full.items() if not k.startswith("2.")}, options=O(full_state_dict=True))
    with pytest.raises(RuntimeError, match=r"size mismatch for 0.weight.*\(3, 3\).*\(6, 4\)"):
        set_model_state_dict(build(1), dict(full, **{"0.weight": torch.zeros(3, 3)}), options=O(full_state_dict=True))
    target = build(1)
    before = target._matrix_fsdp_param_group.flat_buffer.local_shard.clone()
    with pytest.raises(KeyError):                                                        # refused before anything is written
        set_model_state_dict(target, dict(full, **{"extra.weight": torch.zeros(2)}), options=O(full_state_dict=True))
    assert torch.equal(target._matrix_fsdp_param_group.flat_buffer.local_shard, before)
    loaded = build(1)
    set_model_state_dict(loaded, {k: v.double() for k, v in full.items()}, options=O(full_state_dict=True))
    again = get_model_state_dict(loaded, options=O(full_state_dict=True))
    assert all(torch.equal(again[k], full[k]) for k in full) and again["0.weight"].dtype == torch.float32
