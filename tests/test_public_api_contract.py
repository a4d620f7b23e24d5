"""Exported names that the other test files reach only indirectly, one property per test: aliases, optimizer
preparation helpers, placement / constraint helpers, the expert-owner hint rule, optimizer state-dict patching,
and (on two gloo ranks) the mesh helpers and the DTensor view of a shard."""
import copy

import pytest
import torch
from torch import nn

import matrix_fsdp_b200 as P
from dist_utils import check_case, run_cases
from matrix_fsdp_b200.api import reset_shared_owner_planners


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2, bias=False))


def _sharded(**kw):
    reset_shared_owner_planners()
    m = _model()
    P.fully_shard(m, **kw)
    return m


def _step(model, opt, seed=0):
    model(torch.randn(3, 4, generator=torch.Generator().manual_seed(seed))).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()


# ------------------------------------------------------------------------------------------ names
def test_every_exported_name_resolves():
    missing = [n for n in P.__all__ if not hasattr(P, n)]
    assert not missing, missing


def test_aliases_point_at_the_functions_they_abbreviate():
    assert P.configure_matrix_optimizer is P.configure_optimizer
    assert P.matrix_get_state_dict is P.get_state_dict and P.matrix_set_state_dict is P.set_state_dict
    assert P.FSDPRuntimeState is P.FSDPLifecycleState and P.LayoutPlanner is P.GroupPlanner


# ------------------------------------------------------------------------------------------ optimizers
def test_prepare_matrix_optimizer_finds_the_units_from_the_parameters():
    m, ref = _sharded(), _model()
    opt = P.prepare_matrix_optimizer(torch.optim.Adam(m.parameters(), lr=1e-2), max_unsharded_prefetch_units=0)
    assert isinstance(opt, P.MatrixFSDPOptimizer) and [u.module for u in opt.fsdp_param_groups] == [m]
    assert opt.scheduler.config.max_unsharded_prefetch_units == 0
    ropt = torch.optim.Adam(ref.parameters(), lr=1e-2)
    for i in range(2):
        _step(m, opt, i)
        _step(ref, ropt, i)
    for p, q in zip(m.parameters(), ref.parameters()):
        assert torch.allclose(p, q, atol=1e-6)


def test_prepare_matrix_optimizer_refuses_an_optimizer_without_managed_parameters():
    with pytest.raises(ValueError, match="no FSDP-managed"):
        P.prepare_matrix_optimizer(torch.optim.SGD(_model().parameters(), lr=0.1))


def test_optimizer_config_object_carries_kind_options_and_defaults():
    m = _sharded(optimizer_policy="mixed_muon_adamw")
    cfg = P.MatrixOptimizerConfig("mixed_muon_adamw", {"lr": 0.01, "muon_ns_steps": 3})
    opt = P.configure_optimizer(m, cfg, muon_momentum=0.8)            # keywords add to / override the config
    assert isinstance(opt, P.MixedMuonAdamWOptimizer)
    g = opt.muon.param_groups[0]
    assert g["ns_steps"] == 3 and g["momentum"] == 0.8 and g["lr"] == 0.01


def test_make_mixed_optimizer_classifies_by_hint():
    m = _sharded(optimizer_policy="mixed_muon_adamw")
    opt = P.make_mixed_muon_adamw_optimizer(m, lr=0.01)
    kinds = {g.optimizer_type: set(g.fqns) for g in opt.optimizer_group_summary()}
    assert kinds["muon"] == {"0.weight", "1.weight"} and kinds["adamw"] == {"0.bias"}
    other = P.make_mixed_muon_adamw_optimizer(_sharded(optimizer_policy="mixed_muon_adamw"), lr=0.01,
                                              default_matrix_optimizer="adamw")
    assert isinstance(other, P.MixedMuonAdamWOptimizer)


def test_patched_optimizer_state_dict_round_trips_through_the_facade():
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions

    m = _sharded()
    opt = P.configure_optimizer(m, "adamw", lr=1e-2)
    _step(m, opt)
    P.patch_optimizer_state_dict(m, optimizers=opt, options=MatrixStateDictOptions(full_state_dict=True))
    sd = opt.state_dict()
    assert set(sd["optimizer"]["state"]) == {"0.weight", "0.bias", "1.weight"}       # keyed by name, full tensors
    saved = copy.deepcopy(sd)
    _step(m, opt, 1)
    opt.load_state_dict(saved)
    again = opt.state_dict()
    for name, st in saved["optimizer"]["state"].items():
        assert torch.equal(again["optimizer"]["state"][name]["exp_avg"], st["exp_avg"]), name


def test_clearing_the_global_buffer_pool_drops_cached_buffers():
    from matrix_fsdp_b200.parallel.buffer_pool import global_full_param_buffer_pool

    pool = global_full_param_buffer_pool()
    buf = pool.acquire(32, torch.float32, torch.device("cpu"))
    pool.release(buf)
    assert pool.cached_buffers() > 0
    P.clear_global_full_param_buffer_pool()
    assert pool.cached_buffers() == 0


# ------------------------------------------------------------------------------------------ placement / constraints
def test_matrix_shard_from_layout_needs_rank_ordered_chunks():
    from matrix_fsdp_b200.core.layout import LayoutSegment as S
    from matrix_fsdp_b200.core.layout import MatrixGroupLayout

    ordered = MatrixGroupLayout.from_rank_segments(12, [[S(0, 8, 0)], [S(8, 12, 0)]])
    assert P.is_matrix_shard_compatible_plan(ordered) and P.is_matrix_shard_compatible_plan(ordered.to_shard_plan())
    shard = P.matrix_shard_from_layout(ordered)
    assert tuple(shard.local_units) == (2, 1)                                        # 8 : 4 reduced by their gcd
    meta = P.matrix_shard_metadata(shard)
    assert meta == {"type": "MatrixShard", "dims": (0,), "local_units": (2, 1)} and P.matrix_shard_metadata(None) is None
    swapped = MatrixGroupLayout.from_rank_segments(12, [[S(8, 12, 0)], [S(0, 8, 0)]])
    assert not P.is_matrix_shard_compatible_plan(swapped)
    with pytest.raises(ValueError, match="rank-ordered"):
        P.matrix_shard_from_layout(swapped)


def test_constraints_of_one_parameter_follow_its_hint():
    from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry
    from matrix_fsdp_b200.planning.constraints import ShardConstraint

    m = _model()
    hints = {"0.weight": P.ParamShardHint(split_granularity="matrix_owner", optimizer_type="muon")}
    params = ManagedParamRegistry.from_module(m, shard_hints=hints).params
    pc = P.infer_param_constraints(params[0])
    assert isinstance(pc, P.ParamShardConstraints) and pc.fqn == "0.weight" and pc.optimizer_type == "muon"
    assert ShardConstraint.MUON_MATRIX_OWNER in pc.constraints and ShardConstraint.NO_SPLIT_MATRIX in pc.constraints
    assert P.infer_param_constraints(params[1]).constraints == ()


def test_expert_owner_rule_hints_expert_parameters_only():
    class Expert(nn.Module):
        def __init__(self):
            super().__init__()
            self.up = nn.Linear(4, 8, bias=True)

    class Layer(nn.Module):
        def __init__(self):
            super().__init__()
            self.router = nn.Linear(4, 2, bias=False)
            self.experts = nn.ModuleList([Expert(), Expert()])

    layer = Layer()
    rule = P.moe_expert_owner_rule()
    hits = {}
    for fqn, p in layer.named_parameters():
        owner = layer.get_submodule(fqn.rsplit(".", 1)[0])
        hits[fqn] = rule.apply(fqn, owner, fqn.rsplit(".", 1)[1], p)
    assert hits["router.weight"] is None
    w, b = hits["experts.1.up.weight"], hits["experts.1.up.bias"]
    assert w.runtime_kind == P.ParamRuntimeKind.EXPERT_OWNER and w.expert_id == 1 and w.split_granularity == "matrix_owner"
    assert w.optimizer_type == "muon" and b.optimizer_type == "adamw" and b.split_granularity == "parameter"
    assert w.expert_group_id == b.expert_group_id != hits["experts.0.up.weight"].expert_group_id


# ------------------------------------------------------------------------------------------ two ranks: mesh, DTensor
def _mesh_case(rank, world):
    from torch.distributed.device_mesh import init_device_mesh

    mesh = init_device_mesh("cpu", (1, 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    assert P.mesh_shape(mesh) == (1, 2) and P.mesh_dim_name(mesh, 1) == "dp_shard" and P.mesh_dim_name(mesh, None) is None
    assert P.mesh_coordinate(mesh) == (0, rank)
    meta = P.mesh_metadata(mesh, "dp_shard", "dp_replicate")
    assert isinstance(meta, P.DeviceMeshMetadata)
    assert (meta.ndim, meta.shape, meta.shard_mesh_dim, meta.shard_mesh_dim_name, meta.shard_mesh_size) == \
        (2, (1, 2), 1, "dp_shard", 2)
    assert (meta.replicate_mesh_dim, meta.replicate_mesh_dim_name, meta.replicate_mesh_size) == (0, "dp_replicate", 1)
    assert meta.coordinate == (0, rank) and P.mesh_metadata(None) is None


def _dtensor_case(rank, world):
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.tensor import DTensor
    from torch.distributed.tensor.placement_types import Replicate

    mesh = init_device_mesh("cpu", (1, 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    reset_shared_owner_planners()
    m = nn.Linear(4, 6, bias=False)
    P.fully_shard(m, mesh=mesh, dp_mesh_dims=P.DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    unit = m._matrix_fsdp_param_group
    shard = unit.flat_buffer.matrix_shard
    assert shard is not None and isinstance(shard, P.MatrixShard)
    placements = P.make_matrix_placements(mesh, 1, shard)
    assert isinstance(placements[0], Replicate) and placements[1] is shard
    local = unit.flat_buffer.local_shard
    dt = P.make_matrix_dtensor(local, mesh, 1, shard, (6, 4))
    assert isinstance(dt, DTensor) and tuple(dt.shape) == (6, 4) and dt.placements == placements
    assert dt.to_local().data_ptr() == local.data_ptr()                              # metadata only, no copy


@pytest.fixture(scope="module")
def two_rank_outcomes():
    return run_cases(2, [("mesh", _mesh_case, ()), ("dtensor", _dtensor_case, ())])


def test_mesh_helpers_describe_the_shard_and_replicate_dims(two_rank_outcomes):
    check_case(two_rank_outcomes, "mesh")


def test_a_shard_can_be_viewed_as_a_dtensor_with_a_matrix_shard_placement(two_rank_outcomes):
    check_case(two_rank_outcomes, "dtensor")


# ------------------------------------------------------------------------------------------ training helpers
def _tiny_llama():
    from matrix_fsdp_b200.models.llama import LlamaConfig, LlamaModel, shard_llama

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = LlamaModel(LlamaConfig(vocab_size=32, hidden=16, n_layers=1, n_heads=2, head_dim=8, ffn=24, max_seq_len=8))
    shard_llama(model)
    return model, P.configure_optimizer(model, "adamw", lr=1e-2)


def test_train_step_is_forward_backward_step_and_a_loss_read_back():
    from matrix_fsdp_b200.utils.training import device_train_step, pin, train_step

    tok = torch.randint(0, 32, (2, 7), generator=torch.Generator().manual_seed(1))
    x, y = tok[:, :-1], tok[:, 1:]
    a, aopt = _tiny_llama()
    b, bopt = _tiny_llama()
    c, copt = _tiny_llama()
    assert pin(x) is x or pin(x).is_pinned()                               # nothing to pin without a CUDA device
    loss_a = train_step(a, aopt, x, y, "cpu")
    loss_b = device_train_step(b, bopt, x, y)
    loss_c = c(x, y)
    loss_c.backward()
    copt.step()
    copt.zero_grad()
    assert isinstance(loss_a, float) and loss_a == pytest.approx(float(loss_b)) == pytest.approx(float(loss_c.detach()))
    sa = [u.flat_buffer.local_shard for u in P.collect_param_groups(a)]
    for other in (b, c):
        for s, t in zip(sa, [u.flat_buffer.local_shard for u in P.collect_param_groups(other)]):
            assert torch.equal(s, t)
    assert train_step(a, aopt, x, y, "cpu") < loss_a                       # the step went downhill on the same batch


# ------------------------------------------------------------------------------------------ kernel library status
def test_kernel_library_status_says_why_when_it_is_not_available(monkeypatch):
    from matrix_fsdp_b200.ops import NativeKernelStatus, native_kernel_available, native_kernel_status

    st = native_kernel_status()
    assert isinstance(st, NativeKernelStatus) and st.library.endswith("libmfsdp_kernels.so")
    assert native_kernel_available() == st.available
    if st.available:
        assert st.reason is None and st.missing_entry_points == () and st.entry_points >= 40
    else:
        assert st.reason                                                     # never a bare "no"
    monkeypatch.setenv("MFSDP_DISABLE_NATIVE_KERNELS", "1")
    off = native_kernel_status()
    assert not off.available and off.disabled_by_env and "MFSDP_DISABLE_NATIVE_KERNELS" in off.reason


def test_segment_fusion_helpers_merge_per_rank():
    from matrix_fsdp_b200.core.layout import LayoutSegment as S
    from matrix_fsdp_b200.ops import coalesce_contiguous_segments, coalesce_rank_segments

    assert coalesce_contiguous_segments([S(0, 3, 0), S(3, 5, 3), S(9, 12, 5)]) == (S(0, 5, 0), S(9, 12, 5))
    merged = coalesce_rank_segments([[S(0, 3, 0), S(3, 5, 3)], [], [S(5, 6, 0), S(7, 8, 1)]])
    assert merged == ((S(0, 5, 0),), (), (S(5, 6, 0), S(7, 8, 1)))
