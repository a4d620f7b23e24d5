"""Pure unit tests (no process group, CPU) of the layout model, MatrixShard placement, mesh helpers,
mixed-precision validation, sharded-state metadata, hook helpers and wrap policies."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import (LayoutSegment, MatrixGroupLayout, ShardPlan, coalesce_segments,
                                          contiguous_shard_plan, rank_segments_are_rank_contiguous_chunks,
                                          split_segments_by_params)
from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry
from matrix_fsdp_b200.core.placement import (MatrixShard, explain_matrix_shard_compatibility, is_matrix_shard_placement,
                                             matrix_shard_from_plan, shard_sizes_to_matrix_local_units)


# ------------------------------------------------------------------------------------ layout
def test_layout_segment_arithmetic():
    s = LayoutSegment(4, 10, 2)
    assert s.numel == 6 and s.local_end == 8
    assert s.intersects(9, 12) and not s.intersects(10, 12) and not s.intersects(0, 4)


def test_shard_plan_builds_one_segment_per_rank():
    plan = contiguous_shard_plan(10, (3, 3, 2, 2))
    assert plan.world_size == 4 and plan.shard_offsets == (0, 3, 6, 8)
    assert plan.local_range(2) == (6, 8)
    assert plan.local_segments(3) == (LayoutSegment(8, 10, 0),)
    assert rank_segments_are_rank_contiguous_chunks([plan.local_segments(r) for r in range(4)])


def test_coalesce_merges_adjacent_global_and_local():
    segs = [LayoutSegment(0, 4, 0), LayoutSegment(4, 6, 4), LayoutSegment(8, 9, 6), LayoutSegment(9, 12, 9)]
    out = coalesce_segments(segs)
    assert out == (LayoutSegment(0, 6, 0), LayoutSegment(8, 9, 6), LayoutSegment(9, 12, 9))


def _registry():
    m = nn.Sequential(nn.Linear(4, 3), nn.Linear(3, 2, bias=False))
    return ManagedParamRegistry.from_module(m)


def test_group_layout_owner_queries():
    reg = _registry()                      # 0.weight 12, 0.bias 3, 1.weight 6 -> 21 elements
    assert [p.numel for p in reg.params] == [12, 3, 6] and reg.total_numel == 21
    rank_segments = ((LayoutSegment(0, 12, 0),), (LayoutSegment(12, 21, 0),))
    layout = MatrixGroupLayout.from_rank_segments(21, rank_segments, reg.params)
    assert layout.world_size == 2 and layout.shard_sizes == (12, 9)
    assert layout.owner_ranks("0.weight") == (0,) and layout.owner_ranks("1.weight") == (1,)
    assert layout.params_for_rank(1) == ("0.bias", "1.weight")
    segs = layout.rank_segments_for_param(1, "0.bias")
    assert [(s.rank, s.global_start, s.global_end, s.local_start) for s in segs] == [(1, 12, 15, 0)]
    assert layout.rank_segments_for_param(0, "0.bias") == ()
    plan = layout.to_shard_plan()
    assert isinstance(plan, ShardPlan) and plan.shard_sizes == (12, 9)
    again = MatrixGroupLayout.from_shard_plan(plan, reg.params)
    assert again.rank_segments == layout.rank_segments


def test_split_segments_by_params_cuts_at_parameter_boundaries():
    reg = _registry()
    pieces = split_segments_by_params(0, [LayoutSegment(10, 16, 0)], reg.params)
    assert [(p.fqn, p.global_start, p.global_end, p.local_start) for p in pieces] == [
        ("0.weight", 10, 12, 0), ("0.bias", 12, 15, 2), ("1.weight", 15, 16, 5)]


def test_registry_rejects_tied_parameters_and_skips_ignored():
    a, b = nn.Linear(3, 3, bias=False), nn.Linear(3, 3, bias=False)
    b.weight = a.weight
    with pytest.raises(NotImplementedError, match="shared parameters"):
        ManagedParamRegistry.from_module(nn.Sequential(a, b))
    m = nn.Sequential(nn.Linear(2, 2), nn.Linear(2, 2))
    reg = ManagedParamRegistry.from_module(m, ignored_params={m[1].weight, m[1].bias})
    assert [p.fqn for p in reg.params] == ["0.weight", "0.bias"]


# ------------------------------------------------------------------------------------ placement
def test_matrix_shard_units_are_gcd_reduced():
    assert shard_sizes_to_matrix_local_units((6, 9, 3)) == (2, 3, 1)
    ms = matrix_shard_from_plan(contiguous_shard_plan(18, (6, 9, 3)))
    assert ms.local_units == (2, 3, 1) and ms.world_size == 3 and ms.total_units == 6
    assert ms.shard_lengths(18) == (6, 9, 3) and ms.shard_range(1, 18) == (6, 15)
    t = torch.arange(18.0)
    parts = ms.split_tensor(t)
    assert [p.numel() for p in parts] == [6, 9, 3] and torch.equal(ms.local_shard(t, 2), t[15:])
    assert is_matrix_shard_placement(ms) and not is_matrix_shard_placement(object())


def test_matrix_shard_compatibility_needs_rank_ordered_single_segments():
    ok = explain_matrix_shard_compatibility(contiguous_shard_plan(10, (4, 6)))
    assert ok.compatible
    swapped = ShardPlan(10, (4, 6), (0, 4), ((LayoutSegment(6, 10, 0),), (LayoutSegment(0, 6, 0),)))
    bad = explain_matrix_shard_compatibility(swapped)
    assert not bad.compatible and bad.reason
    multi = ShardPlan(10, (4, 6), (0, 4), ((LayoutSegment(0, 2, 0), LayoutSegment(8, 10, 2)), (LayoutSegment(2, 8, 0),)))
    assert not explain_matrix_shard_compatibility(multi).compatible


# ------------------------------------------------------------------------------------ mesh
class _FakeMesh:
    def __init__(self, shape, names):
        self.shape, self.mesh_dim_names, self.ndim = shape, names, len(shape)
        self.device_type = "cpu"
        self.mesh = torch.zeros(shape)

    def get_coordinate(self):
        return [0] * self.ndim


def test_mesh_dim_inference():
    from matrix_fsdp_b200.core.mesh import (DataParallelMeshDims, infer_replicate_mesh_dim, infer_shard_mesh_dim,
                                            normalize_mesh_dim)

    one_d = _FakeMesh((4,), ("dp_shard",))
    assert infer_shard_mesh_dim(one_d) == 0 and infer_replicate_mesh_dim(one_d, 0) is None
    two_d = _FakeMesh((2, 4), ("dp_replicate", "dp_shard"))
    assert infer_shard_mesh_dim(two_d) == 1 and infer_replicate_mesh_dim(two_d, 1) == 0
    unnamed = _FakeMesh((2, 4), None)
    assert infer_shard_mesh_dim(unnamed) == 1
    three_d = _FakeMesh((2, 2, 2), ("dp_replicate", "dp_shard", "tp"))
    assert infer_shard_mesh_dim(three_d) == 1 and infer_replicate_mesh_dim(three_d, 1) == 0
    assert normalize_mesh_dim(two_d, "dp_shard") == 1 and normalize_mesh_dim(two_d, -1) == 1
    with pytest.raises((ValueError, KeyError)):
        normalize_mesh_dim(two_d, "nope")
    dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    assert dims.shard == "dp_shard" and dims.replicate == "dp_replicate"


# ------------------------------------------------------------------------------------ mixed precision / offload
def test_mixed_precision_and_offload_validation():
    from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy, OffloadPolicy

    from matrix_fsdp_b200.core.mixed_precision import (cast_floating_tensors, mixed_precision_policy_metadata,
                                                       validate_mixed_precision_policy,
                                                       validate_offload_policy_for_device)

    validate_mixed_precision_policy(MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32))
    meta = mixed_precision_policy_metadata(MixedPrecisionPolicy(param_dtype=torch.bfloat16))
    assert "bfloat16" in str(meta["param_dtype"])
    with pytest.raises((TypeError, ValueError)):
        validate_mixed_precision_policy(MixedPrecisionPolicy(param_dtype=torch.int32))
    validate_offload_policy_for_device(OffloadPolicy(), torch.device("cpu"))
    validate_offload_policy_for_device(CPUOffloadPolicy(), torch.device("cpu"))
    if torch.cuda.is_available():
        with pytest.raises((NotImplementedError, ValueError)):
            validate_offload_policy_for_device(CPUOffloadPolicy(), torch.device("cuda"))
    nested = {"a": torch.ones(2), "b": [torch.ones(2, dtype=torch.int64), (torch.ones(1, dtype=torch.float64),)]}
    out = cast_floating_tensors(nested, torch.bfloat16)
    assert out["a"].dtype == torch.bfloat16 and out["b"][0].dtype == torch.int64 and out["b"][1][0].dtype == torch.bfloat16


# ------------------------------------------------------------------------------------ sharded state
def test_sharded_state_is_metadata_over_a_plain_tensor():
    from matrix_fsdp_b200.core.state import MatrixShardedState, matrix_sharded_state_metadata

    local = torch.arange(6.0)
    ms = MatrixShard((0,), (2, 1))
    st = MatrixShardedState(local, logical_shape=(9,), placement=ms, rank=0, world_size=2)
    assert st.dtensor is None and not st.uses_dtensor
    assert st.local_tensor is local and st.has_same_data_ptr(local) and st.shares_storage_with(local[2:])
    meta = matrix_sharded_state_metadata(st)
    assert tuple(meta["logical_shape"]) == (9,) and meta["rank"] == 0 and meta["world_size"] == 2
    assert tuple(meta["matrix_shard"]["local_units"]) == (2, 1)


# ------------------------------------------------------------------------------------ hooks
def test_pre_backward_context_fires_once_over_nested_outputs():
    from matrix_fsdp_b200.parallel.hooks import ForwardBackwardContext, iter_tensors, register_pre_backward_hooks

    calls = []
    ctx = ForwardBackwardContext(lambda: calls.append(1))
    x = torch.ones(3, requires_grad=True)
    outs = {"a": x * 2, "b": (x * 3, [x * 4, "not a tensor", torch.ones(1)])}
    assert len(list(iter_tensors(outs))) == 4
    n = register_pre_backward_hooks(outs, ctx)
    assert n == 3                                     # the tensor without grad gets no hook
    (outs["a"].sum() + outs["b"][0].sum() + outs["b"][1][0].sum()).backward()
    assert calls == [1]
    ctx.reset()
    y = {"a": x * 5}
    register_pre_backward_hooks(y, ctx)
    y["a"].sum().backward()
    assert calls == [1, 1]


# ------------------------------------------------------------------------------------ wrap policies
def test_wrap_policies_compose():
    from matrix_fsdp_b200.policy.wrap import and_policy, module_type_policy, not_policy, or_policy, size_based_policy

    lin, big, act = nn.Linear(2, 2), nn.Linear(64, 64), nn.ReLU()
    is_lin = module_type_policy(nn.Linear)
    big_enough = size_based_policy(1000)
    assert is_lin(lin) and not is_lin(act)
    assert big_enough(big) and not big_enough(lin)
    assert and_policy(is_lin, big_enough)(big) and not and_policy(is_lin, big_enough)(lin)
    assert or_policy(is_lin, big_enough)(lin) and not or_policy(is_lin, big_enough)(act)
    assert not_policy(is_lin)(act) and not not_policy(is_lin)(lin)
