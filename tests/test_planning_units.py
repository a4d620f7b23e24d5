"""Unit tests of planner evaluation, layout validation / reporting, constraints and shard-hint rules."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.core.layout import MatrixGroupLayout
from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry, ParamShardHint
from matrix_fsdp_b200.planning.layout_report import report_group_layout
from matrix_fsdp_b200.planning.layout_validator import (explain_runtime_layout_compatibility, flat_reorder_order,
                                                        validate_group_layout)
from matrix_fsdp_b200.planning.planner import contiguous_even_plan, parameter_boundary_plan
from matrix_fsdp_b200.planning.planner_eval import (PlannerCostWeights, call_group_planner, compare_group_planners,
                                                    estimate_layout_resources, newton_schulz_flops,
                                                    select_best_group_planner)
from matrix_fsdp_b200.planning.shard_hint import build_shard_hints


def _mlp():
    return nn.Sequential(nn.Linear(8, 16), nn.Linear(16, 4, bias=False))


def _params(module=None, hints=None):
    return ManagedParamRegistry.from_module(module or _mlp(), shard_hints=hints).params


def _layout(total, rank_segments, params):
    return MatrixGroupLayout.from_rank_segments(total, rank_segments, params)


# ------------------------------------------------------------------------------------ validator
def test_validator_catches_gaps_overlaps_and_wrong_totals():
    params = _params()                                  # 128 + 16 + 64 = 208
    total = sum(p.numel for p in params)
    good = _layout(total, ((S(0, 100, 0),), (S(100, total, 0),)), params)
    validate_group_layout(good, params, 2)
    with pytest.raises(ValueError):
        validate_group_layout(_layout(total, ((S(0, 100, 0),), (S(110, total, 0),)), params), params, 2)    # gap
    with pytest.raises(ValueError):
        validate_group_layout(_layout(total, ((S(0, 120, 0),), (S(100, total, 0),)), params), params, 2)    # overlap
    with pytest.raises(ValueError):
        validate_group_layout(good, params, 3)                                                              # world size


def test_runtime_mode_classification():
    params = _params()
    total = sum(p.numel for p in params)
    even = _layout(total, ((S(0, 104, 0),), (S(104, total, 0),)), params)
    assert explain_runtime_layout_compatibility(even, params, 2).mode == "matrix_shard"
    # rank 1 owns the first parameter, rank 0 the rest: one segment per rank but not rank ordered
    swapped = _layout(total, ((S(128, total, 0),), (S(0, 128, 0),)), params)
    comp = explain_runtime_layout_compatibility(swapped, params, 2)
    assert comp.compatible and comp.mode in ("segment_runtime", "flat_reorder")
    strict = explain_runtime_layout_compatibility(swapped, params, 2, allow_flat_reorder=False, allow_segment_runtime=False)
    assert not strict.compatible and strict.mode == "unsupported" and strict.reason
    assert flat_reorder_order(swapped)[0] in ("0.bias", "1.weight")      # rank 0's parameters come first


def test_validator_enforces_whole_parameter_hints():
    hints = {"0.weight": ParamShardHint(optimizer_type="muon", split_granularity="matrix_owner")}
    params = _params(hints=hints)
    total = sum(p.numel for p in params)
    split = _layout(total, ((S(0, 64, 0),), (S(64, total, 0),)), params)        # cuts 0.weight in two
    with pytest.raises(ValueError, match="0.weight"):
        validate_group_layout(split, params, 2)
    whole = _layout(total, ((S(0, 128, 0),), (S(128, total, 0),)), params)
    validate_group_layout(whole, params, 2)


# ------------------------------------------------------------------------------------ report
def test_layout_report_metrics():
    params = _params()
    total = sum(p.numel for p in params)
    layout = _layout(total, ((S(0, 128, 0),), (S(128, total, 0),)), params)
    rep = report_group_layout(layout)
    assert rep.world_size == 2 and rep.rank_units == (128, 80) and rep.max_rank_units == 128
    assert rep.imbalance_ratio == pytest.approx(128 / 104)
    assert rep.num_split_params == 0
    even = MatrixGroupLayout.from_shard_plan(contiguous_even_plan(total, 2), params)
    rep2 = report_group_layout(even)
    assert rep2.rank_units == (104, 104) and rep2.num_split_params == 1          # 0.weight is cut at 104
    meta = rep2.as_metadata()
    assert meta["world_size"] == 2 and tuple(meta["rank_units"]) == (104, 104)


# ------------------------------------------------------------------------------------ evaluation
def test_resource_estimate_counts_optimizer_states_by_type():
    hints = {"0.weight": ParamShardHint(optimizer_type="muon", split_granularity="matrix_owner"),
             "0.bias": ParamShardHint(optimizer_type="adamw", split_granularity="parameter"),
             "1.weight": ParamShardHint(optimizer_type="muon", split_granularity="matrix_owner")}
    params = _params(hints=hints)
    total = sum(p.numel for p in params)
    layout = _layout(total, ((S(0, 128, 0),), (S(128, total, 0),)), params)
    est = estimate_layout_resources(layout, params)
    # fp32 parameters; rank 0: 128 Muon elements (1 state); rank 1: 16 AdamW (2 states) + 64 Muon (1 state)
    assert est.rank_param_bytes == (128 * 4, 80 * 4)
    assert est.rank_optimizer_bytes == (128 * 4, (16 * 2 + 64) * 4)
    assert est.rank_muon_param_bytes == (128 * 4, 64 * 4) and est.rank_adamw_param_bytes == (0, 16 * 4)
    assert est.max_rank_optimizer_bytes == 128 * 4 and est.as_metadata()["total_param_bytes"] == 208 * 4
    assert est.rank_ns_flops[0] == newton_schulz_flops(16, 8) and est.rank_ns_flops[1] == newton_schulz_flops(4, 16)
    assert newton_schulz_flops(4, 8, steps=1) > 0 and newton_schulz_flops(8, 4) == newton_schulz_flops(4, 8)


def test_compare_and_select_planners():
    params = _params()
    planners = {"even": lambda ps, w: contiguous_even_plan(sum(p.numel for p in ps), w),
                "whole": lambda ps, w: parameter_boundary_plan(ps, w)}
    results = compare_group_planners(params, 2, planners)
    assert [r.name for r in results] and {r.name for r in results} == {"even", "whole"}
    assert all(r.cost >= 0 for r in results)
    best = select_best_group_planner(params, 2, planners)
    assert best.name in planners
    heavy_balance = PlannerCostWeights(imbalance_unit=1000.0, max_rank_unit=1000.0)
    assert select_best_group_planner(params, 2, planners, weights=heavy_balance).name == "even"
    res = call_group_planner(planners["whole"], params, 2, name="whole")
    res.validate()
    summary = res.summary()
    assert summary["planner_name"] == "whole" and summary["world_size"] == 2
    assert res.layout_contract().shard_sizes == res.layout.shard_sizes


# ------------------------------------------------------------------------------------ hints / constraints
def test_default_hint_rules_priority():
    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.embed = nn.Embedding(10, 4)
            self.norm = nn.LayerNorm(4)
            self.proj = nn.Linear(4, 4)
            self.gate = nn.Linear(4, 2, bias=False)
            self.experts = nn.ModuleList([nn.Linear(4, 4, bias=False) for _ in range(2)])
            self.lm_head = nn.Linear(4, 10, bias=False)

    hints = build_shard_hints(Block())
    assert (hints["proj.weight"].optimizer_type, hints["proj.weight"].split_granularity) == ("muon", "matrix_owner")
    assert (hints["proj.bias"].optimizer_type, hints["proj.bias"].split_granularity) == ("adamw", "parameter")
    assert hints["embed.weight"].optimizer_type == "adamw" and hints["norm.weight"].optimizer_type == "adamw"
    assert hints["gate.weight"].parallel_role == "router"
    assert hints["experts.1.weight"].runtime_kind == "expert_owner" and hints["experts.1.weight"].expert_id == 1
    assert hints["lm_head.weight"].optimizer_type == "adamw"            # vocabulary projection stays with AdamW
    over = build_shard_hints(Block(), overrides={"proj.weight": ParamShardHint(optimizer_type="adamw")})
    assert over["proj.weight"].optimizer_type == "adamw"


def test_constraints_follow_hints():
    from matrix_fsdp_b200.planning.constraints import (ShardConstraint, constraint_counts, constraints_metadata,
                                                       infer_group_constraints)

    m = _mlp()
    params = _params(m, hints=build_shard_hints(m))
    cons = infer_group_constraints(params)
    by = {c.fqn: c for c in cons}
    assert ShardConstraint.NO_SPLIT_MATRIX in by["0.weight"].constraints
    assert ShardConstraint.MUON_MATRIX_OWNER in by["0.weight"].constraints
    assert ShardConstraint.NO_SPLIT_PARAM in by["0.bias"].constraints and by["0.bias"].optimizer_type == "adamw"
    counts = constraint_counts(cons)
    assert sum(counts.values()) >= len(params)
    meta = constraints_metadata(cons)
    assert meta[0]["fqn"] == "0.weight"


def test_invalid_hints_are_rejected():
    with pytest.raises((ValueError, TypeError)):
        ManagedParamRegistry.from_module(_mlp(), shard_hints={"0.weight": ParamShardHint(split_granularity="diagonal")})
    with pytest.raises(ValueError):
        ManagedParamRegistry.from_module(_mlp(), shard_hints={"0.weight": ParamShardHint(split_granularity="row_block",
                                                                                       block_shape=(3, 8))})   # 16 rows % 3
    from matrix_fsdp_b200 import fully_shard

    frozen = _mlp()
    frozen[0].weight.requires_grad_(False)
    with pytest.raises(ValueError, match="require grad"):
        fully_shard(frozen)
    ok = _mlp()
    ok[0].weight.requires_grad_(False)
    fully_shard(ok, ignored_params={ok[0].weight})            # frozen parameters may be ignored
