"""Planner evaluation, one property per test: what a planner may return, how its answer becomes a
``PlannerResult``, how cost terms add up and react to weights, how candidates are compared, and what the
self-validation of a result catches.  The reference's counterpart is test/fsdp/test_planner_eval.py (23 tests)."""
from dataclasses import fields, replace

import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.core.layout import MatrixGroupLayout, RankLayout, contiguous_shard_plan
from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry
from matrix_fsdp_b200.planning.planner import contiguous_even_plan, ordered_group_plan, parameter_boundary_plan
from matrix_fsdp_b200.planning.planner_eval import (PlannerCandidate, PlannerCostWeights, PlannerLayoutContract,
                                                    PlannerResult, call_group_planner, compare_group_planners,
                                                    estimate_layout_cost, estimate_layout_cost_breakdown,
                                                    estimate_layout_resources, evaluate_group_planner,
                                                    newton_schulz_flops, normalize_planner_candidates,
                                                    planner_display_name, planner_result_from_output,
                                                    select_best_group_planner)
from matrix_fsdp_b200.planning.shard_hint import build_shard_hints


def _params(hinted=False):
    torch.manual_seed(0)
    m = nn.Sequential(nn.Linear(6, 8), nn.LayerNorm(8), nn.Linear(8, 4, bias=False))
    return ManagedParamRegistry.from_module(m, shard_hints=build_shard_hints(m) if hinted else None).params


def _total(params):
    return sum(p.numel for p in params)


def _even(params, world):
    return contiguous_even_plan(_total(params), world)


# ------------------------------------------------------------------------------------------ planner outputs
def test_a_planner_may_return_a_shard_plan_a_layout_or_a_result():
    params = _params()
    plan = _even(params, 2)
    layout = MatrixGroupLayout.from_shard_plan(plan, params)
    result = planner_result_from_output("given", layout, params, 2)
    for output in (plan, layout, result):
        got = planner_result_from_output("x", output, params, 2)
        assert got.layout.shard_sizes == plan.shard_sizes and got.runtime_compatible
    assert planner_result_from_output("x", result, params, 2).name == "given"      # a result keeps its own name


def test_display_name_is_the_function_name_or_the_class_name():
    class Fancy:
        def __call__(self, params, world):
            return _even(params, world)

    assert planner_display_name(parameter_boundary_plan) == "parameter_boundary_plan"
    assert planner_display_name(Fancy()) == "Fancy"
    assert call_group_planner(Fancy(), _params(), 2).name == "Fancy"
    assert evaluate_group_planner("named", _params(), 2, Fancy()).name == "named"


def test_a_result_carries_runtime_classification_and_constraints():
    params = _params(hinted=True)
    r = call_group_planner(parameter_boundary_plan, params, 2)
    assert r.runtime_mode in ("matrix_shard", "segment_runtime") and r.runtime_compatible
    assert len(r.constraints) == len(params) and r.constraints_satisfied
    assert r.num_rank_segments == r.report.num_rank_segments and r.world_size == 2


def test_an_invalid_answer_is_refused_when_it_is_turned_into_a_result():
    params = _params()
    short = contiguous_shard_plan(_total(params) - 1, (10, _total(params) - 11))
    with pytest.raises(ValueError):
        planner_result_from_output("short", short, params, 2)


# ------------------------------------------------------------------------------------------ costs
def test_cost_is_the_sum_of_weight_times_quantity_over_all_terms():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    assert r.cost == pytest.approx(sum(r.cost_breakdown.terms.values())) == pytest.approx(r.cost_breakdown.total)
    assert set(r.cost_breakdown.terms) == {f.name for f in fields(PlannerCostWeights)}


def test_zero_weights_give_zero_cost_and_one_weight_isolates_its_term():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    zero = PlannerCostWeights(**{f.name: 0.0 for f in fields(PlannerCostWeights)})
    assert estimate_layout_cost(r.report, weights=zero) == 0.0
    only = replace(zero, max_rank_unit=2.0)
    assert estimate_layout_cost(r.report, weights=only) == pytest.approx(2.0 * r.report.max_rank_units)


def test_unsupported_runtime_and_reorder_modes_are_cost_terms():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    zero = PlannerCostWeights(**{f.name: 0.0 for f in fields(PlannerCostWeights)})
    w = replace(zero, runtime_unsupported=100.0, runtime_flat_reorder=7.0, runtime_segment_runtime=3.0)
    assert estimate_layout_cost(r.report, weights=w, runtime_compatible=False) == 100.0
    assert estimate_layout_cost(r.report, weights=w, runtime_mode="flat_reorder") == 7.0
    assert estimate_layout_cost(r.report, weights=w, runtime_mode="segment_runtime") == 3.0
    assert estimate_layout_cost(r.report, weights=w, runtime_mode="matrix_shard") == 0.0


def test_padding_and_collective_counts_can_be_given_by_the_caller():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    zero = PlannerCostWeights(**{f.name: 0.0 for f in fields(PlannerCostWeights)})
    w = replace(zero, padding_unit=1.0, collective=10.0)
    base = estimate_layout_cost_breakdown(r.report, weights=w)
    more = estimate_layout_cost_breakdown(r.report, weights=w, padding_units=5, num_collectives=4)
    assert more.terms["padding_unit"] == base.terms["padding_unit"] + 5.0 and more.terms["collective"] == 40.0


def test_resource_terms_enter_the_cost_only_when_resources_are_given():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    zero = PlannerCostWeights(**{f.name: 0.0 for f in fields(PlannerCostWeights)})
    w = replace(zero, max_rank_memory_byte=1.0)
    assert estimate_layout_cost(r.report, weights=w) == 0.0
    res = estimate_layout_resources(r.layout, params)
    assert estimate_layout_cost(r.report, weights=w, resources=res) == pytest.approx(res.max_rank_memory_bytes)


def test_newton_schulz_flops_grow_with_the_small_side_squared():
    assert newton_schulz_flops(8, 8) > 0
    assert newton_schulz_flops(64, 16) == newton_schulz_flops(16, 64)              # the iteration runs on the small side
    assert newton_schulz_flops(32, 32, steps=10) == 2 * newton_schulz_flops(32, 32, steps=5)


def test_resource_estimate_of_an_even_split_is_balanced():
    params = _params()
    res = estimate_layout_resources(MatrixGroupLayout.from_shard_plan(_even(params, 2), params), params)
    assert abs(res.rank_param_bytes[0] - res.rank_param_bytes[1]) <= 4 and res.total_param_bytes == _total(params) * 4
    assert res.max_rank_memory_bytes >= res.rank_param_bytes[0]


# ------------------------------------------------------------------------------------------ candidates
def test_candidates_from_a_mapping_pick_up_their_per_name_settings():
    cands = normalize_planner_candidates({"a": parameter_boundary_plan, "b": ordered_group_plan},
                                         padding_units_by_name={"a": 3}, num_collectives_by_name={"b": 9})
    assert [c.name for c in cands] == ["a", "b"] and cands[0].padding_units == 3 and cands[1].num_collectives == 9
    assert cands[0].num_collectives is None and cands[1].padding_units == 0


def test_ready_made_candidates_pass_through_unchanged():
    c = PlannerCandidate("mine", parameter_boundary_plan, padding_units=2)
    assert normalize_planner_candidates([c]) == (c,)
    assert normalize_planner_candidates({"other": c})[0] is c


def test_comparison_sorts_by_cost_and_puts_unsupported_layouts_last():
    params = _params()
    planners = {"boundary": parameter_boundary_plan, "ordered": ordered_group_plan, "even": lambda ps, w: _even(ps, w)}
    evals = compare_group_planners(params, 2, planners)
    assert [e.cost for e in evals] == sorted(e.cost for e in evals)
    assert {e.name for e in evals} == {"boundary", "ordered", "even"}
    assert select_best_group_planner(params, 2, planners).name == evals[0].name


def test_weights_change_the_winner():
    params = _params()
    planners = {"boundary": parameter_boundary_plan, "even": lambda ps, w: _even(ps, w)}
    zero = PlannerCostWeights(**{f.name: 0.0 for f in fields(PlannerCostWeights)})
    no_splits = select_best_group_planner(params, 2, planners, weights=replace(zero, split_param=1.0))
    balanced = select_best_group_planner(params, 2, planners, weights=replace(zero, imbalance_unit=1.0))
    assert no_splits.name == "boundary" and no_splits.report.num_split_params == 0
    assert balanced.name == "even" and balanced.report.imbalance_units <= 1


def test_selecting_from_nothing_is_an_error():
    with pytest.raises(ValueError, match="at least one"):
        select_best_group_planner(_params(), 2, {})


# ------------------------------------------------------------------------------------------ self-validation
def test_layout_contract_metadata_lists_ranks_params_and_owner_ranks():
    params = _params()
    meta = call_group_planner(parameter_boundary_plan, params, 2).layout_contract().as_metadata()
    assert meta["world_size"] == 2 and sum(meta["shard_sizes"]) == meta["total_numel"] == _total(params)
    assert [p["fqn"] for p in meta["params"]] == [p.fqn for p in params]
    assert all(p["owner_ranks"] for p in meta["params"]) and len(meta["ranks"]) == 2


def test_contract_validation_finds_a_gap_and_a_wrong_local_count():
    params = _params()
    gap = MatrixGroupLayout.from_rank_segments(_total(params), [[S(0, 10, 0)], [S(11, _total(params), 0)]], params)
    with pytest.raises(ValueError):
        PlannerLayoutContract(gap).validate()
    good = MatrixGroupLayout.from_shard_plan(_even(params, 2), params)
    wrong = MatrixGroupLayout(good.total_numel, (RankLayout(0, 1, good.ranks[0].segments), good.ranks[1]), good.params)
    with pytest.raises(ValueError):
        PlannerLayoutContract(wrong).validate()
    PlannerLayoutContract(good).validate()


def test_result_validation_cross_checks_report_and_layout():
    params = _params()
    r = call_group_planner(parameter_boundary_plan, params, 2)
    r.validate()
    other = call_group_planner(lambda ps, w: _even(ps, w), params, 2)
    with pytest.raises(ValueError, match="rank_units"):
        replace(r, report=other.report).validate()


def test_result_metadata_and_summary_are_plain_data():
    import json

    params = _params(hinted=True)
    r = call_group_planner(parameter_boundary_plan, params, 2, policy="balanced")
    meta, summary = r.as_metadata(), r.summary()
    assert meta["planner_name"] == summary["planner_name"] == "parameter_boundary_plan" and meta["policy"] == "balanced"
    assert meta["rank_units"] == r.layout.shard_sizes and dict(meta["cost_terms"]) == dict(r.cost_breakdown.terms)
    assert summary["runtime"]["mode"] == r.runtime_mode and summary["resources"] is not None
    json.dumps(meta, default=str)                                                   # nothing but plain containers
    json.dumps(summary, default=str)
    assert isinstance(r, PlannerResult)
