"""Invariants every planner and every auto-planner policy must keep, checked over policies x world sizes x
parameter sets: the layout covers the flat space exactly once, validates, respects whole-matrix hints, is
deterministic, and its report / resource estimate are consistent with it.  (The golden vectors of individual
planners live in test_planner.py; the reference's counterparts are test/fsdp/test_auto_planner.py,
test_planner_eval.py and test_layout_validator.py.)"""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry
from matrix_fsdp_b200.planning.auto_planner import (auto_group_plan, available_auto_planner_policies,
                                                    build_auto_planner_report, evaluate_auto_group_planners,
                                                    make_muon_shard_aware_group_planner)
from matrix_fsdp_b200.planning.layout_validator import explain_runtime_layout_compatibility, validate_group_layout
from matrix_fsdp_b200.planning.planner import (contiguous_even_plan, fsdp2_chunk_plan, ordered_group_plan,
                                               ordered_matrix_owner_tail_plan, parameter_boundary_plan)
from matrix_fsdp_b200.planning.planner_eval import call_group_planner, estimate_layout_resources
from matrix_fsdp_b200.planning.shard_hint import build_shard_hints

POLICIES = available_auto_planner_policies()
WORLDS = (1, 2, 3, 8)


class _Block(nn.Module):
    def __init__(self, d=16, f=40):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.q, self.k, self.v, self.o = (nn.Linear(d, d, bias=False) for _ in range(4))
        self.up, self.down = nn.Linear(d, f, bias=False), nn.Linear(f, d, bias=False)


def _params(kind: str, hinted: bool):
    torch.manual_seed(0)
    module = {"block": _Block(), "mlp": nn.Sequential(nn.Linear(8, 16), nn.Linear(16, 4, bias=False)),
              "odd": nn.Sequential(nn.Linear(7, 5), nn.LayerNorm(5), nn.Linear(5, 3))}[kind]
    hints = build_shard_hints(module) if hinted else None
    return ManagedParamRegistry.from_module(module, shard_hints=hints).params


def _layout_of(result):
    return result.layout if hasattr(result, "layout") else result


def _covers_exactly_once(layout, total: int) -> None:
    seen = sorted((s.global_start, s.global_end) for segs in layout.rank_segments for s in segs if s.numel)
    pos = 0
    for a, b in seen:
        assert a == pos, (a, pos)
        pos = b
    assert pos == total


@pytest.mark.parametrize("world", WORLDS)
@pytest.mark.parametrize("policy", POLICIES)
def test_every_policy_yields_a_valid_layout(policy, world):
    params = _params("block", hinted=True)
    total = sum(p.numel for p in params)
    result = call_group_planner(lambda ps, w: auto_group_plan(ps, w, policy=policy), params, world)
    layout = result.layout
    validate_group_layout(layout, params, world)
    _covers_exactly_once(layout, total)
    assert sum(layout.shard_sizes) == total and len(layout.shard_sizes) == world
    compat = explain_runtime_layout_compatibility(layout, params, world)
    assert compat.compatible and compat.mode in ("matrix_shard", "segment_runtime", "flat_reorder")
    assert result.policy == policy and result.runtime_mode == compat.mode


@pytest.mark.parametrize("world", (2, 8))
@pytest.mark.parametrize("policy", ("muon_shard_aware", "muon_full_matrix", "muon_zero_copy"))
def test_muon_policies_keep_hinted_matrices_whole(policy, world):
    params = _params("block", hinted=True)
    layout = auto_group_plan(params, world, policy=policy)
    layout = _layout_of(layout)
    for p in params:
        if p.shape and len(p.shape) == 2:
            owners = {r for r, segs in enumerate(layout.rank_segments)
                      for s in segs if s.numel and s.global_start < p.end and s.global_end > p.offset}
            assert len(owners) == 1, (policy, p.fqn, owners)


@pytest.mark.parametrize("policy", POLICIES)
def test_policies_are_deterministic(policy):
    a = _layout_of(auto_group_plan(_params("block", True), 4, policy=policy))
    b = _layout_of(auto_group_plan(_params("block", True), 4, policy=policy))
    assert a.shard_sizes == b.shard_sizes
    assert [[(s.global_start, s.global_end, s.local_start) for s in segs] for segs in a.rank_segments] == \
           [[(s.global_start, s.global_end, s.local_start) for s in segs] for segs in b.rank_segments]


@pytest.mark.parametrize("kind", ("mlp", "odd", "block"))
@pytest.mark.parametrize("world", WORLDS)
def test_basic_planners_cover_and_validate(kind, world):
    params = _params(kind, hinted=False)
    total = sum(p.numel for p in params)
    sizes = contiguous_even_plan(total, world).shard_sizes
    assert sum(sizes) == total and len(sizes) == world
    if all(p.numel % world == 0 for p in params):
        chunked = fsdp2_chunk_plan(params, world)
        validate_group_layout(chunked, params, world)
        assert len(set(chunked.shard_sizes)) == 1 and sum(chunked.shard_sizes) == total
    else:                                                     # per-parameter chunks need every numel to divide
        with pytest.raises(ValueError, match="divisible"):
            fsdp2_chunk_plan(params, world)
    for group_planner in (parameter_boundary_plan, ordered_group_plan, ordered_matrix_owner_tail_plan):
        layout = _layout_of(call_group_planner(group_planner, params, world).layout)
        validate_group_layout(layout, params, world)
        _covers_exactly_once(layout, total)


@pytest.mark.parametrize("world", (2, 4, 8))
def test_even_plan_is_balanced_to_one_element(world):
    params = _params("block", hinted=False)
    total = sum(p.numel for p in params)
    sizes = contiguous_even_plan(total, world).shard_sizes
    assert max(sizes) - min(sizes) <= max(1, total % world) and sum(sizes) == total


@pytest.mark.parametrize("policy", POLICIES)
def test_candidate_report_marks_exactly_one_selection_with_the_lowest_cost(policy):
    params = _params("block", hinted=True)
    rows = build_auto_planner_report(params, 4, policy=policy)
    assert rows and sum(r.selected for r in rows) == 1 and rows[0].selected
    assert rows[0].cost == min(r.cost for r in rows if r.runtime_compatible)
    for r in rows:
        assert sum(r.rank_units) == sum(p.numel for p in params) and len(r.rank_units) == 4
        assert len(r.rank_memory_bytes) == 4 and all(b >= 0 for b in r.rank_memory_bytes)


@pytest.mark.parametrize("world", (2, 4))
def test_resource_estimate_adds_up(world):
    params = _params("block", hinted=True)
    layout = _layout_of(auto_group_plan(params, world, policy="muon_shard_aware"))
    est = estimate_layout_resources(layout, params)
    assert len(est.rank_param_bytes) == world
    assert sum(est.rank_param_bytes) == est.total_param_bytes > 0
    assert est.max_rank_memory_bytes == max(est.rank_memory_bytes)
    assert est.memory_imbalance_bytes == max(est.rank_memory_bytes) - min(est.rank_memory_bytes)
    assert sum(est.rank_muon_param_bytes) + sum(est.rank_adamw_param_bytes) + sum(est.rank_unknown_param_bytes) \
        == est.total_param_bytes


@pytest.mark.parametrize("assignment", ("rotate", "role_greedy", "cost_aware"))
def test_stateful_owner_planner_spreads_repeated_blocks(assignment):
    planner = make_muon_shard_aware_group_planner(owner_assignment=assignment)
    totals = [0] * 4
    for _ in range(8):
        params = _params("block", hinted=True)
        layout = call_group_planner(planner, params, 4).layout
        validate_group_layout(layout, params, 4)
        for r, n in enumerate(layout.shard_sizes):
            totals[r] += n
    assert max(totals) / (sum(totals) / 4) < 1.2, totals          # cumulative load evens out over the stack


@pytest.mark.parametrize("policy", POLICIES)
def test_evaluation_lists_candidates_sorted_by_cost(policy):
    evals = evaluate_auto_group_planners(_params("block", True), 4, policy=policy)
    assert evals and all(e.policy == policy for e in evals)
    usable = [e.cost for e in evals if e.runtime_compatible]
    assert usable == sorted(usable)


def test_unknown_policy_is_rejected_with_the_list_of_known_ones():
    with pytest.raises(ValueError) as exc:
        auto_group_plan(_params("mlp", False), 2, policy="fastest_please")
    assert "balanced" in str(exc.value)
