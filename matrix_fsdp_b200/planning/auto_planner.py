"""Policy-driven planner selection and the stateful Muon-aware owner planners.

``auto_group_plan`` evaluates a candidate set (whole-param, ordered blocks, matrix row
blocks, matrix-owner variants, hint-driven, expert-owner) under a named weight policy and
returns the cheapest runtime-compatible ``PlannerResult``.

``make_muon_shard_aware_group_planner`` returns a *stateful* planner that remembers the
cumulative per-rank load of the groups it has planned, so successive transformer blocks do
not all put their largest matrices on rank 0.  The scoped and cost-aware variants see all
groups up front.  ``make_model_wide_muon_planner`` (addition) balances by Newton-Schulz
FLOPs across the whole model, which is what bounds the owner's step time on B200.

Parity: ``matrix_fsdp/planning/auto_planner.py:40-1278``.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from dataclasses import dataclass, replace
from math import ceil

from ..core.layout import MatrixGroupLayout
from ..core.managed_param import ManagedParam
from .layout_report import report_group_layout
from .layout_validator import explain_runtime_layout_compatibility
from .planner import (ParamBlock, expert_owner_tail_plan, hint_aware_block_builder, hinted_ordered_group_plan,
                      load_balanced_matrix_owner_tail_group_plans, load_balanced_matrix_owner_tail_plan,
                      ordered_group_plan, ordered_matrix_owner_tail_plan, parameter_boundary_plan,
                      rotate_layout_ranks, whole_param_blocks)
from .planner_eval import (GroupPlanner, PlannerCandidate, PlannerCostWeights, PlannerResourceEstimate, PlannerResult,
                           compare_group_planners, estimate_layout_cost_breakdown, estimate_layout_resources,
                           newton_schulz_flops, planner_result_from_output, select_best_group_planner)

W = PlannerCostWeights


@dataclass(frozen=True)
class AutoPlannerPolicy:
    name: str
    weights: PlannerCostWeights


BALANCED_POLICY = AutoPlannerPolicy("balanced", W(
    runtime_flat_reorder=0.01, split_param_unit=0.001, rank_segment=0.25, max_rank_segment=0.25,
    fragmented_rank_segment=0.5, fragmented_rank_unit=0.001, split_param_segment=0.25, imbalance_unit=0.05,
    memory_imbalance_byte=0.00001, total_comm_byte=0.000001))
MIN_COMM_POLICY = AutoPlannerPolicy("min_comm", W(
    collective=4.0, max_rank_unit=0.1, padding_unit=2.0, split_param=8.0, split_param_unit=0.01, rank_segment=4.0,
    max_rank_segment=2.0, fragmented_rank_segment=8.0, fragmented_rank_unit=0.01, param_segment=1.0,
    split_param_segment=2.0, max_param_segment=1.0, total_comm_unit=0.01, max_rank_comm_unit=0.02))
MAX_BALANCE_POLICY = AutoPlannerPolicy("max_balance", W(
    collective=0.5, max_rank_unit=4.0, padding_unit=0.5, split_param_unit=0.0005, rank_segment=0.1,
    fragmented_rank_segment=0.25, fragmented_rank_unit=0.0005, imbalance_unit=1.0))
MUON_FULL_MATRIX_POLICY = AutoPlannerPolicy("muon_full_matrix", W(
    max_rank_unit=0.5, split_param=100000.0, split_param_unit=10.0, rank_segment=1.0, max_rank_segment=1.0,
    fragmented_rank_segment=2.0, param_segment=10.0, split_param_segment=20.0, max_param_segment=10.0))
ZERO_COPY_FRIENDLY_POLICY = AutoPlannerPolicy("zero_copy_friendly", W(
    runtime_flat_reorder=256.0, split_param_unit=0.001, rank_segment=0.25, max_rank_segment=0.25,
    fragmented_rank_segment=0.5, fragmented_rank_unit=0.001, split_param_segment=0.25, total_comm_unit=0.001,
    max_rank_comm_unit=0.001, imbalance_unit=0.05))
MUON_ZERO_COPY_POLICY = AutoPlannerPolicy("muon_zero_copy", W(
    runtime_flat_reorder=256.0, split_param=100000.0, split_param_unit=10.0, rank_segment=0.5, max_rank_segment=0.5,
    fragmented_rank_segment=1.0, fragmented_rank_unit=0.001, param_segment=10.0, split_param_segment=20.0,
    max_param_segment=10.0, total_comm_unit=0.001, max_rank_comm_unit=0.001, imbalance_unit=0.25,
    parameter_block=0.001, matrix_owner_matrix=0.0001, muon_matrix_owner=0.0001, matrix_owner_tail_param=0.0001,
    adamw_tail_param=0.0001, max_rank_memory_byte=0.00001, memory_imbalance_byte=0.00002,
    max_rank_muon_param_byte=0.00002, muon_param_imbalance_byte=0.00005, total_comm_byte=0.000001,
    max_rank_comm_byte=0.000002))
MUON_SHARD_AWARE_POLICY = AutoPlannerPolicy("muon_shard_aware", W(
    split_param=100000.0, split_param_unit=10.0, rank_segment=1.0, max_rank_segment=1.0,
    fragmented_rank_segment=2.0, fragmented_rank_unit=0.001, param_segment=10.0, split_param_segment=20.0,
    max_param_segment=10.0, imbalance_unit=0.5, parameter_block=0.001, matrix_owner_matrix=0.0001,
    matrix_owner_tail_param=0.0001, adamw_tail_param=0.0001, max_rank_memory_byte=0.00002,
    memory_imbalance_byte=0.00005, max_rank_optimizer_byte=0.00002, optimizer_imbalance_byte=0.00005,
    max_rank_muon_param_byte=0.00005, muon_param_imbalance_byte=0.0001, total_comm_byte=0.000001,
    max_rank_comm_byte=0.000002, comm_imbalance_byte=0.000001, workspace_preferred_unit=0.000001,
    workspace_padding_unit=0.000005, workspace_padding_ratio=10.0))
DEBUG_POLICY = AutoPlannerPolicy("debug", W(
    split_param=1.0, split_param_unit=0.01, rank_segment=1.0, max_rank_segment=1.0, fragmented_rank_segment=1.0,
    fragmented_rank_unit=0.01, param_segment=1.0, split_param_segment=1.0, max_param_segment=1.0,
    total_comm_unit=0.01, max_rank_comm_unit=0.01, imbalance_unit=0.1, block=0.01))

_POLICIES = {p.name: p for p in (BALANCED_POLICY, MIN_COMM_POLICY, MAX_BALANCE_POLICY, MUON_FULL_MATRIX_POLICY,
                                 ZERO_COPY_FRIENDLY_POLICY, MUON_ZERO_COPY_POLICY, MUON_SHARD_AWARE_POLICY,
                                 DEBUG_POLICY)}
_MATRIX_OWNER_POLICIES = {"muon_shard_aware", "muon_zero_copy"}

MuonShardAwareGroupPlanner = Callable[[Sequence[ManagedParam], int], PlannerResult]


def resolve_auto_planner_policy(policy: str | AutoPlannerPolicy) -> AutoPlannerPolicy:
    if isinstance(policy, AutoPlannerPolicy):
        return policy
    if policy not in _POLICIES:
        raise ValueError(f"Unknown auto planner policy={policy!r}. Valid policies: {', '.join(sorted(_POLICIES))}.")
    return _POLICIES[policy]


def available_auto_planner_policies() -> tuple[str, ...]:
    return tuple(sorted(_POLICIES))


# --------------------------------------------------------------------------- candidates
@dataclass(frozen=True)
class AutoGroupPlannerCandidates:
    candidates: tuple[PlannerCandidate, ...]

    @property
    def candidate_by_name(self) -> Mapping[str, PlannerCandidate]:
        return {c.name: c for c in self.candidates}

    @property
    def planners(self) -> Mapping[str, GroupPlanner]:
        return {c.name: c.planner for c in self.candidates}

    @property
    def blocks_by_name(self) -> Mapping[str, tuple[ParamBlock, ...]]:
        return {c.name: c.blocks for c in self.candidates}

    @property
    def padding_units_by_name(self) -> Mapping[str, int]:
        return {c.name: c.padding_units for c in self.candidates}

    @property
    def num_collectives_by_name(self) -> Mapping[str, int]:
        return {c.name: c.num_collectives for c in self.candidates if c.num_collectives is not None}


def _tagged_blocks(params: Sequence[ManagedParam], kind_of: Callable[[ManagedParam], str]) -> tuple[ParamBlock, ...]:
    return tuple(ParamBlock(p.fqn, p.offset, p.end, 0, kind_of(p)) for p in params)


def _matrix_owner_kind(p: ManagedParam) -> str:
    two_d = len(p.shape) == 2
    if two_d:
        return "muon_matrix_owner" if p.shard_hint.optimizer_type == "muon" else "matrix_owner_matrix"
    return "adamw_tail_param" if p.shard_hint.optimizer_type == "adamw" else "matrix_owner_tail_param"


def _expert_owner_kind(p: ManagedParam) -> str:
    h = p.shard_hint
    if h.runtime_kind == "expert_owner" or h.expert_group_id:
        return "expert_owner_param"
    if h.parallel_role == "router":
        return "router_tail_param"
    if len(p.shape) == 2 and h.optimizer_type == "muon":
        return "dense_muon_tail_param"
    return "dense_tail_param"


def _matrix_owner_tail_blocks(params):
    return _tagged_blocks(params, _matrix_owner_kind)


def _has_expert_owner_params(params) -> bool:
    return any(p.shard_hint.runtime_kind == "expert_owner" or p.shard_hint.expert_group_id for p in params)


def _has_explicit_shard_hints(params) -> bool:
    from ..core.managed_param import ParamShardHint
    return any(p.shard_hint != ParamShardHint() for p in params)


def _blocks_for(params, builder) -> tuple[ParamBlock, ...]:
    return tuple(b for p in params for b in builder(p))


def default_auto_group_planner_candidates(params: Sequence[ManagedParam], world_size: int, *,
                                          target_block_units: int | None = None,
                                          include_matrix_owner_tail: bool = False) -> AutoGroupPlannerCandidates:
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}.")
    if _has_expert_owner_params(params):
        return AutoGroupPlannerCandidates((PlannerCandidate("expert_owner_tail", expert_owner_tail_plan,
                                                            _tagged_blocks(params, _expert_owner_kind)),))
    if target_block_units is not None and target_block_units <= 0:
        raise ValueError(f"target_block_units must be positive, got {target_block_units}.")
    total = sum(p.numel for p in params)
    target = target_block_units or (max(1, ceil(total / max(1, world_size * 2))) if total else 1)

    def rows_for(p: ManagedParam) -> int:
        return max(1, target // int(p.shape[1])) if len(p.shape) == 2 else 1

    def builder(default: str, kind: str = "block"):
        return hint_aware_block_builder(default_granularity=default, target_block_units=target,
                                        row_block_units=rows_for, block_kind=kind)

    ordered_b, row_b, hinted_b = builder("block", "ordered_block"), builder("row_block"), builder("parameter")
    cands = [
        PlannerCandidate("whole_param", parameter_boundary_plan, _blocks_for(params, whole_param_blocks)),
        PlannerCandidate("ordered_block", lambda ps, w: ordered_group_plan(ps, w, block_builder=ordered_b),
                         _blocks_for(params, ordered_b)),
        PlannerCandidate("matrix_row_block", lambda ps, w: ordered_group_plan(ps, w, block_builder=row_b),
                         _blocks_for(params, row_b)),
    ]
    if include_matrix_owner_tail and any(len(p.shape) == 2 for p in params):
        mo_blocks = _matrix_owner_tail_blocks(params)
        cands.append(PlannerCandidate("matrix_owner_tail", ordered_matrix_owner_tail_plan, mo_blocks))
        cands.append(PlannerCandidate("matrix_owner_tail_role_greedy", load_balanced_matrix_owner_tail_plan, mo_blocks))
    if _has_explicit_shard_hints(params):
        cands.append(PlannerCandidate(
            "hinted_mixed",
            lambda ps, w: hinted_ordered_group_plan(ps, w, default_granularity="parameter",
                                                    target_block_units=target, row_block_units=rows_for),
            _blocks_for(params, hinted_b)))
    return AutoGroupPlannerCandidates(tuple(cands))


def evaluate_auto_group_planners(params: Sequence[ManagedParam], world_size: int, *, candidates=None,
                                 policy: str | AutoPlannerPolicy = "balanced",
                                 weights: PlannerCostWeights | None = None,
                                 target_block_units: int | None = None) -> tuple[PlannerResult, ...]:
    pol = resolve_auto_planner_policy(policy)
    w = pol.weights if weights is None else weights
    if candidates is None:
        candidates = default_auto_group_planner_candidates(
            params, world_size, target_block_units=target_block_units,
            include_matrix_owner_tail=pol.name in _MATRIX_OWNER_POLICIES).candidates
    return tuple(replace(e, policy=pol.name) for e in compare_group_planners(params, world_size, candidates, weights=w))


def select_auto_group_plan(params: Sequence[ManagedParam], world_size: int, **kwargs) -> PlannerResult:
    evals = evaluate_auto_group_planners(params, world_size, **kwargs)
    if not evals:
        raise ValueError("Expected at least one planner candidate.")
    return evals[0]


def auto_group_plan(params: Sequence[ManagedParam], world_size: int, *, candidates=None,
                    policy: str | AutoPlannerPolicy = "balanced", weights: PlannerCostWeights | None = None,
                    target_block_units: int | None = None) -> PlannerResult:
    return select_auto_group_plan(params, world_size, candidates=candidates, policy=policy, weights=weights,
                                  target_block_units=target_block_units)


# --------------------------------------------------------------------------- stateful Muon planners
def _owner_eval(name: str, layout: MatrixGroupLayout, params, world_size: int, policy) -> PlannerResult:
    pol = resolve_auto_planner_policy(policy)
    return planner_result_from_output(name, layout, params, world_size, blocks=_matrix_owner_tail_blocks(params),
                                      weights=pol.weights, policy=pol.name)


def _role_greedy_eval(params, world_size: int, initial_rank_units, policy, role_weight_fn=None) -> PlannerResult:
    layout = load_balanced_matrix_owner_tail_plan(params, world_size, initial_rank_units=initial_rank_units,
                                                  merge_adjacent_rank_segments=True, role_weight_fn=role_weight_fn)
    return _owner_eval("matrix_owner_tail_role_greedy", layout, params, world_size, policy)


def _rotated_sizes(sizes: Sequence[int], offset: int) -> tuple[int, ...]:
    n = len(sizes)
    return tuple(sizes[(r - offset) % n] for r in range(n)) if n else ()


def _select_rotation_offset(layout: MatrixGroupLayout, cumulative: Sequence[int], *, unit_index: int,
                            rotate_units: bool, rotation_strategy: str) -> int:
    world = layout.world_size
    if not rotate_units or world <= 0:
        return 0
    if rotation_strategy == "round_robin":
        return unit_index % world
    best = None
    for off in range(world):
        nxt = [c + s for c, s in zip(cumulative, _rotated_sizes(layout.shard_sizes, off))]
        avg = sum(nxt) / world
        score = (float(max(nxt) - min(nxt)), float(max(nxt)), sum((u - avg) ** 2 for u in nxt), float(off))
        if best is None or score < best[0]:
            best = (score, off)
    return best[1]


def _rotate_result(result, offset: int, params, world_size: int):
    if isinstance(result, MatrixGroupLayout):
        return rotate_layout_ranks(result, offset)
    layout = rotate_layout_ranks(result.layout, offset)
    report = replace(report_group_layout(layout), num_blocks=result.report.num_blocks,
                     blocks_by_kind=result.report.blocks_by_kind)
    compat = explain_runtime_layout_compatibility(layout, params, world_size)
    res = estimate_layout_resources(layout, params)
    bd = estimate_layout_cost_breakdown(report, weights=result.cost_weights, padding_units=result.padding_units,
                                        num_collectives=result.num_collectives, runtime_compatible=compat.compatible,
                                        runtime_mode=compat.mode, resources=res)
    warnings = result.warnings
    if not compat.compatible and f"runtime unsupported: {compat.reason}" not in warnings:
        warnings = (*warnings, f"runtime unsupported: {compat.reason}")
    return replace(result, layout=layout, report=report, cost=bd.total, cost_breakdown=bd, resource_estimate=res,
                   runtime_compatible=compat.compatible, runtime_mode=compat.mode, runtime_reason=compat.reason,
                   runtime_requires_flat_reorder=compat.requires_flat_reorder,
                   matrix_shard_compatible=compat.matrix_shard_compatible,
                   matrix_shard_reason=compat.matrix_shard_reason, warnings=warnings,
                   total_comm_units=report.total_comm_units, max_rank_comm_units=report.max_rank_comm_units,
                   num_rank_segments=report.num_rank_segments, max_rank_segments=report.max_rank_segments)


def make_muon_shard_aware_group_planner(*, matrix_owner_tail: bool = False, rotate_units: bool = True,
                                        rotation_strategy: str = "greedy_balance", owner_assignment: str = "rotate",
                                        policy: str | AutoPlannerPolicy = "muon_shard_aware",
                                        ) -> MuonShardAwareGroupPlanner:
    """Stateful whole-matrix owner planner; remembers cumulative rank load across calls.

    ``owner_assignment="rotate"`` plans each group on its own and rotates the owner ranks
    (greedy on cumulative balance, or round-robin); ``"role_greedy"`` / ``"cost_aware"`` hand
    each matrix/tail role to the currently lightest rank.
    """
    if rotation_strategy not in ("greedy_balance", "round_robin"):
        raise ValueError(
            f"Unknown rotation_strategy={rotation_strategy!r}. Valid strategies: greedy_balance, round_robin.")
    if owner_assignment not in ("rotate", "role_greedy", "cost_aware"):
        raise ValueError(
            f"Unknown owner_assignment={owner_assignment!r}. Valid assignments: cost_aware, role_greedy, rotate.")
    state = {"index": 0, "units": None}

    def group_planner(params: Sequence[ManagedParam], world_size: int) -> PlannerResult:
        if state["units"] is None or len(state["units"]) != world_size:
            state["units"] = [0] * world_size
        units = state["units"]
        if owner_assignment in ("role_greedy", "cost_aware"):
            result = _role_greedy_eval(params, world_size, units, policy)
        else:
            base = (ordered_matrix_owner_tail_plan(params, world_size) if matrix_owner_tail
                    else auto_group_plan(params, world_size, policy=policy))
            layout = base if isinstance(base, MatrixGroupLayout) else base.layout
            off = _select_rotation_offset(layout, units, unit_index=state["index"], rotate_units=rotate_units,
                                          rotation_strategy=rotation_strategy)
            result = base if off == 0 else _rotate_result(base, off, params, world_size)
        state["index"] += 1
        final_layout = result if isinstance(result, MatrixGroupLayout) else result.layout
        for r, u in enumerate(final_layout.shard_sizes):
            units[r] += u
        return result

    return group_planner


class _PlannedSequence:
    """Serves pre-computed per-group results in call order and checks the order matches."""

    def __init__(self, param_groups, build: Callable[[int], tuple[PlannerResult, ...]], label: str) -> None:
        self._groups, self._build, self._label = param_groups, build, label
        self._planned: dict[int, tuple[PlannerResult, ...]] = {}
        self._next: dict[int, int] = {}

    def __call__(self, params: Sequence[ManagedParam], world_size: int) -> PlannerResult:
        if world_size not in self._planned:
            self._planned[world_size] = self._build(world_size)
            self._next[world_size] = 0
        i = self._next[world_size]
        if i >= len(self._planned[world_size]):
            raise RuntimeError(f"{self._label} planner was called more times than the number of planned groups.")
        if tuple((p.fqn, p.numel) for p in params) != tuple((p.fqn, p.numel) for p in self._groups[i]):
            raise RuntimeError(f"{self._label} planner call order does not match the planned wrap-policy order.")
        self._next[world_size] = i + 1
        return self._planned[world_size][i]


def _scope_plans(param_groups, world_size: int, policy, initial_rank_units, role_weight_fn=None):
    layouts = load_balanced_matrix_owner_tail_group_plans(param_groups, world_size,
                                                          initial_rank_units=initial_rank_units,
                                                          merge_adjacent_rank_segments=True,
                                                          role_weight_fn=role_weight_fn)
    return tuple(_owner_eval("matrix_owner_tail_scope_greedy", lay, ps, world_size, policy)
                 for ps, lay in zip(param_groups, layouts))


def _role_plans(param_groups, world_size: int, policy, initial_rank_units):
    units = [0] * world_size if initial_rank_units is None else list(initial_rank_units)
    if len(units) != world_size:
        raise ValueError(f"initial_rank_units length must match world_size={world_size}, got {len(units)}.")
    out = []
    for ps in param_groups:
        ev = _role_greedy_eval(ps, world_size, units, policy)
        out.append(ev)
        for r, u in enumerate(ev.layout.shard_sizes):
            units[r] += u
    return tuple(out)


def make_scoped_muon_shard_aware_group_planner(param_groups: Sequence[Sequence[ManagedParam]], *,
                                               policy: str | AutoPlannerPolicy = "muon_shard_aware",
                                               initial_rank_units: Sequence[int] | None = None,
                                               ) -> MuonShardAwareGroupPlanner:
    """Look-ahead owner planner: one owner decision over all groups, served group by group."""
    return _PlannedSequence(param_groups, lambda w: _scope_plans(param_groups, w, policy, initial_rank_units),
                            "Scoped Muon shard-aware")


def _owner_plan_stats(plans: Sequence[PlannerResult]) -> dict[str, float]:
    if not plans:
        return dict.fromkeys(("rank_imbalance", "max_rank_units", "total_workspace_numel", "max_workspace_numel",
                              "max_workspace_padding_ratio"), 0.0)
    world = plans[0].world_size
    totals = [0] * world
    ws = []
    pad = 0.0
    for ev in plans:
        for r, u in enumerate(ev.layout.shard_sizes):
            totals[r] += u
        res = ev.resource_estimate or PlannerResourceEstimate.empty(world)
        ws.append(res.workspace_preferred_numel)
        pad = max(pad, res.workspace_padding_waste_ratio)
    return {"rank_imbalance": float(max(totals) - min(totals)), "max_rank_units": float(max(totals)),
            "total_workspace_numel": float(sum(ws)), "max_workspace_numel": float(max(ws)),
            "max_workspace_padding_ratio": float(pad)}


def _select_cost_aware_owner_plans(role_plans, scope_plans, *, max_workspace_ratio: float,
                                   max_workspace_padding_ratio: float):
    rs, ss = _owner_plan_stats(role_plans), _owner_plan_stats(scope_plans)
    better = ss["rank_imbalance"] < rs["rank_imbalance"] or ss["max_rank_units"] < rs["max_rank_units"]
    within = (ss["max_workspace_numel"] <= rs["max_workspace_numel"] * max_workspace_ratio
              and ss["total_workspace_numel"] <= rs["total_workspace_numel"] * max_workspace_ratio
              and ss["max_workspace_padding_ratio"] <= max_workspace_padding_ratio)
    return tuple(scope_plans) if better and within else tuple(role_plans)


def make_cost_aware_muon_shard_aware_group_planner(param_groups: Sequence[Sequence[ManagedParam]], *,
                                                   policy: str | AutoPlannerPolicy = "muon_shard_aware",
                                                   initial_rank_units: Sequence[int] | None = None,
                                                   max_workspace_ratio: float = 1.35,
                                                   max_workspace_padding_ratio: float = 3.0,
                                                   ) -> MuonShardAwareGroupPlanner:
    """Scope-greedy when it improves balance within workspace growth caps, else role-greedy."""
    pol_name = policy.name if isinstance(policy, AutoPlannerPolicy) else policy

    def build(world_size: int):
        chosen = _select_cost_aware_owner_plans(
            _role_plans(param_groups, world_size, policy, initial_rank_units),
            _scope_plans(param_groups, world_size, policy, initial_rank_units),
            max_workspace_ratio=max_workspace_ratio, max_workspace_padding_ratio=max_workspace_padding_ratio)
        tag = {"matrix_owner_tail_scope_greedy": "scope_greedy", "matrix_owner_tail_role_greedy": "role_greedy"}
        return tuple(replace(ev, policy=pol_name,
                             warnings=(*ev.warnings, f"cost_aware_owner_assignment={tag.get(ev.name, ev.name)}"))
                     for ev in chosen)

    return _PlannedSequence(param_groups, build, "Cost-aware Muon shard-aware")


def muon_role_flops(role_params: Sequence[ManagedParam]) -> int:
    """Role weight in Newton-Schulz FLOPs (non-matrix roles count their elements)."""
    total = 0
    for p in role_params:
        if len(p.shape) == 2 and p.shard_hint.optimizer_type in (None, "muon"):
            total += newton_schulz_flops(int(p.shape[0]), int(p.shape[1]))
        else:
            total += p.numel
    return total


def make_model_wide_muon_planner(param_groups: Sequence[Sequence[ManagedParam]], *,
                                 policy: str | AutoPlannerPolicy = "muon_shard_aware",
                                 balance: str = "ns_flops") -> MuonShardAwareGroupPlanner:
    """Owner plan over the whole model balancing Newton-Schulz FLOPs (or elements) per rank."""
    fn = muon_role_flops if balance == "ns_flops" else None
    return _PlannedSequence(param_groups, lambda w: _scope_plans(param_groups, w, policy, None, fn),
                            "Model-wide Muon")


# --------------------------------------------------------------------------- report
@dataclass(frozen=True)
class AutoPlannerReportRow:
    policy: str
    candidate: str
    selected: bool
    cost: float
    rank_units: tuple[int, ...]
    params_by_rank: tuple[tuple[str, ...], ...]
    block_kinds: tuple[tuple[str, int], ...]
    cost_terms: tuple[tuple[str, float], ...]
    num_rank_segments: int
    max_rank_segments: int
    fragmented_rank_segments: int
    fragmented_rank_units: int
    num_split_params: int
    split_param_units: int
    split_param_segments: int
    total_comm_units: int
    max_rank_comm_units: int
    rank_memory_bytes: tuple[int, ...]
    rank_comm_bytes: tuple[int, ...]
    rank_muon_param_bytes: tuple[int, ...]
    rank_adamw_param_bytes: tuple[int, ...]
    rank_optimizer_bytes: tuple[int, ...]
    max_rank_memory_bytes: int
    memory_imbalance_bytes: int
    total_comm_bytes: int
    max_rank_comm_bytes: int
    muon_param_imbalance_bytes: int
    workspace_preferred_numel: int
    workspace_padding_waste_numel: int
    workspace_padding_waste_ratio: float
    estimated_padding_units: int
    estimated_collectives: int
    candidate_padding_units: int
    candidate_collectives: int
    constraint_counts: tuple[tuple[str, int], ...]
    runtime_mode: str
    runtime_compatible: bool
    runtime_requires_flat_reorder: bool
    runtime_reason: str | None
    warnings: tuple[str, ...]
    planner_summary: dict[str, object]
    layout_contract: dict[str, object]
    report: dict[str, object]
    resources: dict[str, object] | None
    expert_owner_groups: tuple[dict[str, object], ...]
    rank_role_units: tuple[dict[str, int], ...]


def _report_row(policy: str, ev: PlannerResult, selected: bool) -> AutoPlannerReportRow:
    rep, res = ev.report, ev.resource_estimate or PlannerResourceEstimate.empty(ev.world_size)
    meta = ev.as_metadata()
    return AutoPlannerReportRow(
        policy=policy, candidate=ev.name, selected=selected, cost=ev.cost, rank_units=rep.rank_units,
        params_by_rank=rep.params_by_rank, block_kinds=tuple(sorted(rep.blocks_by_kind.items())),
        cost_terms=tuple((k, v) for k, v in ev.cost_breakdown.terms.items() if v),
        num_rank_segments=rep.num_rank_segments, max_rank_segments=rep.max_rank_segments,
        fragmented_rank_segments=rep.fragmented_rank_segments, fragmented_rank_units=rep.fragmented_rank_units,
        num_split_params=rep.num_split_params, split_param_units=rep.split_param_units,
        split_param_segments=rep.split_param_segments, total_comm_units=rep.total_comm_units,
        max_rank_comm_units=rep.max_rank_comm_units, rank_memory_bytes=res.rank_memory_bytes,
        rank_comm_bytes=res.rank_comm_bytes, rank_muon_param_bytes=res.rank_muon_param_bytes,
        rank_adamw_param_bytes=res.rank_adamw_param_bytes, rank_optimizer_bytes=res.rank_optimizer_bytes,
        max_rank_memory_bytes=res.max_rank_memory_bytes, memory_imbalance_bytes=res.memory_imbalance_bytes,
        total_comm_bytes=res.total_comm_bytes, max_rank_comm_bytes=res.max_rank_comm_bytes,
        muon_param_imbalance_bytes=res.muon_param_imbalance_bytes,
        workspace_preferred_numel=res.workspace_preferred_numel,
        workspace_padding_waste_numel=res.workspace_padding_waste_numel,
        workspace_padding_waste_ratio=res.workspace_padding_waste_ratio,
        estimated_padding_units=rep.estimated_padding_units, estimated_collectives=rep.estimated_collectives,
        candidate_padding_units=ev.padding_units, candidate_collectives=ev.num_collectives,
        constraint_counts=meta["constraint_counts"], runtime_mode=ev.runtime_mode,
        runtime_compatible=ev.runtime_compatible, runtime_requires_flat_reorder=ev.runtime_requires_flat_reorder,
        runtime_reason=ev.runtime_reason, warnings=ev.warnings, planner_summary=ev.summary(),
        layout_contract=meta["layout_contract"], report=meta["report"], resources=meta["resource_estimate"],
        expert_owner_groups=meta["expert_owner_groups"], rank_role_units=meta["rank_role_units"])


def build_auto_planner_report(params: Sequence[ManagedParam], world_size: int, *,
                              policy: str | AutoPlannerPolicy = "balanced", target_block_units: int | None = None,
                              show_candidates: bool = True) -> tuple[AutoPlannerReportRow, ...]:
    evals = evaluate_auto_group_planners(params, world_size, policy=policy, target_block_units=target_block_units)
    if not evals:
        return ()
    pol = evals[0].policy or (policy.name if isinstance(policy, AutoPlannerPolicy) else policy)
    rows = tuple(_report_row(pol, ev, i == 0) for i, ev in enumerate(evals))
    return rows if show_candidates else rows[:1]


def format_auto_planner_report(rows: Sequence[AutoPlannerReportRow]) -> str:
    """Fixed-width table: one line per candidate, the selected one starred."""
    if not rows:
        return "(no planner candidates)"
    header = ("sel", "policy", "candidate", "cost", "runtime", "rank_units", "segs", "split", "collectives",
              "max_mem_B", "imbalance_B")
    body = []
    for r in rows:
        runtime = r.runtime_mode if r.runtime_compatible else f"unsupported({r.runtime_reason})"
        body.append(("*" if r.selected else "", r.policy, r.candidate, f"{r.cost:.3f}", runtime,
                     "(" + ",".join(map(str, r.rank_units)) + ")", str(r.num_rank_segments),
                     str(r.num_split_params), str(r.candidate_collectives), str(r.max_rank_memory_bytes),
                     str(r.memory_imbalance_bytes)))
    widths = [max(len(h), *(len(b[i]) for b in body)) for i, h in enumerate(header)]
    fmt = lambda vals: "  ".join(v.ljust(w) for v, w in zip(vals, widths)).rstrip()  # noqa: E731
    lines = [fmt(header), fmt(tuple("-" * w for w in widths))] + [fmt(b) for b in body]
    sel = next((r for r in rows if r.selected), rows[0])
    lines.append("")
    lines.append(f"selected={sel.candidate} params_by_rank=" +
                 "; ".join(f"r{i}:[{','.join(names)}]" for i, names in enumerate(sel.params_by_rank)))
    if sel.warnings:
        lines.append("warnings: " + " | ".join(sel.warnings))
    return "\n".join(lines)
