"""Planner evaluation: cost model, per-rank resource estimates and the ``PlannerResult`` record.

A ``GroupPlanner`` is any callable ``(params, world_size) -> MatrixGroupLayout | ShardPlan |
PlannerResult``.  :func:`call_group_planner` normalises its output into a ``PlannerResult``
carrying the layout, a structural report, the runtime mode it maps to, a resource estimate
(param / grad / optimizer-state / communication bytes per rank; Muon keeps one state
tensor, AdamW two) and a weighted cost built from a table of named terms.

Parity: ``matrix_fsdp/planning/planner_eval.py:24-1008`` (same weight, term and metadata
names).  Addition: ``rank_ns_flops`` in the resource estimate — Newton-Schulz work per rank —
because on B200 the Muon owner's step time follows NS FLOPs, not element counts.
"""
from __future__ import annotations

from collections.abc import Callable, Mapping, Sequence
from dataclasses import asdict, dataclass, field, fields, replace

import torch

from ..core.layout import LayoutSegment, MatrixGroupLayout, ParamLayout, ParamSegment, ShardPlan
from ..core.managed_param import ManagedParam
from .constraints import (ParamShardConstraints, ShardConstraint, constraint_count_metadata, constraint_counts,
                          constraints_metadata, infer_group_constraints)
from .layout_report import MatrixGroupLayoutReport, report_group_layout
from .layout_validator import explain_runtime_layout_compatibility
from .planner import ParamBlock


@dataclass(frozen=True)
class PlannerCostWeights:
    runtime_unsupported: float = 1_000_000_000_000.0
    runtime_flat_reorder: float = 0.0
    runtime_segment_runtime: float = 0.0
    collective: float = 1.0
    max_rank_unit: float = 1.0
    padding_unit: float = 1.0
    split_param: float = 0.0
    split_param_unit: float = 0.0
    rank_segment: float = 0.0
    max_rank_segment: float = 0.0
    fragmented_rank_segment: float = 0.0
    fragmented_rank_unit: float = 0.0
    param_segment: float = 0.0
    split_param_segment: float = 0.0
    max_param_segment: float = 0.0
    total_comm_unit: float = 0.0
    max_rank_comm_unit: float = 0.0
    imbalance_unit: float = 0.0
    imbalance_ratio: float = 0.0
    block: float = 0.0
    parameter_block: float = 0.0
    ordered_block: float = 0.0
    matrix_row_block: float = 0.0
    quant_block: float = 0.0
    matrix_owner_matrix: float = 0.0
    muon_matrix_owner: float = 0.0
    matrix_owner_tail_param: float = 0.0
    adamw_tail_param: float = 0.0
    max_rank_memory_byte: float = 0.0
    memory_imbalance_byte: float = 0.0
    max_rank_optimizer_byte: float = 0.0
    optimizer_imbalance_byte: float = 0.0
    max_rank_muon_param_byte: float = 0.0
    muon_param_imbalance_byte: float = 0.0
    total_comm_byte: float = 0.0
    max_rank_comm_byte: float = 0.0
    comm_imbalance_byte: float = 0.0
    workspace_preferred_unit: float = 0.0
    workspace_padding_unit: float = 0.0
    workspace_padding_ratio: float = 0.0


@dataclass(frozen=True)
class PlannerResourceEstimate:
    rank_param_bytes: tuple[int, ...]
    rank_grad_bytes: tuple[int, ...]
    rank_optimizer_bytes: tuple[int, ...]
    rank_memory_bytes: tuple[int, ...]
    rank_comm_bytes: tuple[int, ...]
    rank_muon_param_bytes: tuple[int, ...]
    rank_adamw_param_bytes: tuple[int, ...]
    rank_unknown_param_bytes: tuple[int, ...]
    total_param_bytes: int
    total_grad_bytes: int
    total_optimizer_bytes: int
    total_memory_bytes: int
    total_comm_bytes: int
    max_rank_memory_bytes: int
    memory_imbalance_bytes: int
    max_rank_optimizer_bytes: int
    optimizer_imbalance_bytes: int
    max_rank_muon_param_bytes: int
    muon_param_imbalance_bytes: int
    max_rank_comm_bytes: int
    comm_imbalance_bytes: int
    workspace_preferred_numel: int
    workspace_padding_waste_numel: int
    workspace_padding_waste_ratio: float
    rank_ns_flops: tuple[int, ...] = ()

    @classmethod
    def empty(cls, world_size: int = 0) -> "PlannerResourceEstimate":
        z = (0,) * world_size
        return cls(z, z, z, z, z, z, z, z, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0.0, z)

    def as_metadata(self) -> dict[str, object]:
        return asdict(self)


def newton_schulz_flops(rows: int, cols: int, steps: int = 5) -> int:
    """FLOPs of ``steps`` quintic Newton-Schulz iterations on a rows×cols matrix."""
    small, large = min(rows, cols), max(rows, cols)
    per_iter = 2 * small * small * large * 2 + 2 * small * small * small
    return steps * per_iter


def _spread(values: Sequence[int]) -> int:
    return (max(values) - min(values)) if values else 0


def estimate_layout_resources(layout: MatrixGroupLayout, params: Sequence[ManagedParam]) -> PlannerResourceEstimate:
    """Deterministic per-rank memory / traffic model: one gather + one reduce-scatter per step."""
    world = layout.world_size
    if world == 0:
        return PlannerResourceEstimate.empty()
    by_fqn = {p.fqn: p for p in params}
    pbytes, obytes = [0] * world, [0] * world
    muon, adamw, unknown, nsf = [0] * world, [0] * world, [0] * world, [0] * world
    for pl in layout.params:
        mp = by_fqn.get(pl.fqn)
        if mp is None:
            continue
        esize = torch.empty((), dtype=mp.dtype).element_size()
        opt = mp.shard_hint.optimizer_type if mp.shard_hint.optimizer_type in ("muon", "adamw") else None
        mult = {"muon": 1, "adamw": 2}.get(opt, 0)
        for seg in pl.segments:
            b = seg.numel * esize
            pbytes[seg.rank] += b
            obytes[seg.rank] += mult * b
            (muon if opt == "muon" else adamw if opt == "adamw" else unknown)[seg.rank] += b
            if opt == "muon" and len(mp.shape) == 2 and seg.numel == mp.numel:
                nsf[seg.rank] += newton_schulz_flops(int(mp.shape[0]), int(mp.shape[1]))
    total_p = sum(pbytes)
    mem = tuple(2 * p + o for p, o in zip(pbytes, obytes))
    comm = tuple(2 * max(0, total_p - p) for p in pbytes)
    pref = layout.total_numel if world <= 1 else world * max(layout.shard_sizes, default=0)
    waste = max(pref - layout.total_numel, 0)
    return PlannerResourceEstimate(
        rank_param_bytes=tuple(pbytes), rank_grad_bytes=tuple(pbytes), rank_optimizer_bytes=tuple(obytes),
        rank_memory_bytes=mem, rank_comm_bytes=comm, rank_muon_param_bytes=tuple(muon),
        rank_adamw_param_bytes=tuple(adamw), rank_unknown_param_bytes=tuple(unknown),
        total_param_bytes=total_p, total_grad_bytes=total_p, total_optimizer_bytes=sum(obytes),
        total_memory_bytes=sum(mem), total_comm_bytes=sum(comm), max_rank_memory_bytes=max(mem, default=0),
        memory_imbalance_bytes=_spread(mem), max_rank_optimizer_bytes=max(obytes, default=0),
        optimizer_imbalance_bytes=_spread(obytes), max_rank_muon_param_bytes=max(muon, default=0),
        muon_param_imbalance_bytes=_spread(muon), max_rank_comm_bytes=max(comm, default=0),
        comm_imbalance_bytes=_spread(comm), workspace_preferred_numel=pref, workspace_padding_waste_numel=waste,
        workspace_padding_waste_ratio=(waste / layout.total_numel) if layout.total_numel else 0.0,
        rank_ns_flops=tuple(nsf))


@dataclass(frozen=True)
class PlannerCostBreakdown:
    terms: Mapping[str, float]

    @property
    def total(self) -> float:
        return sum(self.terms.values())


# weight name -> how to read its quantity from (report, resources, ctx)
_REPORT_TERMS = {
    "max_rank_unit": "max_rank_units", "split_param": "num_split_params", "split_param_unit": "split_param_units",
    "rank_segment": "num_rank_segments", "max_rank_segment": "max_rank_segments",
    "fragmented_rank_segment": "fragmented_rank_segments", "fragmented_rank_unit": "fragmented_rank_units",
    "param_segment": "num_param_segments", "split_param_segment": "split_param_segments",
    "max_param_segment": "max_param_segments", "total_comm_unit": "total_comm_units",
    "max_rank_comm_unit": "max_rank_comm_units", "imbalance_unit": "imbalance_units",
    "imbalance_ratio": "imbalance_ratio", "block": "num_blocks",
}
_BLOCK_KIND_TERMS = {
    "parameter_block": "parameter", "ordered_block": "ordered_block", "matrix_row_block": "matrix_row_block",
    "quant_block": "quant_block", "matrix_owner_matrix": "matrix_owner_matrix",
    "muon_matrix_owner": "muon_matrix_owner", "matrix_owner_tail_param": "matrix_owner_tail_param",
    "adamw_tail_param": "adamw_tail_param",
}
_RESOURCE_TERMS = {
    "max_rank_memory_byte": "max_rank_memory_bytes", "memory_imbalance_byte": "memory_imbalance_bytes",
    "max_rank_optimizer_byte": "max_rank_optimizer_bytes", "optimizer_imbalance_byte": "optimizer_imbalance_bytes",
    "max_rank_muon_param_byte": "max_rank_muon_param_bytes", "muon_param_imbalance_byte": "muon_param_imbalance_bytes",
    "total_comm_byte": "total_comm_bytes", "max_rank_comm_byte": "max_rank_comm_bytes",
    "comm_imbalance_byte": "comm_imbalance_bytes", "workspace_preferred_unit": "workspace_preferred_numel",
    "workspace_padding_unit": "workspace_padding_waste_numel", "workspace_padding_ratio": "workspace_padding_waste_ratio",
}


def estimate_layout_cost_breakdown(report: MatrixGroupLayoutReport, *, weights: PlannerCostWeights = PlannerCostWeights(),
                                   padding_units: int = 0, num_collectives: int | None = None,
                                   runtime_compatible: bool = True, runtime_mode: str | None = None,
                                   resources: PlannerResourceEstimate | None = None) -> PlannerCostBreakdown:
    res = resources or PlannerResourceEstimate.empty(report.world_size)
    quantities: dict[str, float] = {
        "runtime_unsupported": 0 if runtime_compatible else 1,
        "runtime_flat_reorder": 1 if runtime_mode == "flat_reorder" else 0,
        "runtime_segment_runtime": 1 if runtime_mode == "segment_runtime" else 0,
        "collective": report.estimated_collectives if num_collectives is None else num_collectives,
        "padding_unit": padding_units + report.estimated_padding_units,
    }
    quantities.update({k: getattr(report, a) for k, a in _REPORT_TERMS.items()})
    quantities.update({k: report.blocks_by_kind.get(kind, 0) for k, kind in _BLOCK_KIND_TERMS.items()})
    quantities.update({k: getattr(res, a) for k, a in _RESOURCE_TERMS.items()})
    terms = {f.name: getattr(weights, f.name) * quantities[f.name] for f in fields(weights)}
    return PlannerCostBreakdown(terms)


def estimate_layout_cost(report: MatrixGroupLayoutReport, **kwargs) -> float:
    return estimate_layout_cost_breakdown(report, **kwargs).total


def _seg_meta(seg: LayoutSegment) -> dict[str, int]:
    return {"global_start": seg.global_start, "global_end": seg.global_end, "local_start": seg.local_start,
            "local_end": seg.local_end, "numel": seg.numel}


def _pseg_meta(seg: ParamSegment) -> dict[str, object]:
    return {"fqn": seg.fqn, "rank": seg.rank, **_seg_meta(seg.to_layout_segment())}


@dataclass(frozen=True)
class PlannerLayoutContract:
    """The part of a planner's answer the runtime depends on, with self-validation."""

    layout: MatrixGroupLayout

    total_numel = property(lambda self: self.layout.total_numel)
    world_size = property(lambda self: self.layout.world_size)
    shard_sizes = property(lambda self: self.layout.shard_sizes)
    rank_segments = property(lambda self: self.layout.rank_segments)
    params = property(lambda self: self.layout.params)

    def to_shard_plan(self) -> ShardPlan:
        return self.layout.to_shard_plan()

    def params_for_rank(self, rank: int) -> tuple[str, ...]:
        return self.layout.params_for_rank(rank)

    def owner_ranks(self, fqn: str) -> tuple[int, ...]:
        return self.layout.owner_ranks(fqn)

    def rank_segments_for_param(self, rank: int, fqn: str) -> tuple[ParamSegment, ...]:
        return self.layout.rank_segments_for_param(rank, fqn)

    def as_metadata(self) -> dict[str, object]:
        lay = self.layout
        return {
            "total_numel": lay.total_numel, "world_size": lay.world_size, "shard_sizes": lay.shard_sizes,
            "ranks": tuple({"rank": r.rank, "local_units": r.local_units,
                            "segments": tuple(_seg_meta(s) for s in r.segments)} for r in lay.ranks),
            "params": tuple({"fqn": p.fqn, "global_start": p.global_start, "global_end": p.global_end,
                             "numel": p.numel, "owner_ranks": tuple(sorted({s.rank for s in p.segments})),
                             "segments": tuple(_pseg_meta(s) for s in p.segments)} for p in lay.params),
        }

    def validate(self) -> None:
        lay = self.layout
        if sum(lay.shard_sizes) != lay.total_numel:
            raise ValueError(f"Layout shard sizes sum to {sum(lay.shard_sizes)}, expected {lay.total_numel}.")
        covered = sorted((s.global_start, s.global_end) for r in lay.ranks for s in r.segments if s.numel)
        cur = 0
        for start, end in covered:
            if start != cur:
                raise ValueError(f"Layout rank segments overlap or leave a gap at offset {min(cur, start)}.")
            cur = end
        if cur != lay.total_numel:
            raise ValueError(f"Layout rank segments cover {cur} elements, expected {lay.total_numel}.")
        for r in lay.ranks:
            if sum(s.numel for s in r.segments) != r.local_units:
                raise ValueError(f"Rank {r.rank} local_units={r.local_units} does not match its segments.")
        for p in lay.params:
            if sum(s.numel for s in p.segments) != p.numel:
                raise ValueError(f"Param {p.fqn} segments cover {sum(s.numel for s in p.segments)} of {p.numel}.")


def _expert_owner_groups_metadata(constraints, layout: MatrixGroupLayout) -> tuple[dict[str, object], ...]:
    groups: dict[str, dict] = {}
    by_fqn = {p.fqn: p for p in layout.params}
    for pc in constraints:
        if ShardConstraint.EXPERT_OWNER not in pc.constraints:
            continue
        gid = pc.expert_group_id or pc.fqn
        g = groups.setdefault(gid, {"expert_group_id": gid, "expert_id": _expert_id(gid), "owner_ranks": set(),
                                    "param_fqns": [], "units": 0})
        pl = by_fqn.get(pc.fqn)
        if pl is not None:
            g["owner_ranks"].update(s.rank for s in pl.segments)
            g["units"] += pl.numel
        g["param_fqns"].append(pc.fqn)
    return tuple({**g, "owner_ranks": tuple(sorted(g["owner_ranks"])), "param_fqns": tuple(g["param_fqns"])}
                 for g in groups.values())


def _expert_id(group_id: str) -> int | None:
    tail = group_id.rsplit(".", 1)[-1]
    return int(tail) if tail.isdigit() else None


def _role_of(pc: ParamShardConstraints | None) -> str:
    if pc is None:
        return "unknown"
    if ShardConstraint.EXPERT_OWNER in pc.constraints:
        return "routed_expert"
    if pc.parallel_role:
        return pc.parallel_role
    if ShardConstraint.MUON_MATRIX_OWNER in pc.constraints:
        return "muon_matrix"
    return pc.optimizer_type or "unknown"


def _rank_role_units_metadata(constraints, layout: MatrixGroupLayout) -> tuple[dict[str, int], ...]:
    by = {pc.fqn: pc for pc in constraints}
    out: list[dict[str, int]] = [dict() for _ in range(layout.world_size)]
    for p in layout.params:
        role = _role_of(by.get(p.fqn))
        for s in p.segments:
            out[s.rank][role] = out[s.rank].get(role, 0) + s.numel
    return tuple(out)


@dataclass(frozen=True)
class PlannerResult:
    name: str
    layout: MatrixGroupLayout
    report: MatrixGroupLayoutReport
    cost: float
    constraints_satisfied: bool = True
    constraints: tuple[ParamShardConstraints, ...] = ()
    warnings: tuple[str, ...] = ()
    runtime_compatible: bool = True
    runtime_mode: str = "unknown"
    runtime_reason: str | None = None
    runtime_requires_flat_reorder: bool = False
    matrix_shard_compatible: bool = False
    matrix_shard_reason: str | None = None
    shard_mesh_dim: int | str | None = None
    padding_units: int = 0
    num_collectives: int = 0
    total_comm_units: int = 0
    max_rank_comm_units: int = 0
    resource_estimate: PlannerResourceEstimate | None = None
    num_rank_segments: int = 0
    max_rank_segments: int = 0
    policy: str | None = None
    cost_weights: PlannerCostWeights = PlannerCostWeights()
    cost_breakdown: PlannerCostBreakdown = field(default_factory=lambda: PlannerCostBreakdown({}))

    @property
    def planner_name(self) -> str:
        return self.name

    @property
    def world_size(self) -> int:
        return self.layout.world_size

    def layout_contract(self) -> PlannerLayoutContract:
        return PlannerLayoutContract(self.layout)

    def validate(self) -> None:
        self.layout_contract().validate()
        for what, got, want in (("total_numel", self.report.total_numel, self.layout.total_numel),
                                ("world_size", self.report.world_size, self.layout.world_size),
                                ("rank_units", self.report.rank_units, self.layout.shard_sizes)):
            if got != want:
                raise ValueError(f"Planner report {what}={got} does not match layout {want}.")
        if self.resource_estimate is not None and len(self.resource_estimate.rank_memory_bytes) != self.world_size:
            raise ValueError(
                f"Planner resource estimate has {len(self.resource_estimate.rank_memory_bytes)} ranks, "
                f"expected {self.world_size}.")

    def _runtime_meta(self) -> dict[str, object]:
        return {"compatible": self.runtime_compatible, "mode": self.runtime_mode, "reason": self.runtime_reason,
                "requires_flat_reorder": self.runtime_requires_flat_reorder,
                "matrix_shard_compatible": self.matrix_shard_compatible,
                "matrix_shard_reason": self.matrix_shard_reason}

    def summary(self) -> dict[str, object]:
        return {
            "planner_name": self.name, "policy": self.policy, "cost": self.cost, "world_size": self.world_size,
            "constraints_satisfied": self.constraints_satisfied, "runtime": self._runtime_meta(),
            "layout": self.layout_contract().as_metadata(), "report": self.report.as_metadata(),
            "resources": self.resource_estimate.as_metadata() if self.resource_estimate else None,
            "expert_owner_groups": _expert_owner_groups_metadata(self.constraints, self.layout),
            "rank_role_units": _rank_role_units_metadata(self.constraints, self.layout),
            "cost_terms": tuple(self.cost_breakdown.terms.items()), "warnings": self.warnings,
        }

    def as_metadata(self) -> dict[str, object]:
        rt = self._runtime_meta()
        return {
            "planner_name": self.name, "policy": self.policy, "cost": self.cost,
            "constraints_satisfied": self.constraints_satisfied,
            "constraints": constraints_metadata(self.constraints),
            "constraint_counts": constraint_count_metadata(constraint_counts(self.constraints)),
            "warnings": self.warnings, "runtime_compatible": rt["compatible"], "runtime_mode": rt["mode"],
            "runtime_reason": rt["reason"], "runtime_requires_flat_reorder": rt["requires_flat_reorder"],
            "matrix_shard_compatible": rt["matrix_shard_compatible"], "matrix_shard_reason": rt["matrix_shard_reason"],
            "world_size": self.world_size, "shard_mesh_dim": self.shard_mesh_dim,
            "rank_units": self.layout.shard_sizes, "layout_contract": self.layout_contract().as_metadata(),
            "report": self.report.as_metadata(), "cost_terms": tuple(self.cost_breakdown.terms.items()),
            "resource_estimate": self.resource_estimate.as_metadata() if self.resource_estimate else None,
            "expert_owner_groups": _expert_owner_groups_metadata(self.constraints, self.layout),
            "rank_role_units": _rank_role_units_metadata(self.constraints, self.layout),
        }


PlannerEvaluation = PlannerResult
PlannerOutput = MatrixGroupLayout | ShardPlan | PlannerResult
GroupPlanner = Callable[[Sequence[ManagedParam], int], PlannerOutput]


def planner_display_name(planner: object) -> str:
    return getattr(planner, "__name__", planner.__class__.__name__)


def _with_runtime_warning(compat, warnings: tuple[str, ...]) -> tuple[str, ...]:
    if compat.compatible:
        return warnings
    msg = f"runtime unsupported: {compat.reason}"
    return warnings if msg in warnings else (*warnings, msg)


def planner_result_from_output(name: str, output: PlannerOutput, params: Sequence[ManagedParam], world_size: int, *,
                               blocks: Sequence[ParamBlock] = (), weights: PlannerCostWeights = PlannerCostWeights(),
                               padding_units: int = 0, num_collectives: int | None = None,
                               padding_alignment: int | None = None, collectives_per_segmented_exchange: int = 2,
                               policy: str | None = None, shard_mesh_dim: int | str | None = None) -> PlannerResult:
    prior = output if isinstance(output, PlannerResult) else None
    if prior is not None:
        layout = prior.layout
    elif isinstance(output, ShardPlan):
        layout = MatrixGroupLayout.from_shard_plan(output, params)
    else:
        layout = output
    compat = explain_runtime_layout_compatibility(layout, params, world_size)
    resources = estimate_layout_resources(layout, params)
    if prior is not None:
        report, w, pad, ncoll = prior.report, prior.cost_weights, prior.padding_units, prior.num_collectives
    else:
        report = report_group_layout(layout, blocks, padding_alignment=padding_alignment,
                                     collectives_per_segmented_exchange=collectives_per_segmented_exchange)
        w, pad, ncoll = weights, padding_units, num_collectives
    breakdown = estimate_layout_cost_breakdown(report, weights=w, padding_units=pad, num_collectives=ncoll,
                                               runtime_compatible=compat.compatible, runtime_mode=compat.mode,
                                               resources=resources)
    common = dict(
        cost=breakdown.total, cost_breakdown=breakdown, resource_estimate=resources,
        runtime_compatible=compat.compatible, runtime_mode=compat.mode, runtime_reason=compat.reason,
        runtime_requires_flat_reorder=compat.requires_flat_reorder,
        matrix_shard_compatible=compat.matrix_shard_compatible, matrix_shard_reason=compat.matrix_shard_reason)
    if prior is not None:
        extra = {}
        if shard_mesh_dim is not None and prior.shard_mesh_dim is None:
            extra["shard_mesh_dim"] = shard_mesh_dim
        if not prior.constraints:
            extra["constraints"] = infer_group_constraints(params)
        return replace(prior, warnings=_with_runtime_warning(compat, prior.warnings), **common, **extra)
    return PlannerResult(
        name=name, layout=layout, report=report, shard_mesh_dim=shard_mesh_dim,
        constraints=infer_group_constraints(params), warnings=_with_runtime_warning(compat, ()),
        padding_units=padding_units,
        num_collectives=report.estimated_collectives if num_collectives is None else num_collectives,
        total_comm_units=report.total_comm_units, max_rank_comm_units=report.max_rank_comm_units,
        num_rank_segments=report.num_rank_segments, max_rank_segments=report.max_rank_segments, policy=policy,
        cost_weights=weights, **common)


def call_group_planner(planner: GroupPlanner, params: Sequence[ManagedParam], world_size: int, *,
                       name: str | None = None, **kwargs) -> PlannerResult:
    return planner_result_from_output(name or planner_display_name(planner), planner(params, world_size), params,
                                      world_size, **kwargs)


def evaluate_group_planner(name: str, params: Sequence[ManagedParam], world_size: int, planner: GroupPlanner,
                           **kwargs) -> PlannerResult:
    return call_group_planner(planner, params, world_size, name=name, **kwargs)


@dataclass(frozen=True)
class PlannerCandidate:
    name: str
    planner: GroupPlanner
    blocks: tuple[ParamBlock, ...] = ()
    padding_units: int = 0
    num_collectives: int | None = None
    padding_alignment: int | None = None
    collectives_per_segmented_exchange: int = 2

    def evaluate(self, params: Sequence[ManagedParam], world_size: int, *,
                 weights: PlannerCostWeights = PlannerCostWeights(), policy: str | None = None,
                 shard_mesh_dim: int | str | None = None) -> PlannerResult:
        return call_group_planner(
            self.planner, params, world_size, name=self.name, blocks=self.blocks, weights=weights,
            padding_units=self.padding_units, num_collectives=self.num_collectives,
            padding_alignment=self.padding_alignment,
            collectives_per_segmented_exchange=self.collectives_per_segmented_exchange, policy=policy,
            shard_mesh_dim=shard_mesh_dim)


def normalize_planner_candidates(planners, *, blocks_by_name=None, padding_units_by_name=None,
                                 num_collectives_by_name=None, padding_alignment_by_name=None,
                                 collectives_per_segmented_exchange_by_name=None) -> tuple[PlannerCandidate, ...]:
    if not isinstance(planners, Mapping):
        return tuple(planners)
    out = []
    for name, item in planners.items():
        if isinstance(item, PlannerCandidate):
            out.append(item)
            continue
        out.append(PlannerCandidate(
            name=name, planner=item, blocks=tuple((blocks_by_name or {}).get(name, ())),
            padding_units=(padding_units_by_name or {}).get(name, 0),
            num_collectives=(num_collectives_by_name or {}).get(name),
            padding_alignment=(padding_alignment_by_name or {}).get(name),
            collectives_per_segmented_exchange=(collectives_per_segmented_exchange_by_name or {}).get(name, 2)))
    return tuple(out)


def compare_group_planners(params: Sequence[ManagedParam], world_size: int, planners, *,
                           weights: PlannerCostWeights = PlannerCostWeights(), **by_name) -> tuple[PlannerResult, ...]:
    cands = normalize_planner_candidates(planners, **by_name)
    evals = [c.evaluate(params, world_size, weights=weights) for c in cands]
    return tuple(sorted(evals, key=lambda e: (not e.runtime_compatible, e.cost, e.name)))


def select_best_group_planner(params: Sequence[ManagedParam], world_size: int, planners, **kwargs) -> PlannerResult:
    evals = compare_group_planners(params, world_size, planners, **kwargs)
    if not evals:
        raise ValueError("Expected at least one planner candidate.")
    return evals[0]
