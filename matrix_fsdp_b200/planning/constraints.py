"""Shard constraints implied by hints (what a planner must not cut).

Parity: ``matrix_fsdp/planning/constraints.py:1-95``.
"""
from __future__ import annotations

from collections import Counter
from collections.abc import Mapping, Sequence
from dataclasses import dataclass
from enum import Enum

from ..core.managed_param import ManagedParam, ParamRuntimeKind


class ShardConstraint(str, Enum):
    NO_SPLIT_PARAM = "no_split_param"
    NO_SPLIT_MATRIX = "no_split_matrix"
    WHOLE_PARAM_OWNER = "whole_param_owner"
    BLOCK_ALIGNED = "block_aligned"
    ROW_BLOCK_ALIGNED = "row_block_aligned"
    MUON_MATRIX_OWNER = "muon_matrix_owner"
    EXPERT_OWNER = "expert_owner"


_BY_GRANULARITY = {
    "parameter": (ShardConstraint.NO_SPLIT_PARAM, ShardConstraint.WHOLE_PARAM_OWNER),
    "matrix_owner": (ShardConstraint.NO_SPLIT_PARAM, ShardConstraint.NO_SPLIT_MATRIX,
                     ShardConstraint.WHOLE_PARAM_OWNER, ShardConstraint.MUON_MATRIX_OWNER),
    "block": (ShardConstraint.BLOCK_ALIGNED,),
    "row_block": (ShardConstraint.ROW_BLOCK_ALIGNED,),
}


@dataclass(frozen=True)
class ParamShardConstraints:
    fqn: str
    constraints: tuple[ShardConstraint, ...]
    block_shape: tuple[int, ...] | None = None
    optimizer_type: str | None = None
    runtime_kind: str | None = None
    parallel_role: str | None = None
    expert_group_id: str | None = None


def infer_param_constraints(param: ManagedParam) -> ParamShardConstraints:
    h = param.shard_hint
    cons = list(_BY_GRANULARITY.get(h.split_granularity, ()))
    if h.runtime_kind == ParamRuntimeKind.EXPERT_OWNER:
        cons.append(ShardConstraint.EXPERT_OWNER)
    return ParamShardConstraints(param.fqn, tuple(cons), h.block_shape, h.optimizer_type, h.runtime_kind,
                                 h.parallel_role, h.expert_group_id)


def infer_group_constraints(params: Sequence[ManagedParam]) -> tuple[ParamShardConstraints, ...]:
    return tuple(infer_param_constraints(p) for p in params)


def constraint_counts(constraints: Sequence[ParamShardConstraints]) -> dict[ShardConstraint, int]:
    return dict(Counter(c for pc in constraints for c in pc.constraints))


def constraints_metadata(constraints: Sequence[ParamShardConstraints]) -> tuple[dict[str, object], ...]:
    return tuple({"fqn": pc.fqn, "constraints": tuple(c.value for c in pc.constraints), "block_shape": pc.block_shape,
                  "optimizer_type": pc.optimizer_type, "runtime_kind": pc.runtime_kind,
                  "parallel_role": pc.parallel_role, "expert_group_id": pc.expert_group_id} for pc in constraints)


def constraint_count_metadata(counts: Mapping[ShardConstraint, int]) -> tuple[tuple[str, int], ...]:
    return tuple((c.value, n) for c, n in sorted(counts.items(), key=lambda kv: kv[0].value))
