"""matrix_fsdp_b200: a Blackwell-native FSDP2-style parameter-sharding runtime.

Public surface (same names as ``matrix_fsdp/__init__.py:186-323`` of the reference, so user code
switches by changing the import): ``fully_shard`` / ``matrix_fully_shard``,
``DataParallelMeshDims``, planners and layout types, ``configure_optimizer`` and the optimizer
wrappers, ``save_matrix_dcp`` / ``load_matrix_dcp`` and the state-dict facade, summaries and wrap
policies.  Flat module aliases (``matrix_fsdp_b200.planner``, ``.layout``, …) mirror the
reference's legacy aliases (``__init__.py:148-184``).
"""
from __future__ import annotations

import importlib
import sys

from .api import LayoutPlanner, WrapPolicy, fully_shard, matrix_fully_shard, reset_shared_owner_planners
from .checkpoint import (get_model_state_dict, get_optimizer_state_dict, get_state_dict, load_matrix_dcp,
                         load_matrix_dcp_full_state, load_matrix_state_dict, matrix_get_state_dict,
                         matrix_set_state_dict, matrix_state_dict, patch_model_state_dict,
                         patch_optimizer_state_dict, save_matrix_dcp, set_model_state_dict,
                         set_optimizer_state_dict, set_state_dict)
from .core.layout import (LayoutSegment, MatrixGroupLayout, ParamLayout, ParamSegment, RankLayout, ShardPlan,
                          rank_segments_are_rank_contiguous_chunks)
from .core.managed_param import ManagedParam, ManagedParamRegistry, ParamRuntimeKind, ParamShardHint
from .core.mesh import (DataParallelMeshDims, DeviceMeshMetadata, infer_replicate_mesh_dim, infer_shard_mesh_dim,
                        mesh_coordinate, mesh_dim_name, mesh_dim_names, mesh_metadata, mesh_shape, normalize_mesh_dim)
from .core.placement import (MatrixShard, MatrixShardPlacement, PlacementCompatibility,
                             explain_matrix_shard_compatibility, is_matrix_shard_compatible_plan,
                             is_matrix_shard_placement, matrix_shard_from_layout, matrix_shard_from_plan,
                             shard_sizes_to_matrix_local_units)
from .core.state import MatrixShardedState, matrix_shard_metadata, matrix_sharded_state_metadata
from .core.torch_dtensor import make_matrix_dtensor, make_matrix_placements
from .optim import (ClassifiedMatrixOptimizerParams, DEFAULT_MUON_ADJUST_LR_FN, FlatShardedAdamW, FlatShardedSGD,
                    LocalOptimizerParamInfo, LocalOptimizerStateTensor, MatrixFSDPOptimizer,
                    MatrixFSDPOptimizerStateManager, MatrixMuon, MatrixOptimizerConfig,
                    MatrixOptimizerParamGroupSummary, MixedMuonAdamWOptimizer, OptimizerStateSummary,
                    PreparedMatrixOptimizer, classify_matrix_optimizer_params, configure_matrix_optimizer,
                    configure_optimizer, install_matrix_optimizer_auto_prepare, make_mixed_muon_adamw_optimizer,
                    prepare_matrix_optimizer)
from .parallel.buffer_pool import FullParamBufferPool, clear_global_full_param_buffer_pool
from .parallel.fsdp_unit import FSDPLifecycleState, FSDPRuntimeState, MatrixFSDPNoSync, MatrixFSDPParamGroup
from .parallel.param_buffers import (ElasticCommunicationPlan, ElasticParamBuffer, ElasticParamBufferLayout,
                                     ElasticParamBufferWorkspace, ElasticParamBufferWorkspaceLease,
                                     ElasticParamBufferWorkspacePlan, ElasticRankChunk, StaticParamBuffer,
                                     StaticParamBufferLayout, StaticParamBufferWorkspacePlan)
from .parallel.runtime_event import (CommBufferId, PlannerGroupId, RuntimeEvent, RuntimeParamGroupId, RuntimeUnitId,
                                     RuntimeUnitMetadata)
from .parallel.scheduler import (BackwardPrefetchTiming, MatrixFSDPScheduler, MatrixFSDPSchedulerConfig,
                                 PrefetchPolicy, PrefetchProfileResult)
from .parallel.summary import (format_param_group_summary, format_runtime_events, summarize_param_groups,
                               summarize_runtime_events, summarize_scheduler)
from .parallel.unit_collection import collect_param_groups
from .parallel.workspace_cache import CommWorkspaceCache, CommWorkspaceLease
from .planning.auto_planner import (AutoPlannerReportRow, auto_group_plan, build_auto_planner_report,
                                    format_auto_planner_report, make_cost_aware_muon_shard_aware_group_planner,
                                    make_model_wide_muon_planner, make_muon_shard_aware_group_planner,
                                    make_scoped_muon_shard_aware_group_planner)
from .planning.constraints import (ParamShardConstraints, ShardConstraint, constraint_counts, infer_group_constraints,
                                   infer_param_constraints)
from .planning.layout_validator import (RuntimeLayoutCompatibility, explain_runtime_layout_compatibility,
                                        validate_runtime_layout)
from .planning.planner import (expert_owner_tail_plan, fsdp2_chunk_plan, hinted_ordered_group_plan,
                               load_balanced_matrix_owner_tail_group_plans, load_balanced_matrix_owner_tail_plan,
                               ordered_matrix_owner_tail_plan)
from .planning.planner_eval import (GroupPlanner, PlannerCandidate, PlannerCostBreakdown, PlannerCostWeights,
                                    PlannerLayoutContract, PlannerResourceEstimate, PlannerResult, call_group_planner,
                                    estimate_layout_resources, normalize_planner_candidates, planner_display_name,
                                    planner_result_from_output)
from .planning.shard_hint import build_shard_hints, moe_expert_owner_rule
from .policy.wrap import and_policy, module_type_policy, not_policy, or_policy, size_based_policy

__version__ = "0.1.0"

_MODULE_ALIASES = {
    "auto_planner": "planning.auto_planner", "buffer_pool": "parallel.buffer_pool", "collectives": "parallel.collectives",
    "constraints": "planning.constraints", "elastic_param_buffer": "parallel.param_buffers",
    "flat_buffer": "parallel.flat_buffer", "fsdp_unit": "parallel.fsdp_unit", "param_group": "parallel.param_group",
    "grad_bucket": "parallel.grad_bucket", "hooks": "parallel.hooks", "kernels": "ops", "layout": "core.layout",
    "layout_report": "planning.layout_report", "layout_validator": "planning.layout_validator",
    "managed_param": "core.managed_param", "mesh": "core.mesh", "mixed_precision": "core.mixed_precision",
    "optim_state": "optim.state", "placement": "core.placement", "planner": "planning.planner",
    "planner_eval": "planning.planner_eval", "runtime_event": "parallel.runtime_event",
    "scheduler": "parallel.scheduler", "shard_hint": "planning.shard_hint", "state": "core.state",
    "static_param_buffer": "parallel.param_buffers", "summary": "parallel.summary",
    "torch_dtensor": "core.torch_dtensor", "unit_collection": "parallel.unit_collection", "wrap": "policy.wrap",
    "workspace_cache": "parallel.workspace_cache", "runtime": "parallel",
}
for _alias, _target in _MODULE_ALIASES.items():
    sys.modules.setdefault(f"{__name__}.{_alias}", importlib.import_module(f".{_target}", __name__))

__all__ = sorted(n for n in dir() if not n.startswith("_") and n not in ("importlib", "sys", "annotations"))
