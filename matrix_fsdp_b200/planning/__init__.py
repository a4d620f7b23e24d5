from .auto_planner import (AutoPlannerPolicy, AutoPlannerReportRow, auto_group_plan, build_auto_planner_report,
                           format_auto_planner_report, make_cost_aware_muon_shard_aware_group_planner,
                           make_model_wide_muon_planner, make_muon_shard_aware_group_planner,
                           make_scoped_muon_shard_aware_group_planner)
from .constraints import ParamShardConstraints, ShardConstraint
from .planner import (contiguous_even_plan, expert_owner_tail_plan, fsdp2_chunk_plan, hinted_ordered_group_plan,
                      load_balanced_matrix_owner_tail_group_plans, load_balanced_matrix_owner_tail_plan,
                      ordered_group_plan, ordered_matrix_owner_tail_plan, parameter_boundary_plan,
                      rotate_layout_ranks)
from .planner_eval import (GroupPlanner, PlannerCandidate, PlannerCostBreakdown, PlannerCostWeights,
                           PlannerLayoutContract, PlannerResourceEstimate, PlannerResult, call_group_planner)
from .shard_hint import build_shard_hints
