"""Public entry points: ``fully_shard`` (FSDP2-shaped) and ``matrix_fully_shard`` (all knobs).

``fully_shard(module, *, mesh, reshard_after_forward, shard_placement_fn, mp_policy,
offload_policy, ignored_params, dp_mesh_dims, optimizer_policy)`` returns the same module with
``module._matrix_fsdp_param_group`` and ``module.no_sync()`` attached; parameters stay plain
``nn.Parameter`` objects whose ``.data`` is swapped between shard and full views.

``optimizer_policy`` in {"mixed_muon_adamw", "muon_adamw", "muon_shard_aware", "muon"} selects
whole-matrix owner layouts (role-greedy, remembered across successive calls so that stacked
blocks spread their matrices over ranks); None/"default"/"none"/"adamw"/"sgd" selects the dense
even split.  ``shard_placement_fn`` may only return ``Shard(0)`` (row sharding).

Parity: ``matrix_fsdp/api.py:34-623``.  Difference from the reference: the stateful owner
planner is shared by successive ``fully_shard`` calls with the same mesh (the reference builds a
fresh one per call, so every block assigns its largest matrix to rank 0,
``api.py:101-120,456-464``).
"""
from __future__ import annotations

import weakref
from collections.abc import Callable, Mapping
from functools import partial

from torch import nn
from torch.distributed.fsdp import MixedPrecisionPolicy, OffloadPolicy
from torch.distributed.tensor.placement_types import Shard

from .core.managed_param import ManagedParamRegistry, ParamShardHint
from .core.mesh import DataParallelMeshDims, MeshDim
from .core.mixed_precision import validate_mixed_precision_policy, validate_offload_policy
from .parallel.fsdp_unit import MatrixFSDPNoSync, MatrixFSDPParamGroup
from .parallel.scheduler import DEFAULT_MAX_UNSHARDED_PREFETCH_UNITS, MatrixFSDPScheduler
from .parallel.unit_collection import collect_param_groups
from .planning.auto_planner import (AutoPlannerPolicy, auto_group_plan, make_cost_aware_muon_shard_aware_group_planner,
                                    make_model_wide_muon_planner, make_muon_shard_aware_group_planner,
                                    make_scoped_muon_shard_aware_group_planner)
from .planning.planner import ShardPlan, hinted_ordered_group_plan
from .planning.planner_eval import GroupPlanner
from .planning.shard_hint import build_shard_hints

LayoutPlanner = GroupPlanner
WrapPolicy = Callable[[nn.Module], bool]

_DEFAULT_MP_POLICY = MixedPrecisionPolicy()
_DEFAULT_OFFLOAD_POLICY = OffloadPolicy()
_MUON_POLICIES = {"mixed_muon_adamw", "muon_adamw", "muon_shard_aware", "muon"}
_NOOP_POLICIES = {"default", "none", "adamw", "sgd"}

# one stateful owner planner per mesh so successive fully_shard(block) calls balance globally
_SHARED_OWNER_PLANNERS: "weakref.WeakKeyDictionary" = weakref.WeakKeyDictionary()
_SHARED_OWNER_PLANNER_NO_MESH: dict[str, GroupPlanner] = {}


def reset_shared_owner_planners() -> None:
    """Forget cumulative owner load (call between independent models in one process)."""
    _SHARED_OWNER_PLANNERS.clear()
    _SHARED_OWNER_PLANNER_NO_MESH.clear()


def _single_dp_mesh_dim(value, *, arg_name: str):
    if not isinstance(value, tuple):
        return value
    if len(value) != 1:
        raise NotImplementedError(
            f"{arg_name} with flattened mesh dims is not supported yet; pass a single mesh dimension.")
    return value[0]


def _resolve_dp_mesh_dims(dp_mesh_dims, *, dp_shard_mesh_dim, dp_replicate_mesh_dim):
    if dp_mesh_dims is None:
        return dp_shard_mesh_dim, dp_replicate_mesh_dim
    if dp_shard_mesh_dim is not None or dp_replicate_mesh_dim is not None:
        raise ValueError("Pass either dp_mesh_dims or dp_shard_mesh_dim/dp_replicate_mesh_dim, not both.")
    shard, replicate = getattr(dp_mesh_dims, "shard", None), getattr(dp_mesh_dims, "replicate", None)
    if shard is None and replicate is None:
        raise ValueError("dp_mesh_dims must specify at least one of shard or replicate.")
    return (_single_dp_mesh_dim(shard, arg_name="dp_mesh_dims.shard"),
            _single_dp_mesh_dim(replicate, arg_name="dp_mesh_dims.replicate"))


def _resolve_optimizer_policy(optimizer_policy: str | None):
    """→ (auto_shard_hints, auto_planner_policy, owner_assignment)."""
    if optimizer_policy is None:
        return False, None, "rotate"
    key = str(optimizer_policy).lower()
    if key in _NOOP_POLICIES:
        return False, None, "rotate"
    if key in _MUON_POLICIES:
        return True, "muon_shard_aware", "role_greedy"
    valid = ", ".join(sorted(_MUON_POLICIES | _NOOP_POLICIES))
    raise ValueError(f"Unknown fully_shard optimizer_policy={optimizer_policy!r}. Valid policies: {valid}.")


def _resolve_shard_placement_hints(module: nn.Module, shard_placement_fn, *, ignored_params):
    """``Shard(0)`` answers become row-block (2-D+) or unit-block (1-D) hints plus a hinted planner."""
    if shard_placement_fn is None:
        return None, None
    ignored = {id(p) for p in ignored_params or ()}
    hints: dict[str, ParamShardHint] = {}
    for fqn, p in module.named_parameters(recurse=True, remove_duplicate=True):
        if id(p) in ignored:
            continue
        placement = shard_placement_fn(p)
        if placement is None:
            placement = Shard(0)
        if not isinstance(placement, Shard):
            raise NotImplementedError(f"shard_placement_fn must return Shard(0) or None, got {placement!r} for {fqn}.")
        if placement.dim != 0:
            raise NotImplementedError(f"Only Shard(0) placements are supported, got Shard({placement.dim}) for {fqn}.")
        if p.ndim >= 2:
            cols = p.numel() // p.shape[0]
            if p.ndim == 2:
                hints[fqn] = ParamShardHint(split_granularity="row_block", block_shape=(1, int(cols)))
            else:
                hints[fqn] = ParamShardHint(split_granularity="block", block_shape=(int(cols),))
        else:
            hints[fqn] = ParamShardHint(split_granularity="block", block_shape=(1,))
    planner = partial(hinted_ordered_group_plan, default_granularity="parameter")
    planner.__name__ = "hinted_ordered_group_plan"  # type: ignore[attr-defined]
    return hints, planner


def _resolve_reshard_after_forward(value):
    if value is None:
        return True
    if isinstance(value, bool):
        return value
    if isinstance(value, int):
        if value <= 1:
            raise ValueError(f"reshard_after_forward as an int must be a non-trivial divisor, got {value}.")
        raise NotImplementedError("reshard_after_forward=int is not supported; pass a bool.")
    raise TypeError("reshard_after_forward must be a bool, an int or None.")


def _resolve_auto_group_planner(policy, *, target_block_units=None, rotation_strategy="greedy_balance",
                                owner_assignment="rotate") -> GroupPlanner:
    name = policy.name if isinstance(policy, AutoPlannerPolicy) else policy
    if name == "muon_shard_aware":
        return make_muon_shard_aware_group_planner(policy=policy, rotation_strategy=rotation_strategy,
                                                   owner_assignment=owner_assignment)
    if rotation_strategy != "greedy_balance" or owner_assignment != "rotate":
        raise ValueError("rotation_strategy and owner_assignment are only supported with "
                         "auto_planner_policy='muon_shard_aware'.")
    planner = partial(auto_group_plan, policy=policy, target_block_units=target_block_units)
    planner.__name__ = "auto_group_plan"  # type: ignore[attr-defined]
    return planner


def _shared_owner_planner(mesh, policy, owner_assignment) -> GroupPlanner:
    key = f"{policy}:{owner_assignment}"
    if mesh is None:
        store = _SHARED_OWNER_PLANNER_NO_MESH
    else:
        store = _SHARED_OWNER_PLANNERS.setdefault(mesh, {})
    if key not in store:
        store[key] = _resolve_auto_group_planner(policy, owner_assignment=owner_assignment)
    return store[key]


def _attach_no_sync(module: nn.Module, units) -> None:
    units = list(units)

    def no_sync() -> MatrixFSDPNoSync:
        return MatrixFSDPNoSync(collect_param_groups(module) or units)

    module.no_sync = no_sync  # type: ignore[assignment]


def fully_shard(module: nn.Module, *, mesh=None, reshard_after_forward: bool | int | None = None,
                shard_placement_fn: Callable[[nn.Parameter], object | None] | None = None,
                mp_policy: MixedPrecisionPolicy = _DEFAULT_MP_POLICY,
                offload_policy: OffloadPolicy = _DEFAULT_OFFLOAD_POLICY,
                ignored_params: set[nn.Parameter] | None = None, dp_mesh_dims: DataParallelMeshDims | object | None = None,
                optimizer_policy: str | None = None) -> nn.Module:
    validate_mixed_precision_policy(mp_policy)
    validate_offload_policy(offload_policy)
    auto_hints, auto_policy, owner_assignment = _resolve_optimizer_policy(optimizer_policy)
    if auto_policy is not None and shard_placement_fn is not None:
        raise ValueError("fully_shard optimizer_policy cannot be combined with shard_placement_fn.")
    hints, group_planner = _resolve_shard_placement_hints(module, shard_placement_fn, ignored_params=ignored_params)
    shard_dim, replicate_dim = _resolve_dp_mesh_dims(dp_mesh_dims, dp_shard_mesh_dim=None, dp_replicate_mesh_dim=None)
    if auto_policy is not None:
        group_planner = _shared_owner_planner(mesh, auto_policy, owner_assignment)
    return _matrix_fully_shard_single(
        module, mesh=mesh, dp_shard_mesh_dim=shard_dim, dp_replicate_mesh_dim=replicate_dim,
        ignored_params=ignored_params, shard_hints=hints, group_planner=group_planner, auto_shard_hints=auto_hints,
        reshard_after_forward=_resolve_reshard_after_forward(reshard_after_forward), mp_policy=mp_policy,
        offload_policy=offload_policy)


def _collect_wrap_policy_modules(module: nn.Module, wrap_policy: WrapPolicy, *, ignored_params=None) -> list[nn.Module]:
    """Post-order (children before parents) list of sub-modules selected by ``wrap_policy``."""
    ignored = {id(p) for p in ignored_params or ()}
    out: list[nn.Module] = []
    claimed: set[int] = set()     # parameters that a selected descendant will already manage

    def visit(m: nn.Module) -> None:
        for child in m.children():
            visit(child)
        if wrap_policy(m):
            own = {id(p) for p in m.parameters()} - ignored - claimed
            if own:
                out.append(m)
                claimed.update(own)

    visit(module)
    return out


def matrix_fully_shard(module: nn.Module, mesh=None, *, dp_mesh_dims=None, dp_shard_mesh_dim: MeshDim | None = None,
                       dp_replicate_mesh_dim: MeshDim | None = None,
                       planner: Callable[[int, int], ShardPlan] | None = None, group_planner: GroupPlanner | None = None,
                       layout_planner: LayoutPlanner | None = None,
                       shard_hints: Mapping[str, ParamShardHint] | None = None,
                       ignored_params: set[nn.Parameter] | None = None, auto_shard_hints: bool = False,
                       auto_planner_policy: str | AutoPlannerPolicy | None = None,
                       target_block_units: int | None = None, rotation_strategy: str = "greedy_balance",
                       owner_assignment: str = "rotate", divide_grads_by_world: bool = True,
                       reshard_after_forward: bool | int = True, forward_prefetch: bool = True,
                       backward_prefetch: bool = True, finalize_after_backward: bool = True,
                       mp_policy: MixedPrecisionPolicy = _DEFAULT_MP_POLICY,
                       offload_policy: OffloadPolicy = _DEFAULT_OFFLOAD_POLICY, param_gather_strategy: str = "auto",
                       matrix_collective_backend: str = "owner_broadcast", grad_reduce_strategy: str | None = None,
                       backward_reduce_strategy: str | None = None, runtime_layout_policy: str = "auto",
                       wrap_policy: WrapPolicy | None = None, runtime_trace_enabled: bool = True,
                       use_saved_tensor_hooks: bool = False, use_zero_copy_grad_bucket: bool = False,
                       shrink_full_param_storage_after_backward: bool = True, allow_shared_params: bool = False,
                       transport=None) -> nn.Module:
    """Expert API: every planner / runtime knob, plus ``wrap_policy`` recursion with look-ahead planning."""
    if backward_reduce_strategy is None:
        backward_reduce_strategy = grad_reduce_strategy or "bucket_reduce_scatter"
    elif grad_reduce_strategy is not None and grad_reduce_strategy != backward_reduce_strategy:
        raise ValueError("Pass only one of grad_reduce_strategy or backward_reduce_strategy, or pass the same value.")
    validate_mixed_precision_policy(mp_policy)
    validate_offload_policy(offload_policy)
    shard_dim, replicate_dim = _resolve_dp_mesh_dims(dp_mesh_dims, dp_shard_mesh_dim=dp_shard_mesh_dim,
                                                     dp_replicate_mesh_dim=dp_replicate_mesh_dim)
    common = dict(
        mesh=mesh, dp_shard_mesh_dim=shard_dim, dp_replicate_mesh_dim=replicate_dim, planner=planner,
        layout_planner=layout_planner, ignored_params=ignored_params, auto_shard_hints=auto_shard_hints,
        divide_grads_by_world=divide_grads_by_world, reshard_after_forward=reshard_after_forward,
        forward_prefetch=forward_prefetch, backward_prefetch=backward_prefetch,
        finalize_after_backward=finalize_after_backward, mp_policy=mp_policy, offload_policy=offload_policy,
        param_gather_strategy=param_gather_strategy, matrix_collective_backend=matrix_collective_backend,
        backward_reduce_strategy=backward_reduce_strategy, runtime_layout_policy=runtime_layout_policy,
        runtime_trace_enabled=runtime_trace_enabled, use_saved_tensor_hooks=use_saved_tensor_hooks,
        use_zero_copy_grad_bucket=use_zero_copy_grad_bucket,
        shrink_full_param_storage_after_backward=shrink_full_param_storage_after_backward,
        allow_shared_params=allow_shared_params, transport=transport)
    if wrap_policy is None:
        return _matrix_fully_shard_single(module, shard_hints=shard_hints, group_planner=group_planner,
                                          auto_planner_policy=auto_planner_policy,
                                          target_block_units=target_block_units, rotation_strategy=rotation_strategy,
                                          owner_assignment=owner_assignment, **common)
    if shard_hints is not None:
        raise ValueError("wrap_policy does not support explicit shard_hints yet.")
    selected = _collect_wrap_policy_modules(module, wrap_policy, ignored_params=ignored_params)
    if not selected:
        raise ValueError("wrap_policy did not select any modules to shard.")
    if auto_planner_policy is not None:
        if group_planner is not None or layout_planner is not None:
            raise ValueError("Pass either auto_planner_policy or an explicit group/layout planner, not both.")
        if owner_assignment in ("scope_greedy", "cost_aware", "model_wide"):
            claimed: set[int] = set()
            scoped = []
            for m in selected:
                extra_ignored = set(ignored_params or ()) | {p for p in m.parameters() if id(p) in claimed}
                reg = ManagedParamRegistry.from_module(
                    m, shard_hints=_filter_hints(m, build_shard_hints(m) if auto_shard_hints else None, extra_ignored),
                    ignored_params=extra_ignored, allow_shared=allow_shared_params)
                claimed |= {id(mp.param) for mp in reg}
                scoped.append(reg.params)
            # all three see every selected module's parameters before the first unit is planned; "model_wide"
            # balances the owners by Newton-Schulz FLOPs over the whole model
            maker = {"cost_aware": make_cost_aware_muon_shard_aware_group_planner,
                     "scope_greedy": make_scoped_muon_shard_aware_group_planner,
                     "model_wide": make_model_wide_muon_planner}[owner_assignment]
            group_planner = maker(tuple(scoped), policy=auto_planner_policy)
        else:
            group_planner = _resolve_auto_group_planner(auto_planner_policy, target_block_units=target_block_units,
                                                        rotation_strategy=rotation_strategy,
                                                        owner_assignment=owner_assignment)
    for m in selected:
        _matrix_fully_shard_single(m, shard_hints=None, group_planner=group_planner, **common)
    units = collect_param_groups(module)
    MatrixFSDPScheduler(units, max_unsharded_prefetch_units=DEFAULT_MAX_UNSHARDED_PREFETCH_UNITS)
    _attach_no_sync(module, units)
    return module


def _filter_hints(module: nn.Module, hints, ignored: set) -> dict | None:
    if hints is None:
        return None
    ids = {id(p) for p in ignored}
    keep = {fqn for fqn, p in module.named_parameters(recurse=True, remove_duplicate=True) if id(p) not in ids}
    return {k: v for k, v in hints.items() if k in keep}


def _matrix_fully_shard_single(module: nn.Module, *, mesh=None, dp_shard_mesh_dim=None, dp_replicate_mesh_dim=None,
                               planner=None, group_planner=None, layout_planner=None, shard_hints=None,
                               ignored_params=None, auto_shard_hints=False, auto_planner_policy=None,
                               target_block_units=None, rotation_strategy="greedy_balance", owner_assignment="rotate",
                               **unit_kwargs) -> nn.Module:
    if sum(x is not None for x in (planner, group_planner, layout_planner)) > 1:
        raise ValueError("Pass at most one of planner, group_planner and layout_planner.")
    if auto_planner_policy is not None:
        if planner is not None or group_planner is not None or layout_planner is not None:
            raise ValueError("Pass either auto_planner_policy or an explicit planner, not both.")
        group_planner = _resolve_auto_group_planner(auto_planner_policy, target_block_units=target_block_units,
                                                    rotation_strategy=rotation_strategy,
                                                    owner_assignment=owner_assignment)
    unit = MatrixFSDPParamGroup(module, mesh=mesh, dp_shard_mesh_dim=dp_shard_mesh_dim,
                                dp_replicate_mesh_dim=dp_replicate_mesh_dim, planner=planner,
                                group_planner=group_planner, layout_planner=layout_planner, shard_hints=shard_hints,
                                ignored_params=ignored_params, auto_shard_hints=auto_shard_hints, **unit_kwargs)
    unit.init()
    _attach_no_sync(module, [unit])
    return module
