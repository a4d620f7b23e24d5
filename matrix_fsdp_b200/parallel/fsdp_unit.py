"""``MatrixFSDPParamGroup``: lifecycle engine of one FSDP unit (one ``fully_shard`` call).

States and transitions::

    SHARDED --unshard--> UNSHARDED --post-forward reshard--> FORWARD_RESHARDED
       ^                     |                                     |
       |                     +<-------- pre-backward unshard <-----+
       +---- finalize backward (collect grads, reshard, reduce-scatter) ----+

Hooks: a forward pre-hook (unshard + wait + prefetch the next unit), a forward hook (register
pre-backward tensor hooks on the outputs, reshard), a post-accumulate-grad hook per parameter
(count gradients; the last one finalises the unit) and an end-of-backward engine callback that
finalises units whose parameters did not all receive gradients.  Forwards that run *inside* a
backward pass (activation-checkpoint recompute) find the unit already UNSHARDED and skip all
of this.

Parity: ``matrix_fsdp/runtime/fsdp_unit.py:63-1773``.
"""
from __future__ import annotations

import os
import time
import weakref
from collections.abc import Callable, Mapping
from enum import Enum
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ..core.layout import MatrixGroupLayout, ShardPlan
from ..core.managed_param import ManagedParamRegistry, ParamShardHint
from ..core.mesh import ResolvedGroups, resolve_groups
from ..core.mixed_precision import (cast_floating_tensors, mixed_precision_policy_metadata, offload_policy_metadata,
                                    validate_offload_policy_for_device)
from ..planning.layout_validator import flat_reorder_order, validate_group_layout, validate_runtime_layout
from ..planning.planner import contiguous_even_plan
from ..planning.planner_eval import PlannerResult, call_group_planner, planner_result_from_output
from ..planning.shard_hint import build_shard_hints
from .flat_buffer import MatrixFlatBuffer
from .hooks import ForwardBackwardContext, register_pre_backward_hooks
from .runtime_event import (RuntimeEvent, RuntimeUnitMetadata, next_event_sequence, next_runtime_param_group_id,
                            nvtx_range)
from .transport import make_transport


class FSDPLifecycleState(str, Enum):
    SHARDED = "sharded"
    UNSHARDED = "unsharded"
    FORWARD_RESHARDED = "forward_resharded"


FSDPRuntimeState = FSDPLifecycleState

# ``param_gather_strategy``: "auto" leaves the choice to the unit's transport; every other value names a
# library collective (matrix_fsdp/runtime/flat_buffer.py:304-382) and is run as such.
_GATHER_STRATEGIES = {"auto": None, "equal_all_gather": "equal_all_gather", "matrix_all_gather": "padded",
                      "owner_broadcast": "owner_broadcast", "uneven_all_gather": "uneven_all_gather",
                      "all_reduce": "all_reduce"}

_ALLOWED = {
    (FSDPLifecycleState.SHARDED, FSDPLifecycleState.UNSHARDED),
    (FSDPLifecycleState.UNSHARDED, FSDPLifecycleState.FORWARD_RESHARDED),
    (FSDPLifecycleState.UNSHARDED, FSDPLifecycleState.SHARDED),
    (FSDPLifecycleState.FORWARD_RESHARDED, FSDPLifecycleState.UNSHARDED),
    (FSDPLifecycleState.FORWARD_RESHARDED, FSDPLifecycleState.SHARDED),
}


def _in_backward() -> bool:
    try:
        return torch._C._current_graph_task_id() != -1
    except Exception:  # pragma: no cover
        return False


class _SavedFullView:
    """What autograd keeps instead of a view of an unsharded buffer (``use_saved_tensor_hooks``)."""

    __slots__ = ("unit", "offset", "size", "stride", "requires_grad")

    def __init__(self, unit, offset: int, size: tuple, stride: tuple, requires_grad: bool) -> None:
        self.unit, self.offset, self.size, self.stride, self.requires_grad = unit, offset, size, stride, requires_grad


class MatrixFSDPNoSync:
    """Context manager deferring gradient reduction of a set of units (gradient accumulation)."""

    def __init__(self, units) -> None:
        self.units = list(units)
        self._prev: list[tuple[bool, bool]] = []

    def __enter__(self):
        # both flags are put back as they were found, so contexts nest: leaving an inner one keeps the outer in force
        self._prev = [(u.defer_backward_reduce, u.in_no_sync) for u in self.units]
        for u in self.units:
            u.defer_backward_reduce = True
            u.in_no_sync = True
        return self

    def __exit__(self, *exc):
        for u, (defer, inside) in zip(self.units, self._prev):
            u.defer_backward_reduce = defer
            u.in_no_sync = inside
        return False


class MatrixFSDPParamGroup:
    def __init__(self, module: nn.Module, *, mesh=None, dp_shard_mesh_dim=None, dp_replicate_mesh_dim=None,
                 planner: Callable[[int, int], ShardPlan] | None = None, group_planner=None, layout_planner=None,
                 shard_hints: Mapping[str, ParamShardHint] | None = None, ignored_params=None,
                 auto_shard_hints: bool = False, divide_grads_by_world: bool = True,
                 reshard_after_forward: bool | int = True, forward_prefetch: bool = True,
                 backward_prefetch: bool = True, finalize_after_backward: bool = True, mp_policy=None,
                 offload_policy=None, param_gather_strategy: str = "auto",
                 matrix_collective_backend: str = "owner_broadcast",
                 backward_reduce_strategy: str = "bucket_reduce_scatter", runtime_layout_policy: str = "auto",
                 runtime_trace_enabled: bool = True, use_saved_tensor_hooks: bool = False,
                 use_zero_copy_grad_bucket: bool = False, shrink_full_param_storage_after_backward: bool = True,
                 allow_shared_params: bool = False, transport=None, use_world_without_mesh: bool = True) -> None:
        if isinstance(reshard_after_forward, bool):
            self.reshard_after_forward = reshard_after_forward
        elif isinstance(reshard_after_forward, int):
            if reshard_after_forward <= 1:
                raise ValueError("reshard_after_forward as an int must be a non-trivial divisor of the shard "
                                 f"world size, got {reshard_after_forward}.")
            raise NotImplementedError("reshard_after_forward=int (resharding to a smaller subgroup) is not supported; "
                                      "pass a bool.")
        else:
            raise TypeError("reshard_after_forward must be a bool.")
        valid_reduce = {"bucket_reduce_scatter", "flat", "per_param", "per_param_allreduce"}
        if backward_reduce_strategy not in valid_reduce:
            raise ValueError(f"Unknown backward_reduce_strategy={backward_reduce_strategy!r}; "
                             f"expected one of {sorted(valid_reduce)}.")
        if runtime_layout_policy not in ("auto", "matrix_shard", "segment_runtime", "flat_reorder"):
            raise ValueError(f"Unknown runtime_layout_policy={runtime_layout_policy!r}.")
        if param_gather_strategy not in _GATHER_STRATEGIES:
            raise ValueError(f"param_gather_strategy must be one of {sorted(_GATHER_STRATEGIES)}, "
                             f"got {param_gather_strategy!r}.")
        if matrix_collective_backend not in ("torch", "owner_broadcast", "custom"):
            raise ValueError("matrix_collective_backend must be 'torch', 'owner_broadcast', or 'custom'.")
        self.module = module
        self.mesh = mesh
        self.groups: ResolvedGroups = resolve_groups(mesh, dp_shard_mesh_dim, dp_replicate_mesh_dim,
                                                     use_world_without_mesh=use_world_without_mesh)
        self.rank, self.world_size = self.groups.shard_rank, self.groups.shard_world
        self.replicate_rank, self.replicate_world_size = self.groups.replicate_rank, self.groups.replicate_world
        self.planner, self.group_planner, self.layout_planner = planner, group_planner, layout_planner
        self.shard_hints = shard_hints
        self.ignored_params = ignored_params
        self.auto_shard_hints = auto_shard_hints
        self.divide_grads_by_world = divide_grads_by_world
        self.forward_prefetch, self.backward_prefetch = forward_prefetch, backward_prefetch
        self.finalize_after_backward = finalize_after_backward
        self.mp_policy, self.offload_policy = mp_policy, offload_policy
        self.param_gather_strategy = param_gather_strategy
        self.matrix_collective_backend = matrix_collective_backend
        self.backward_reduce_strategy = backward_reduce_strategy
        self.runtime_layout_policy = runtime_layout_policy
        self.runtime_trace_enabled = runtime_trace_enabled
        # (lo, hi, row_len) of the weight whose all-gather may be fused into the block's first GEMM
        self.fused_first_gemm_range: tuple | None = None
        self._module_fuses_first_gemm = False
        self.use_saved_tensor_hooks = use_saved_tensor_hooks
        self.use_zero_copy_grad_bucket = use_zero_copy_grad_bucket
        self.shrink_full_param_storage_after_backward = shrink_full_param_storage_after_backward
        self.allow_shared_params = allow_shared_params
        self._transport_override = transport

        self.metadata = RuntimeUnitMetadata(next_runtime_param_group_id(), 0, 0)
        self.metadata = RuntimeUnitMetadata(self.metadata.runtime_param_group_id, self.metadata.runtime_param_group_id,
                                            self.metadata.runtime_param_group_id)
        self.name = self.metadata.name
        self.state = FSDPLifecycleState.SHARDED
        self.runtime_events: list[RuntimeEvent] = []
        self.scheduler = None
        self.all_gather_stream = None
        self.reduce_scatter_stream = None
        self.defer_backward_reduce = False
        self.in_no_sync = False
        self.finalized_after_backward = False
        self.has_accumulated_grads = False
        self.forward_count_since_backward = 0
        self.used_in_forward = False
        self.unshard_prefetched = False
        self._grads_seen: set[str] = set()
        self._direct_written: set[str] = set()
        self._pre_backward_done = False
        self._backward_contexts: list = []          # weak references to the hook contexts of live graphs
        self._backward_callback_queued = False
        self._hook_handles: list = []
        self._initialized = False
        self._saved_hooks_ctx = None
        self._saved_view_count = 0
        self._zero_copy_grads: dict[str, torch.Tensor] = {}
        self.planner_result: PlannerResult | None = None
        self.registry: ManagedParamRegistry | None = None
        self.flat_buffer: MatrixFlatBuffer | None = None
        self.runtime_mode = "unknown"

    # ------------------------------------------------------------------ init
    def init(self) -> "MatrixFSDPParamGroup":
        if self._initialized:
            return self
        module = self.module
        if getattr(module, "_matrix_fsdp_param_group", None) is not None:
            raise ValueError("This module is already managed by an FSDP unit.")
        ignored = set(self.ignored_params or ())
        # parameters already managed by nested units stay with them; a parameter managed by a unit that is NOT
        # inside this module is shared between two modules, and its other user would read it while the owning
        # unit keeps it sharded
        inner = {id(m) for m in module.modules()}
        nested = set()
        for fqn, p in module.named_parameters():
            ref = getattr(p, "_mfsdp_unit_ref", None)
            owner = ref() if ref is not None else None
            if owner is None:
                continue
            if id(owner.module) not in inner and p not in ignored:
                raise ValueError(f"Parameter {fqn!r} is shared with a module that another FSDP unit ({owner.name}) "
                                 "already manages; shard both users in one unit (allow_shared_params=True on a common "
                                 "parent) or pass it through ignored_params.")
            nested.add(id(p))
        ignored |= {p for p in module.parameters() if id(p) in nested}
        hints = self.shard_hints
        if hints is None and self.auto_shard_hints:
            hints = build_shard_hints(module)
        if hints is not None:
            keep = {fqn for fqn, p in module.named_parameters() if p not in ignored}
            hints = {k: v for k, v in hints.items() if k in keep}
        registry = ManagedParamRegistry.from_module(module, shard_hints=hints, ignored_params=ignored,
                                                    allow_shared=self.allow_shared_params)
        if len(registry) == 0:
            raise ValueError("fully_shard needs a module with at least one parameter that is not ignored.")
        frozen = [mp.fqn for mp in registry if not mp.param.requires_grad]
        if frozen:
            raise ValueError(f"Managed parameters must require grad; frozen parameters: {', '.join(frozen)}. "
                             "Pass them through ignored_params.")
        device = registry[0].device
        if self.offload_policy is not None:
            validate_offload_policy_for_device(self.offload_policy, device)
        self.registry = registry

        result = self._plan(registry)
        compat = validate_runtime_layout(
            result.layout, registry.params, self.world_size,
            allow_segment_runtime=self.runtime_layout_policy in ("auto", "segment_runtime"),
            allow_flat_reorder=self.runtime_layout_policy in ("auto", "flat_reorder"))
        if self.runtime_layout_policy == "matrix_shard" and compat.mode != "matrix_shard":
            raise ValueError(f"MatrixFSDP runtime cannot execute planner layout. Reason: {compat.reason}.")
        if compat.mode == "flat_reorder" or (self.runtime_layout_policy == "flat_reorder" and compat.mode != "matrix_shard"):
            result = self._flat_reorder(registry, result)
            compat = validate_runtime_layout(result.layout, registry.params, self.world_size)
        self.planner_result = result
        self.runtime_mode = compat.mode
        validate_group_layout(result.layout, registry.params, self.world_size)

        if device.type == "cuda":
            self.all_gather_stream = torch.cuda.Stream(device=device, priority=-1)
            self.reduce_scatter_stream = torch.cuda.Stream(device=device, priority=-1)
        # matrix_collective_backend: "torch" = library collectives only, "custom" = the peer kernels or an
        # error, "owner_broadcast" (default) = whatever the node offers
        prefer = {"torch": "torch_dist", "custom": "peer"}.get(self.matrix_collective_backend)
        if prefer == "peer" and (device.type != "cuda" or self.world_size <= 1):
            prefer = None
        transport = self._transport_override or make_transport(self.groups.shard_group, self.world_size, device,
                                                               prefer=prefer)
        mp = self.mp_policy
        self.flat_buffer = MatrixFlatBuffer(
            registry, result.layout, rank=self.rank, world_size=self.world_size, transport=transport,
            replicate_group=self.groups.replicate_group, replicate_world_size=self.replicate_world_size,
            param_dtype=getattr(mp, "param_dtype", None), reduce_dtype=getattr(mp, "reduce_dtype", None),
            divide_grads_by_world=self.divide_grads_by_world, unit_key=self.name,
            exclusive_full_buffer=not self.reshard_after_forward or not self.shrink_full_param_storage_after_backward,
            gather_impl=_GATHER_STRATEGIES[self.param_gather_strategy], shard_group=self.groups.shard_group)
        self.flat_buffer.use_local_shards()
        if self.use_saved_tensor_hooks:
            from .buffer_pool import global_full_param_buffer_pool

            # saved views are re-created from the buffer of backward time, so the buffer can be pooled
            self.flat_buffer.use_full_param_pool(global_full_param_buffer_pool())

        ref = weakref.ref(self)
        for mpm in registry:
            # a name of this package's own: the reference package hooks every torch optimizer in the process and
            # reads its own back-reference from the parameters, so the two must not share the attribute
            mpm.param._mfsdp_unit_ref = ref
            mpm.param._matrix_fsdp_fqn = mpm.fqn
        module._matrix_fsdp_param_group = self
        self._register_hooks()
        self._initialized = True
        self._record("init", reason=f"planner={result.name}")
        return self

    def _plan(self, registry: ManagedParamRegistry) -> PlannerResult:
        params, world = registry.params, self.world_size
        chosen = self.group_planner or self.layout_planner
        if chosen is not None:
            return call_group_planner(chosen, params, world,
                                      shard_mesh_dim=self.groups.metadata.shard_mesh_dim if self.groups.metadata else None)
        if self.planner is not None:
            plan = self.planner(registry.total_numel, world)
            return planner_result_from_output(getattr(self.planner, "__name__", "planner"), plan, params, world)
        if any(mp.shard_hint is not None and mp.shard_hint.split_granularity is not None for mp in params):
            # hints without a planner: an even split would cut what the hints forbid to cut (and be refused by the
            # validator), so take the rank-contiguous plan that cuts only where every hint allows
            from ..planning.planner import hinted_ordered_group_plan

            return call_group_planner(hinted_ordered_group_plan, params, world)
        # on CUDA every shard boundary sits on a 16-byte boundary of the bf16 wire format so the peer
        # kernels (and TMA) can address any rank's shard with full-width vector accesses
        align = 8 if registry[0].device.type == "cuda" and registry.total_numel >= 64 * world else 1
        return planner_result_from_output("contiguous_even_plan",
                                          contiguous_even_plan(registry.total_numel, world, align=align), params, world)

    def _flat_reorder(self, registry: ManagedParamRegistry, result: PlannerResult) -> PlannerResult:
        """Re-lay the flat space rank-major so a whole-param owner layout becomes rank-contiguous."""
        order = flat_reorder_order(result.layout)
        owners = {fqn: result.layout.owner_ranks(fqn)[0] for fqn in order}
        registry.reassign_offsets(order)
        from ..core.layout import LayoutSegment

        per_rank: list[list] = [[] for _ in range(self.world_size)]
        cursor = [0] * self.world_size
        for mp in registry.params:
            r = owners[mp.fqn]
            per_rank[r].append(LayoutSegment(mp.offset, mp.end, cursor[r]))
            cursor[r] += mp.numel
        from ..core.layout import coalesce_segments

        layout = MatrixGroupLayout.from_rank_segments(registry.total_numel, [coalesce_segments(s) for s in per_rank],
                                                      registry.params)
        return planner_result_from_output(result.name, layout, registry.params, self.world_size, policy=result.policy,
                                          weights=result.cost_weights)

    def _register_hooks(self) -> None:
        m = self.module
        self._hook_handles.append(m.register_forward_pre_hook(self._pre_forward, with_kwargs=True, prepend=True))
        self._hook_handles.append(m.register_forward_hook(self._post_forward, prepend=False))
        for mp in self.registry:
            self._hook_handles.append(mp.param.register_post_accumulate_grad_hook(self._make_grad_hook(mp.fqn)))

    # ------------------------------------------------------------------ events
    def _record(self, name: str, *, start: float | None = None, handle=None, **kw) -> None:
        if not self.runtime_trace_enabled:
            return
        dur = (time.perf_counter() - start) * 1e3 if start is not None else 0.0
        info = getattr(handle, "info", None) or {}
        span = getattr(handle, "span", None)
        if span is not None:
            kw["extra"] = {**kw.get("extra", {}), "span": span}      # device-side times, resolved by the summaries
        if info.get("host_phases_ms"):
            kw["extra"] = {**kw.get("extra", {}), "host_phases_ms": dict(info["host_phases_ms"])}
        snap = self.flat_buffer.memory_snapshot() if self.flat_buffer is not None else {}
        sched = self.scheduler
        self.runtime_events.append(RuntimeEvent(
            name=name, unit=self.name, sequence=next_event_sequence(), lifecycle_state=self.state.value,
            duration_ms=dur, collective_kind=info.get("kind"), collective_backend=info.get("backend"),
            collective_impl=info.get("impl"), collective_bytes=int(info.get("bytes", 0)),
            collective_count=int(info.get("count", 0)), collective_sync_mode=info.get("sync_mode"),
            workspace_numel=int(info.get("workspace_numel", 0)), workspace_reused=bool(info.get("workspace_reused", False)),
            materialization=info.get("materialization"),
            full_param_buffer_numel=snap.get("full_param_buffer_numel", 0),
            full_param_buffer_bytes=snap.get("full_param_buffer_bytes", 0),
            grad_bucket_numel=snap.get("grad_bucket_numel", 0), grad_bucket_bytes=snap.get("grad_bucket_bytes", 0),
            local_grad_shard_numel=snap.get("local_grad_shard_numel", 0),
            local_grad_shard_bytes=snap.get("local_grad_shard_bytes", 0),
            active_full_param_buffers=sched.active_full_param_buffers() if sched is not None else 0,
            pending_reduce_scatter_count=sched.pending_reduce_count() if sched is not None else
            int(self.flat_buffer is not None and self.flat_buffer.pending_reduce is not None),
            **kw))

    def clear_runtime_events(self) -> None:
        self.runtime_events.clear()

    # ------------------------------------------------------------------ state machine
    def _transition(self, new: FSDPLifecycleState) -> None:
        if new == self.state:
            return
        if (self.state, new) not in _ALLOWED:
            raise RuntimeError(f"{self.name}: illegal lifecycle transition {self.state.value} -> {new.value}.")
        self.state = new

    def _check_invariants(self) -> None:
        fb = self.flat_buffer
        if self.state == FSDPLifecycleState.UNSHARDED:
            if not fb.full_materialized:
                raise RuntimeError(f"{self.name}: UNSHARDED without a materialised full buffer.")
        else:
            if fb.params_use_full:
                raise RuntimeError(f"{self.name}: {self.state.value} but parameters still view the full buffer.")

    # ------------------------------------------------------------------ unshard / reshard
    def start_unshard(self, reason: str = "manual", after_event=None) -> None:
        """``after_event``: the parameters of this unit are final once this CUDA event has happened (its
        update ran inside its own reduce-scatter); the gather waits for it instead of the whole optimizer step."""
        if self.flat_buffer.pending_gather is not None or self.state == FSDPLifecycleState.UNSHARDED:
            return
        t0 = time.perf_counter()
        if after_event is not None and self.all_gather_stream is not None:
            self.all_gather_stream.wait_event(after_event)
            if self.scheduler is not None:
                self.scheduler.note_unshard_started(self)
        elif self.scheduler is not None:
            self.scheduler.wait_for_post_optimizer_event_before_all_gather(self)
            self.scheduler.note_unshard_started(self)
        # Fuse the q|k|v rows into the block's first GEMM when the gather is on the critical path (issued by
        # the forward that needs it); a prefetched gather is already hidden behind the previous block.
        defer = None
        if "backward" not in reason and getattr(self, "fused_first_gemm_range", None) is not None \
                and not _in_backward() and torch.is_grad_enabled() \
                and (not reason.endswith("prefetch") or os.environ.get("MFSDP_FUSED_AG_GEMM", "exposed") == "always") \
                and not self.flat_buffer.full_persistent:
            defer = self.fused_first_gemm_range
        with nvtx_range(f"mfsdp.all_gather:{self.name}"):
            h = self.flat_buffer.start_all_gather_full_params(stream=self.all_gather_stream, defer=defer,
                                                              ordered_by_caller=after_event is not None)
        self.unshard_prefetched = reason.endswith("prefetch")
        if getattr(h, "span", None) is not None:
            h.span.unit, h.span.reason = self.name, reason
        self._record(f"start_unshard:{reason}", start=t0, handle=h, reason=reason, prefetched=self.unshard_prefetched)

    def wait_unshard(self, reason: str = "manual") -> None:
        t0 = time.perf_counter()
        if self.state == FSDPLifecycleState.UNSHARDED:
            return
        if self.flat_buffer.pending_gather is None:
            self.start_unshard(reason)
        # rows left to the block's first GEMM stay pending only when the module said it will run that GEMM
        h = self.flat_buffer.wait_all_gather(keep_deferred=(reason == "pre_forward" and self._module_fuses_first_gemm))
        if self.scheduler is not None and h is not None:
            self.scheduler.note_unshard_wait(self, (time.perf_counter() - t0) * 1e3, getattr(h, "span", None))
        self.flat_buffer.use_full_param_buffer()
        self._transition(FSDPLifecycleState.UNSHARDED)
        self._record(f"wait_unshard:{reason}", start=t0, handle=h, reason=reason)
        self._record("unshard", reason=reason, prefetched=self.unshard_prefetched)

    def unshard(self, reason: str = "manual") -> "MatrixFSDPParamGroup":
        self.start_unshard(reason)
        self.wait_unshard(reason)
        return self

    def reshard(self, reason: str = "manual", *, to: FSDPLifecycleState = FSDPLifecycleState.SHARDED,
                keep_storage: bool = False) -> None:
        """``keep_storage``: leave the unsharded storage allocated (its contents are stale from here on and
        the next unshard gathers into it again); trades memory for allocator traffic."""
        if self.state != FSDPLifecycleState.UNSHARDED and self.flat_buffer.pending_gather is None:
            if to == FSDPLifecycleState.SHARDED and self.state == FSDPLifecycleState.FORWARD_RESHARDED:
                self._transition(to)
            return
        t0 = time.perf_counter()
        self.flat_buffer.use_local_shards()
        self.flat_buffer.clear_full_params(keep_storage=keep_storage)
        if self.state == FSDPLifecycleState.UNSHARDED:
            self._transition(to)
        if self.scheduler is not None:
            self.scheduler.note_resharded(self)
        self._record(reason if reason.startswith("reshard") else f"reshard:{reason}", start=t0, reason=reason)

    def discard_unused_prefetch(self) -> None:
        """Drop a gather that was prefetched but never consumed by a forward/backward."""
        if self.flat_buffer.pending_gather is not None and self.state != FSDPLifecycleState.UNSHARDED:
            self.flat_buffer.wait_all_gather()
            self.flat_buffer.clear_full_params()
            if self.scheduler is not None:
                self.scheduler.note_resharded(self)
            self._record("discard_unused_prefetch")

    # ------------------------------------------------------------------ forward hooks
    def _pre_forward(self, module, args, kwargs):
        if _in_backward() and self.state == FSDPLifecycleState.UNSHARDED:
            self._record("pre_forward_recompute_skip", recompute=True)
            return None
        grad_mode = torch.is_grad_enabled()
        if self.state == FSDPLifecycleState.FORWARD_RESHARDED and grad_mode and not _in_backward():
            raise RuntimeError(
                f"{self.name}: another forward before the backward of the previous one; multiple forwards before "
                "a backward need reshard_after_forward=False.")
        if self.flat_buffer.pending_reduce is not None:
            # a reduction from an earlier backward has not been consumed by an optimizer step yet:
            # finish it so its result can be folded into the next one
            if self.scheduler is not None:
                self.scheduler.drop_pending_reduce(self)
            self.wait_post_backward_reduce()
        t0 = time.perf_counter()
        self._record("pre_forward")
        self.flat_buffer.stash_local_grads_for_accumulation()
        self.used_in_forward = True
        self.finalized_after_backward = False
        probe = getattr(module, "mfsdp_fuses_first_gemm", None)
        self._module_fuses_first_gemm = bool(probe(*args, **kwargs)) if probe is not None else False
        self.start_unshard("pre_forward")
        self.wait_unshard("pre_forward")
        self._module_fuses_first_gemm = False
        if self.scheduler is not None:
            self.scheduler.on_pre_forward(self)
        if self.use_saved_tensor_hooks and grad_mode:
            self._enter_saved_tensor_hooks()
        mp = self.mp_policy
        if mp is not None and getattr(mp, "cast_forward_inputs", False) and mp.param_dtype is not None:
            args = cast_floating_tensors(args, mp.param_dtype)
            kwargs = cast_floating_tensors(kwargs, mp.param_dtype)
            return args, kwargs
        del t0
        return None

    # ------------------------------------------------------------------ saved-tensor hooks
    def _enter_saved_tensor_hooks(self) -> None:
        """While the module's forward runs, tensors that autograd saves and that are views of this unit's
        unsharded buffer are saved as (offset, size, stride) and rebuilt from the buffer as it is at
        backward time.  The graph then keeps no reference to the forward's storage, so the buffer may be
        a different allocation in backward (and the saved views never pin a released one).
        Parity: ``matrix_fsdp/runtime/fsdp_unit.py:1325-1382``."""
        if self._saved_hooks_ctx is not None:
            return
        ref = weakref.ref(self)

        def pack(t: torch.Tensor):
            unit = ref()
            if unit is None or not isinstance(t, torch.Tensor) or t.device != unit.flat_buffer.device:
                return t
            full = unit.flat_buffer.full_buffer
            if not unit.flat_buffer.full_materialized or t.dtype != full.dtype or t.numel() == 0:
                return t
            try:
                same = t.untyped_storage().data_ptr() == full.untyped_storage().data_ptr()
            except RuntimeError:
                return t
            if not same:
                return t
            unit._saved_view_count += 1
            return _SavedFullView(ref, t.storage_offset() - full.storage_offset(), tuple(t.shape), tuple(t.stride()),
                                  t.requires_grad)

        def unpack(obj):
            if not isinstance(obj, _SavedFullView):
                return obj
            unit = obj.unit()
            if unit is None:
                raise RuntimeError("the FSDP unit that owned a saved parameter view no longer exists")
            if unit.state != FSDPLifecycleState.UNSHARDED:
                raise RuntimeError(f"{unit.name}: a saved parameter view was needed while the unit is "
                                   f"{unit.state.value}; its backward has to run between pre-backward unshard and reshard.")
            full = unit.flat_buffer.full_buffer
            return full.as_strided(obj.size, obj.stride, full.storage_offset() + obj.offset)

        self._saved_hooks_ctx = torch.autograd.graph.saved_tensors_hooks(pack, unpack)
        self._saved_hooks_ctx.__enter__()
        self._record("enter_saved_tensor_hooks")

    def _exit_saved_tensor_hooks(self) -> None:
        ctx, self._saved_hooks_ctx = self._saved_hooks_ctx, None
        if ctx is not None:
            ctx.__exit__(None, None, None)
            self._record("exit_saved_tensor_hooks", extra={"saved_views": self._saved_view_count})

    def _post_forward(self, module, args, output):
        self._exit_saved_tensor_hooks()
        if _in_backward() and self._pre_backward_done and self.state == FSDPLifecycleState.UNSHARDED:
            self._record("post_forward_recompute_skip", recompute=True)
            return output
        grad_mode = torch.is_grad_enabled()
        mp = self.mp_policy
        if mp is not None and getattr(mp, "output_dtype", None) is not None:
            output = cast_floating_tensors(output, mp.output_dtype)
        hooks = 0
        if grad_mode:
            ctx = ForwardBackwardContext(self._pre_backward_unshard)
            hooks = register_pre_backward_hooks(output, ctx)
            self.forward_count_since_backward += 1
            if hooks:
                # remembered (weakly: the hooks on the outputs own it) so that it can fire again in a later
                # backward pass over the same graph, see ``finalize_backward``
                self._backward_contexts = [r for r in self._backward_contexts if r() is not None]
                self._backward_contexts.append(weakref.ref(ctx))
        if self.reshard_after_forward and grad_mode and hooks and self.scheduler is not None \
                and self.scheduler.keeps_unsharded_into_backward(self):
            # the unit that closes the forward opens the backward: resharding it now would only make the
            # backward start with the same gather again
            self._record("keep_unsharded_into_backward")
        elif self.reshard_after_forward:
            self.reshard("reshard_after_forward",
                         to=FSDPLifecycleState.FORWARD_RESHARDED if (grad_mode and hooks) else FSDPLifecycleState.SHARDED)
        elif not (grad_mode and hooks) and not self._keep_unsharded_in_eval():
            self.reshard("reshard_after_forward", to=FSDPLifecycleState.SHARDED)
        if self.scheduler is not None:
            self.scheduler.record_post_forward(self)
        self._record("post_forward", extra={"hooks": hooks})
        return output

    def _keep_unsharded_in_eval(self) -> bool:
        return not self.reshard_after_forward

    # ------------------------------------------------------------------ backward
    def _pre_backward_unshard(self) -> None:
        if self._pre_backward_done and self.state == FSDPLifecycleState.UNSHARDED:
            return
        if self.state == FSDPLifecycleState.SHARDED and self.finalized_after_backward:
            # another backward pass over a graph that was kept: this unit already reduced the gradients of the
            # earlier pass.  Finish that reduction, take its result off the parameters (their shapes are about to
            # change) and let this pass's reduction add to it, exactly as a new forward would.
            if self.flat_buffer.pending_reduce is not None:
                if self.scheduler is not None:
                    self.scheduler.drop_pending_reduce(self)
                self.wait_post_backward_reduce()
            self.flat_buffer.stash_local_grads_for_accumulation()
            self.finalized_after_backward = False
        self._record("pre_backward_unshard")
        self._pre_backward_done = True
        self._queue_backward_callback()
        self.start_unshard("pre_backward")
        self.wait_unshard("pre_backward")
        if self._wants_direct_grad_writes():
            self.flat_buffer.prepare_grad_bucket()
        elif self.use_zero_copy_grad_bucket:
            self._attach_zero_copy_grads()
        if self.scheduler is not None:
            self.scheduler.on_pre_backward(self)

    def _wants_direct_grad_writes(self) -> bool:
        return bool(getattr(self.module, "_mfsdp_direct_grad", False))

    def _attach_zero_copy_grads(self) -> None:
        """``use_zero_copy_grad_bucket``: give every parameter a ``.grad`` that is a view of the unit's
        gradient bucket before autograd runs, so gradient accumulation writes the reduce-scatter input
        in place and no copy-in happens afterwards.  Needs the bucket in the parameters' dtype; the views
        start at zero unless gradients of earlier micro-batches are being accumulated.
        Parity: ``matrix_fsdp/runtime/flat_buffer.py:447-486,1208-1230``."""
        fb = self.flat_buffer
        if fb.bucket.dtype != fb.param_dtype:
            return                                   # reduce dtype differs: gradients have to be converted anyway
        buf = fb.prepare_grad_bucket()
        if not self.has_accumulated_grads:
            buf.zero_()
        self._zero_copy_grads = {}
        for mp in self.registry:
            view = buf[mp.offset:mp.end].view(mp.shape)
            mp.param.grad = view
            self._zero_copy_grads[mp.fqn] = view
        self._record("attach_zero_copy_grads")

    def grad_target(self, fqn: str) -> tuple[torch.Tensor, bool]:
        """Bucket view an op may write this parameter's gradient into, and whether to accumulate."""
        mp = self.registry.param(fqn)
        self.flat_buffer.prepare_grad_bucket()
        view = self.flat_buffer.bucket.buffer[mp.offset:mp.end].view(mp.shape)
        accumulate = self.has_accumulated_grads or fqn in self._direct_written
        return view, accumulate

    def mark_grad_written(self, fqn: str) -> None:
        """An op wrote (or accumulated) this parameter's gradient straight into the bucket."""
        self._direct_written.add(fqn)
        self._on_grad(fqn)

    def _queue_backward_callback(self) -> None:
        if self._backward_callback_queued:
            return
        try:
            torch.autograd.Variable._execution_engine.queue_callback(self._end_of_backward)
            self._backward_callback_queued = True
        except Exception:  # not inside a backward pass
            self._backward_callback_queued = False

    def _make_grad_hook(self, fqn: str):
        def hook(param):
            self._on_grad(fqn)
        return hook

    def _on_grad(self, fqn: str) -> None:
        if self.state != FSDPLifecycleState.UNSHARDED:
            return
        self._grads_seen.add(fqn)
        if len(self._grads_seen) >= len(self.registry) and self.finalize_after_backward:
            self.finalize_backward("all_grads_ready")

    def _end_of_backward(self) -> None:
        self._backward_callback_queued = False
        if self.state == FSDPLifecycleState.UNSHARDED and self._pre_backward_done:
            self.finalize_backward("end_of_backward")
        elif self.state == FSDPLifecycleState.FORWARD_RESHARDED:
            # forward ran but no gradient reached this unit's outputs
            self._transition(FSDPLifecycleState.SHARDED)
            self.forward_count_since_backward = 0

    def finalize_backward(self, reason: str = "manual") -> None:
        if self.state != FSDPLifecycleState.UNSHARDED:
            return
        t0 = time.perf_counter()
        fb = self.flat_buffer
        if self._zero_copy_grads:
            for mp in self.registry:
                view = self._zero_copy_grads.get(mp.fqn)
                g = mp.param.grad
                if view is not None and g is not None and g.data_ptr() == view.data_ptr():
                    self._direct_written.add(mp.fqn)     # autograd accumulated into the bucket in place
            self._zero_copy_grads = {}
        any_grad = bool(self._direct_written) or any(mp.param.grad is not None for mp in self.registry)
        how = None
        if any_grad or self.has_accumulated_grads:
            how = fb.collect_param_grads(accumulate=self.has_accumulated_grads, written_direct=self._direct_written)
        self.reshard("reshard_after_backward", to=FSDPLifecycleState.SHARDED,
                     keep_storage=not self.shrink_full_param_storage_after_backward)
        self._grads_seen.clear()
        self._direct_written = set()
        self._pre_backward_done = False
        self.forward_count_since_backward = 0
        self.finalized_after_backward = True
        # a graph that is kept (``retain_graph=True``, two losses over one forward) can be walked again: its
        # output hooks have to gather the parameters again, and the gradients of that pass add to this one's
        for r in self._backward_contexts:
            ctx = r()
            if ctx is not None:
                ctx.reset()
        self._record("finalize_backward", start=t0, reason=reason, extra={"copy_in": how})
        if not (any_grad or self.has_accumulated_grads):
            return
        if self.defer_backward_reduce:
            self.has_accumulated_grads = True
            self._record("defer_backward_reduce")
            return
        self._start_reduce()

    def _start_reduce(self) -> None:
        t0 = time.perf_counter()
        if self.scheduler is not None:
            self.scheduler.before_backward_reduce(self)
        if self.backward_reduce_strategy == "per_param_allreduce":
            h = self._reduce_by_allreduce()
        else:
            with nvtx_range(f"mfsdp.reduce_scatter:{self.name}"):
                h = self.flat_buffer.start_reduce_grad_bucket_to_local_shard(
                    stream=self.reduce_scatter_stream, strategy=self.backward_reduce_strategy)
        self.has_accumulated_grads = False
        if getattr(h, "span", None) is not None:
            h.span.unit, h.span.reason = self.name, "post_backward"
        self._record("start_reduce_scatter", start=t0, handle=h)
        if self.scheduler is not None:
            self.scheduler.after_backward_reduce_started(self)
        else:
            self.wait_post_backward_reduce()

    def _reduce_by_allreduce(self):
        """Diagnostic strategy: all-reduce the whole bucket, then keep the owned slice."""
        from .collectives import MatrixCollectiveHandle, gather_local_segments

        fb = self.flat_buffer
        buf = fb.bucket.ensure()
        fb.transport.all_reduce(buf, self.groups.shard_group)
        if self.replicate_world_size > 1:
            fb.transport.all_reduce(buf, self.groups.replicate_group)
        out = fb._ensure_local_grad_shard()
        tmp = torch.empty(fb.local_numel, dtype=buf.dtype, device=buf.device)
        gather_local_segments(buf, tmp, fb.tables.my_segments)
        out.copy_(tmp)
        out.mul_(fb.grad_scale())
        h = MatrixCollectiveHandle(info={"kind": "all_reduce", "impl": "per_param_allreduce", "backend": fb.transport.kind,
                                         "bytes": buf.numel() * buf.element_size(), "count": 1, "sync_mode": "blocking"})
        fb.pending_reduce = h
        fb.local_grad_valid = True
        return h

    def wait_post_backward_reduce(self) -> None:
        fb = self.flat_buffer
        if fb.pending_reduce is None:
            return
        t0 = time.perf_counter()
        h = fb.wait_reduce()
        fb.release_grad_bucket()
        fb.use_local_grad_shard()
        self._record("wait_reduce_scatter", start=t0, handle=h)

    def flush_deferred_reduce(self) -> None:
        """Reduce gradients accumulated under ``no_sync`` (used when stepping after accumulation)."""
        if self.has_accumulated_grads and self.state == FSDPLifecycleState.SHARDED:
            self._start_reduce()

    # ------------------------------------------------------------------ optimizer interplay
    def assert_optimizer_ready(self) -> None:
        if self.in_no_sync:
            raise RuntimeError(f"{self.name}: optimizer step / zero_grad inside no_sync() is not allowed.")
        if self.state != FSDPLifecycleState.SHARDED:
            raise RuntimeError(f"{self.name}: optimizer step needs every unit SHARDED, found {self.state.value}.")
        if self.flat_buffer.pending_reduce is not None or self.flat_buffer.pending_gather is not None:
            raise RuntimeError(f"{self.name}: collectives still in flight at optimizer step.")

    def prepare_for_optimizer_step(self) -> None:
        if self.in_no_sync:
            raise RuntimeError(f"{self.name}: optimizer step / zero_grad inside no_sync() is not allowed.")
        if self.state == FSDPLifecycleState.UNSHARDED and self._pre_backward_done:
            self.finalize_backward("optimizer_step_straggler")
        elif self.state == FSDPLifecycleState.FORWARD_RESHARDED:
            self._transition(FSDPLifecycleState.SHARDED)
            self.forward_count_since_backward = 0
        elif self.state == FSDPLifecycleState.UNSHARDED:
            self.reshard("reshard_before_optimizer")
        self.discard_unused_prefetch()
        self.flush_deferred_reduce()
        self.wait_post_backward_reduce()
        fb = self.flat_buffer
        if fb.local_grad_valid and not fb.params_use_full and fb.pending_reduce is None:
            # reduced gradients that were taken off the parameters for a pass that then produced nothing (a forward
            # without a backward, an output that reaches no parameter) go back on: optimizers that read
            # ``param.grad`` must see what the flat ones read from the shard
            fb.use_local_grad_shard()
        self.used_in_forward = False

    def no_sync(self) -> MatrixFSDPNoSync:
        return MatrixFSDPNoSync([self])

    # ------------------------------------------------------------------ introspection
    @property
    def layout(self) -> MatrixGroupLayout:
        return self.planner_result.layout

    def owner_ranks(self, fqn: str) -> tuple[int, ...]:
        return self.layout.owner_ranks(fqn)

    def params_for_rank(self, rank: int | None = None) -> tuple[str, ...]:
        return self.layout.params_for_rank(self.rank if rank is None else rank)

    def rank_segments_for_param(self, fqn: str, rank: int | None = None):
        return self.layout.rank_segments_for_param(self.rank if rank is None else rank, fqn)

    def managed_params(self):
        return self.registry.params

    def state_dict(self) -> dict[str, Any]:
        """Debug dictionary of this unit's sharded state (metadata plus the local shard tensor)."""
        fb = self.flat_buffer
        return {
            "name": self.name, "rank": self.rank, "world_size": self.world_size,
            "replicate_rank": self.replicate_rank, "replicate_world_size": self.replicate_world_size,
            "state": self.state.value, "runtime_mode": self.runtime_mode, "total_numel": fb.total_numel,
            "shard_sizes": self.layout.shard_sizes,
            "local_segments": tuple((s.global_start, s.global_end, s.local_start) for s in fb.tables.my_segments),
            "param_fqns": self.registry.fqns, "param_shard": fb.local_shard,
            "planner": self.planner_result.name, "policy": self.planner_result.policy,
            "mp_policy": mixed_precision_policy_metadata(self.mp_policy),
            "offload_policy": offload_policy_metadata(self.offload_policy),
        }

    def full_param_storage_nbytes(self) -> int:
        return self.flat_buffer.full_storage_nbytes()
