"""Human- and machine-readable summaries of units, schedulers and runtime event logs.

Parity: ``matrix_fsdp/runtime/summary.py:1-893`` (``summarize_param_groups``,
``summarize_runtime_events``, the two formatters).
"""
from __future__ import annotations

from collections import defaultdict
from collections.abc import Iterable
from statistics import mean

from .param_buffers import describe_unit_param_buffer
from .runtime_event import RuntimeEvent
from .unit_collection import collect_param_groups

EVENT_CATEGORIES = {
    "unshard": ("start_unshard", "wait_unshard", "unshard"),
    "reshard": ("reshard",),
    "prefetch": ("forward_prefetch", "backward_prefetch", "discard_unused_prefetch"),
    "forward": ("pre_forward", "post_forward"),
    "backward": ("pre_backward", "finalize_backward", "defer_backward_reduce"),
    "reduce": ("start_reduce_scatter", "wait_reduce_scatter"),
    "init": ("init",),
}


def _category(name: str) -> str:
    base = name.split(":", 1)[0]
    for cat, prefixes in EVENT_CATEGORIES.items():
        if any(base.startswith(p) for p in prefixes):
            return cat
    return "other"


def summarize_param_groups(module_or_units) -> list[dict[str, object]]:
    """One dict per unit: planner, runtime mode, per-rank estimates, communication summary, memory."""
    out = []
    for u in collect_param_groups(module_or_units):
        fb, res = u.flat_buffer, u.planner_result
        desc = describe_unit_param_buffer(u)
        comm = desc.communication_summary(
            param_gather_strategy=u.param_gather_strategy, matrix_collective_backend=u.matrix_collective_backend,
            can_direct_all_gather=fb.tables.equal_contiguous, transport_kind=fb.transport.kind)
        est = res.resource_estimate
        out.append({
            "name": u.name, "rank": u.rank, "world_size": u.world_size,
            "replicate_world_size": u.replicate_world_size, "state": u.state.value,
            "planner_name": res.name, "planner_policy": res.policy, "runtime_mode": u.runtime_mode,
            "num_params": len(u.registry), "total_numel": fb.total_numel, "local_numel": fb.local_numel,
            "shard_sizes": res.layout.shard_sizes, "param_dtype": str(fb.param_dtype),
            "shard_dtype": str(fb.shard_dtype), "reduce_dtype": str(fb.reduce_dtype),
            "transport": fb.transport.kind,
            "transport_detail": fb.transport.describe() if hasattr(fb.transport, "describe") else fb.transport.kind,
            "full_buffer_mode": ("alias" if fb.full_aliases_shard else "persistent_slot" if fb.full_persistent
                                 else "pool" if fb.full_pool is not None else "storage_resize"),
            "grad_bucket_dtype": str(fb.bucket.dtype), "mixed_precision": fb.mixed,
            "fused_reduce_update": fb.fused_reduce_update is not None,
            "reshard_after_forward": u.reshard_after_forward, "forward_prefetch": u.forward_prefetch,
            "backward_prefetch": u.backward_prefetch, "backward_reduce_strategy": u.backward_reduce_strategy,
            "param_gather_strategy": u.param_gather_strategy, "matrix_collective_backend": u.matrix_collective_backend,
            "use_saved_tensor_hooks": u.use_saved_tensor_hooks, "use_zero_copy_grad_bucket": u.use_zero_copy_grad_bucket,
            "owned_params": len(fb.pieces), "max_shard_numel": fb.tables.max_shard,
            "communication": comm, "memory": fb.memory_snapshot(),
            "rank_memory_bytes": est.rank_memory_bytes if est else (), "rank_comm_bytes": est.rank_comm_bytes if est else (),
            "rank_ns_flops": est.rank_ns_flops if est else (), "planner_cost": res.cost, "warnings": res.warnings,
            "num_events": len(u.runtime_events),
            "scheduler": u.scheduler.summary() if u.scheduler is not None else None,
        })
    return out


def format_param_group_summary(module_or_units) -> str:
    rows = summarize_param_groups(module_or_units)
    if not rows:
        return "(no FSDP units)"
    lines = []
    for r in rows:
        comm = r["communication"]
        lines.append(
            f"{r['name']}: rank {r['rank']}/{r['world_size']} state={r['state']} planner={r['planner_name']}"
            f"({r['planner_policy']}) mode={r['runtime_mode']} params={r['num_params']} numel={r['total_numel']} "
            f"local={r['local_numel']} transport={r['transport']} gather={comm['effective_param_gather_backend']} "
            f"reduce={comm['effective_grad_reduce_backend']} pad_waste={comm['padding_waste_ratio']:.3f} "
            f"owner_imbalance={comm['owner_imbalance_ratio']:.3f}")
    sched = rows[0]["scheduler"]
    if sched:
        c = sched["counters"]
        lines.append(f"scheduler: units={sched['num_units']} fwd_prefetch={c['forward_prefetch_issued']} "
                     f"bwd_prefetch={c['backward_prefetch_issued']} reduce_waits={c['reduce_waits']} "
                     f"high_water_full_bytes={c['high_water_active_full_param_bytes']}")
    return "\n".join(lines)


def _stats(values: list[float]) -> dict[str, float]:
    if not values:
        return {"count": 0, "total_ms": 0.0, "mean_ms": 0.0, "max_ms": 0.0}
    return {"count": len(values), "total_ms": sum(values), "mean_ms": mean(values), "max_ms": max(values)}


# lifecycle phase of an event, from its name / reason (a step is forward, backward, optimizer boundary)
_PHASE_RULES = (
    ("optimizer", ("reshard_before_optimizer", "optimizer_step", "discard_unused_prefetch")),
    ("backward", ("pre_backward", "backward_prefetch", "finalize_backward", "reshard_after_backward",
                  "start_reduce_scatter", "wait_reduce_scatter", "defer_backward_reduce", "attach_zero_copy_grads",
                  "start_unshard:pre_backward", "wait_unshard:pre_backward", "start_unshard:backward_prefetch",
                  "start_unshard:post_reshard_prefetch", "pre_forward_recompute_skip", "post_forward_recompute_skip")),
    ("forward", ("pre_forward", "post_forward", "forward_prefetch", "reshard_after_forward",
                 "start_unshard:pre_forward", "wait_unshard:pre_forward", "start_unshard:forward_prefetch",
                 "start_unshard:next_step_prefetch", "enter_saved_tensor_hooks", "exit_saved_tensor_hooks")),
    ("init", ("init",)),
)


def _phase(event: RuntimeEvent) -> str:
    name = event.name
    for phase, prefixes in _PHASE_RULES:
        if any(name == p or name.startswith(p + ":") or name.startswith(p) for p in prefixes):
            return phase
    if name == "unshard":
        return "backward" if (event.reason or "").startswith(("pre_backward", "backward")) else "forward"
    return "other"


def _span_times(event: RuntimeEvent) -> tuple[float | None, float | None]:
    """(device ms, exposed ms) of the collective behind an event, when its CUDA events have completed."""
    span = event.extra.get("span") if isinstance(event.extra, dict) else None
    if span is None:
        return event.device_ms, None
    from .device_timeline import try_resolve_span

    if not try_resolve_span(span):
        return None, None
    return span.device_ms, span.exposed_ms


def summarize_scheduler(module_or_units) -> dict[str, object] | None:
    """Counters, limits and pool statistics of the scheduler that serves these units (None without one)."""
    units = collect_param_groups(module_or_units)
    sched = next((u.scheduler for u in units if u.scheduler is not None), None)
    if sched is None:
        return None
    s = sched.summary()
    cfg, ctr = s["config"], s["counters"]
    return {
        "num_units": s["num_units"], "prefetch_policy": cfg["prefetch_policy"],
        "forward_prefetch_depth": sched._fwd_budget(), "backward_prefetch_depth": sched._bwd_budget(),
        "backward_prefetch_timing": cfg["backward_prefetch_timing"],
        "max_pending_backward_reduces": cfg["max_pending_backward_reduces"],
        "counters": ctr, "pool": s["pool"],
        "prefetch_hit_ratio": (ctr["forward_prefetch_issued"] + ctr["backward_prefetch_issued"]
                               + ctr["next_step_prefetch_issued"]) / max(ctr["unshard_waits"] * 2, 1),
        "pending_reduces": s["pending_reduces"], "active_full_param_buffers": s["active_full_param_buffers"],
    }


def summarize_runtime_events(module_or_units_or_events) -> dict[str, object]:
    """Aggregate event logs per name, per category, per phase, per collective kind/impl and per unit; the
    collective rows also carry device time and exposed wait when the device timeline recorded them."""
    events: list[RuntimeEvent] = []
    if isinstance(module_or_units_or_events, Iterable) and not hasattr(module_or_units_or_events, "modules"):
        items = list(module_or_units_or_events)
        if items and isinstance(items[0], RuntimeEvent):
            events = items
        else:
            for u in collect_param_groups(items):
                events.extend(u.runtime_events)
    else:
        for u in collect_param_groups(module_or_units_or_events):
            events.extend(u.runtime_events)
    events.sort(key=lambda e: e.sequence)
    by_name, by_cat, by_unit = defaultdict(list), defaultdict(list), defaultdict(list)
    by_phase: dict[str, dict] = {}
    by_coll: dict[tuple, dict] = {}
    for e in events:
        by_name[e.name].append(e.duration_ms)
        by_cat[_category(e.name)].append(e.duration_ms)
        by_unit[e.unit].append(e.duration_ms)
        ph = by_phase.setdefault(_phase(e), {"count": 0, "host_ms": 0.0, "collectives": 0, "collective_bytes": 0,
                                             "device_ms": 0.0, "exposed_ms": 0.0})
        ph["count"] += 1
        ph["host_ms"] += e.duration_ms
        if e.collective_kind:
            key = (e.collective_kind, e.collective_backend, e.collective_impl)
            d = by_coll.setdefault(key, {"count": 0, "bytes": 0, "host_ms": 0.0, "collective_count": 0,
                                         "issue_host_ms": 0.0, "wait_host_ms": 0.0, "device_ms": 0.0,
                                         "exposed_ms": 0.0, "device_timed": 0, "prefetched": 0,
                                         "workspace_reused": 0, "max_bytes": 0})
            if e.name.startswith(("start_", "wait_")):
                d["host_ms"] += e.duration_ms
            if e.name.startswith("wait_"):
                d["wait_host_ms"] += e.duration_ms
                _, exposed = _span_times(e)
                if exposed is not None:
                    d["exposed_ms"] += exposed
                    ph["exposed_ms"] += exposed
            if e.name.startswith("start_"):
                d["count"] += 1
                d["bytes"] += e.collective_bytes
                d["max_bytes"] = max(d["max_bytes"], e.collective_bytes)
                d["collective_count"] += e.collective_count
                d["issue_host_ms"] += e.duration_ms
                for phase, ms in ((e.extra or {}).get("host_phases_ms") or {}).items():
                    d[f"host_{phase}_ms"] = d.get(f"host_{phase}_ms", 0.0) + float(ms)     # inside the collective call
                d["prefetched"] += int(e.prefetched)
                d["workspace_reused"] += int(e.workspace_reused)
                ph["collectives"] += 1
                ph["collective_bytes"] += e.collective_bytes
                dev, _ = _span_times(e)
                if dev is not None:
                    d["device_ms"] += dev
                    d["device_timed"] += 1
                    ph["device_ms"] += dev
    for d in by_coll.values():
        d["device_gbytes_per_s"] = (d["bytes"] * d["device_timed"] / max(d["count"], 1)) / d["device_ms"] / 1e6 \
            if d["device_ms"] > 0 else None
    return {
        "num_events": len(events),
        "by_name": {k: _stats(v) for k, v in by_name.items()},
        "by_category": {k: _stats(v) for k, v in by_cat.items()},
        "by_unit": {k: _stats(v) for k, v in by_unit.items()},
        "by_collective": {"/".join(str(x) for x in k): v for k, v in by_coll.items()},
        "by_phase": by_phase,
        "max_active_full_param_buffers": max((e.active_full_param_buffers for e in events), default=0),
        "max_pending_reduce_scatter": max((e.pending_reduce_scatter_count for e in events), default=0),
        "max_grad_bucket_bytes": max((e.grad_bucket_bytes for e in events), default=0),
        "prefetched_unshards": sum(1 for e in events if e.name == "unshard" and e.prefetched),
        "recompute_skips": sum(1 for e in events if e.recompute),
    }


def format_runtime_events(module_or_units_or_events, *, limit: int | None = None) -> str:
    s = summarize_runtime_events(module_or_units_or_events)
    lines = [f"runtime events: {s['num_events']}"]
    lines.append("by category:")
    for k, v in sorted(s["by_category"].items()):
        lines.append(f"  {k:10s} n={v['count']:5d} total={v['total_ms']:.3f}ms mean={v['mean_ms']:.4f}ms max={v['max_ms']:.3f}ms")
    lines.append("by name:")
    names = sorted(s["by_name"].items(), key=lambda kv: -kv[1]["total_ms"])
    for k, v in names[: limit or len(names)]:
        lines.append(f"  {k:34s} n={v['count']:5d} total={v['total_ms']:.3f}ms max={v['max_ms']:.3f}ms")
    if s["by_phase"]:
        lines.append("by phase:")
        for k, v in sorted(s["by_phase"].items()):
            lines.append(f"  {k:10s} events={v['count']:5d} host={v['host_ms']:.3f}ms collectives={v['collectives']} "
                         f"bytes={v['collective_bytes']} device={v['device_ms']:.3f}ms exposed={v['exposed_ms']:.3f}ms")
    if s["by_collective"]:
        lines.append("collectives:")
        for k, v in s["by_collective"].items():
            dev = f" device_ms={v['device_ms']:.3f} exposed_ms={v['exposed_ms']:.3f}" if v["device_timed"] else ""
            rate = f" {v['device_gbytes_per_s']:.1f}GB/s" if v.get("device_gbytes_per_s") else ""
            lines.append(f"  {k}: launches={v['count']} bytes={v['bytes']} issue_host_ms={v['issue_host_ms']:.3f} "
                         f"wait_host_ms={v['wait_host_ms']:.3f} prefetched={v['prefetched']}{dev}{rate}")
    lines.append(f"max_active_full_param_buffers={s['max_active_full_param_buffers']} "
                 f"max_pending_reduce_scatter={s['max_pending_reduce_scatter']} "
                 f"prefetched_unshards={s['prefetched_unshards']} recompute_skips={s['recompute_skips']}")
    return "\n".join(lines)
