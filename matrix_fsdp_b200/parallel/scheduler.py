"""Cross-unit scheduler: prefetch windows, in-flight caps, pending reduce queue, stream sharing.

One scheduler serves all units of a model.  It

* orders units (construction order = ``param_group_N`` id) and records the order in which their
  forwards *finish*, because backward prefetch walks that recorded order in reverse;
* issues forward prefetches (``max_forward_prefetch_units`` ahead, bounded by
  ``max_unsharded_prefetch_units`` and the active-full-buffer caps) and backward prefetches
  (at ``pre_backward`` or right after the previous unit resharded);
* bounds the number of reduce-scatters in flight (``max_pending_backward_reduces``) and drains
  them before the optimizer step;
* makes the all-gather stream wait for the optimizer's writes (post-optimizer event);
* shares one all-gather and one reduce-scatter stream across units and keeps counters.

Parity: ``matrix_fsdp/runtime/scheduler.py:28-1238``.  The ordered owner-prefetch queue and the
per-iteration barrier of the reference exist to keep NCCL point-to-point calls in the same
order on every rank (``scheduler.py:331-364,1019-1029``); the peer transport's pulls are
one-sided, so no cross-rank ordering is needed and neither mechanism exists here.
"""
from __future__ import annotations

import os
from dataclasses import asdict, dataclass, field
from enum import Enum

import torch
import torch.distributed as dist

from .buffer_pool import FullParamBufferPool

DEFAULT_MAX_UNSHARDED_PREFETCH_UNITS = 1


class BackwardPrefetchTiming(str, Enum):
    PRE_BACKWARD = "pre_backward"
    POST_RESHARD = "post_reshard"


class PrefetchPolicy(str, Enum):
    STATIC = "static"
    ADAPTIVE = "adaptive"
    PROFILE_GUIDED = "profile_guided"


@dataclass
class PrefetchProfileResult:
    forward_prefetch_units: int
    backward_prefetch_units: int
    samples: int
    mean_unshard_wait_ms: float


@dataclass
class MatrixFSDPSchedulerConfig:
    max_unsharded_prefetch_units: int = DEFAULT_MAX_UNSHARDED_PREFETCH_UNITS
    max_forward_prefetch_units: int | None = None
    max_backward_prefetch_units: int | None = None
    backward_prefetch_timing: str = "pre_backward"
    prefetch_policy: str = "static"
    max_cached_full_param_buffers_per_key: int = 2
    max_cached_workspaces_per_key: int = 1
    max_active_full_param_buffers: int | None = None
    max_active_full_param_numel: int | None = None
    max_active_full_param_memory_mb: float | None = None
    max_pending_backward_reduces: int = 1
    owner_backward_prefetch_with_pending_reduce: str = "auto"
    trim_cuda_cache: bool = False
    cuda_cache_trim_threshold_mb: float = 1024.0
    validate_unit_order: bool = False
    # after optimizer.step(): start the all-gather of the unit that ran first in the last forward, so the
    # next step does not begin with an exposed gather (None: on for CUDA, off on CPU)
    prefetch_first_unit_after_step: bool | None = None
    # how many units of the next forward are gathered right after the step.  More than one only happens for
    # units whose update was fused into their reduce-scatter: each of those gathers waits for its own unit's
    # update alone, so the gather of the second unit runs beside the reduce-scatter of the first (opposite
    # link directions) instead of after the whole optimizer step.
    next_step_prefetch_units: int = 2
    # the unit whose forward ran last in the previous iteration is not resharded after its forward (its
    # backward follows at once); None: on for CUDA with more than one unit, off on CPU
    keep_last_forward_unit_unsharded: bool | None = None
    # adaptive / profile_guided: exposed unshard wait (ms per unit) above which the prefetch depth grows,
    # and how many iterations each candidate depth is measured for
    adaptive_wait_threshold_ms: float = 0.05
    profile_iterations: int = 3

    def __post_init__(self) -> None:
        if self.max_unsharded_prefetch_units < 0:
            raise ValueError("max_unsharded_prefetch_units must be >= 0")
        BackwardPrefetchTiming(self.backward_prefetch_timing)
        PrefetchPolicy(self.prefetch_policy)
        if self.max_pending_backward_reduces < 0:
            raise ValueError("max_pending_backward_reduces must be >= 0")


SCHEDULER_KWARGS = tuple(MatrixFSDPSchedulerConfig.__dataclass_fields__) + (
    "scheduler_config", "max_cached_full_param_buffers_per_key", "max_cached_workspaces_per_key")

_POLICY_MAX_DEPTH = 2     # deepest prefetch the measuring policies try


@dataclass
class SchedulerCounters:
    forward_prefetch_issued: int = 0
    backward_prefetch_issued: int = 0
    prefetch_blocked_by_budget: int = 0
    prefetch_blocked_by_caps: int = 0
    prefetch_deferred_pending_reduce: int = 0
    unshard_waits: int = 0
    reduce_waits: int = 0
    post_optimizer_waits: int = 0
    high_water_active_full_param_buffers: int = 0
    high_water_active_full_param_bytes: int = 0
    iterations: int = 0
    cache_trims: int = 0
    next_step_prefetch_issued: int = 0
    policy_adjustments: int = 0
    mean_unshard_wait_us: int = 0

    def as_dict(self) -> dict[str, int]:
        return asdict(self)


@dataclass
class MatrixFSDPCommContext:
    """Streams and pools shared by every unit under one scheduler."""

    all_gather_stream: object = None
    reduce_scatter_stream: object = None
    full_param_pool: FullParamBufferPool = field(default_factory=FullParamBufferPool)


class MatrixFSDPScheduler:
    def __init__(self, units, config: MatrixFSDPSchedulerConfig | None = None, **overrides) -> None:
        cfg = config or MatrixFSDPSchedulerConfig()
        for k, v in overrides.items():
            if v is None and k not in ("max_forward_prefetch_units", "max_backward_prefetch_units"):
                continue
            if not hasattr(cfg, k):
                raise TypeError(f"Unknown scheduler option {k!r}.")
            setattr(cfg, k, v)
        cfg.__post_init__()
        self.config = cfg
        self.units = sorted(list(units), key=lambda u: u.metadata.runtime_param_group_id)
        if not self.units:
            raise ValueError("MatrixFSDPScheduler needs at least one unit.")
        self._index = {id(u): i for i, u in enumerate(self.units)}
        self.counters = SchedulerCounters()
        self.post_forward_order: list = []
        self.forward_order: list = []
        self._pre_forward_seen: list = []
        self._active: dict[int, object] = {}
        self._pending_reduces: list = []
        self._post_optimizer_event = None
        self._waited_post_optimizer: set[int] = set()
        self.comm = MatrixFSDPCommContext(full_param_pool=FullParamBufferPool(cfg.max_cached_full_param_buffers_per_key))
        first = self.units[0]
        self.comm.all_gather_stream = first.all_gather_stream
        self.comm.reduce_scatter_stream = first.reduce_scatter_stream
        for u in self.units:
            u.scheduler = self
            u.all_gather_stream = self.comm.all_gather_stream
            u.reduce_scatter_stream = self.comm.reduce_scatter_stream
            # units that take their unsharded buffer from a pool share this scheduler's one
            fb = getattr(u, "flat_buffer", None)
            if getattr(u, "use_saved_tensor_hooks", False) and hasattr(fb, "use_full_param_pool"):
                fb.use_full_param_pool(self.comm.full_param_pool)
        if cfg.validate_unit_order:
            self.validate_unit_order()
        # measuring prefetch policies: exposed waits of this iteration / of the one before (whose CUDA
        # events have certainly completed by the time they are read, so reading them never blocks)
        self._wait_samples: list[tuple] = []
        self._prev_wait_samples: list[tuple] = []
        self._profile: dict = {"depth": None, "iters": 0, "results": {}, "done": False}
        if cfg.prefetch_policy != "static" and self.units[0].flat_buffer.device.type == "cuda":
            from . import device_timeline

            if not device_timeline.enabled():
                device_timeline.enable(True, collect=False)

    # ------------------------------------------------------------------ limits
    def _fwd_budget(self) -> int:
        c = self.config
        n = c.max_unsharded_prefetch_units if c.max_forward_prefetch_units is None else c.max_forward_prefetch_units
        return min(n, c.max_unsharded_prefetch_units) if c.max_forward_prefetch_units is None else n

    def _bwd_budget(self) -> int:
        c = self.config
        return c.max_unsharded_prefetch_units if c.max_backward_prefetch_units is None else c.max_backward_prefetch_units

    def active_full_param_buffers(self) -> int:
        return len(self._active)

    def active_full_param_numel(self) -> int:
        return sum(u.flat_buffer.total_numel for u in self._active.values() if not u.flat_buffer.full_aliases_shard)

    def active_full_param_bytes(self) -> int:
        return sum(u.flat_buffer.total_numel * u.flat_buffer.full_buffer.element_size()
                   for u in self._active.values() if not u.flat_buffer.full_aliases_shard)

    def pending_reduce_count(self) -> int:
        return len(self._pending_reduces)

    def _caps_allow(self, unit) -> bool:
        c = self.config
        slot_free = getattr(unit.flat_buffer, "full_slot_available", None)
        if slot_free is not None and not slot_free():
            return False      # its full-parameter slot still holds another unit (persistent symmetric slots)
        if c.max_active_full_param_buffers is not None and len(self._active) + 1 > c.max_active_full_param_buffers:
            return False
        extra = 0 if unit.flat_buffer.full_aliases_shard else unit.flat_buffer.total_numel
        if c.max_active_full_param_numel is not None and self.active_full_param_numel() + extra > c.max_active_full_param_numel:
            return False
        if c.max_active_full_param_memory_mb is not None:
            nbytes = self.active_full_param_bytes() + extra * unit.flat_buffer.full_buffer.element_size()
            if nbytes > c.max_active_full_param_memory_mb * 2 ** 20:
                return False
        return True

    def note_unshard_started(self, unit) -> None:
        self._active[id(unit)] = unit
        ctr = self.counters
        ctr.high_water_active_full_param_buffers = max(ctr.high_water_active_full_param_buffers, len(self._active))
        ctr.high_water_active_full_param_bytes = max(ctr.high_water_active_full_param_bytes,
                                                     self.active_full_param_bytes())

    def note_resharded(self, unit) -> None:
        self._active.pop(id(unit), None)
        if self.config.backward_prefetch_timing == "post_reshard" and unit.finalized_after_backward is False \
                and unit._pre_backward_done:
            self._prefetch_backward(unit, reason="post_reshard_prefetch")

    # ------------------------------------------------------------------ forward
    def on_pre_forward(self, unit) -> None:
        self.counters.unshard_waits += 1
        if not unit.forward_prefetch:
            return
        if unit not in self._pre_forward_seen:
            self._pre_forward_seen.append(unit)
        # construction order on the first iteration, afterwards the order forwards actually ran in
        # (a root unit that wraps the blocks is built last but runs first)
        order = self.forward_order if (self.forward_order and unit in self.forward_order) else self.units
        i = order.index(unit)
        budget = self._fwd_budget()
        issued = 0
        for nxt in order[i + 1:]:
            if issued >= budget:
                if budget == 0:
                    self.counters.prefetch_blocked_by_budget += 1
                break
            if nxt.state.value != "sharded" or nxt.flat_buffer.pending_gather is not None:
                issued += 1 if nxt.flat_buffer.pending_gather is not None else 0
                continue
            if not self._caps_allow(nxt):
                self.counters.prefetch_blocked_by_caps += 1
                break
            nxt._record("forward_prefetch", reason=f"from={unit.name}")
            nxt.start_unshard("forward_prefetch")
            self.counters.forward_prefetch_issued += 1
            issued += 1

    def keeps_unsharded_into_backward(self, unit) -> bool:
        want = self.config.keep_last_forward_unit_unsharded
        if want is None:
            want = unit.flat_buffer.device.type == "cuda"
        return bool(want) and len(self.units) > 1 and bool(self.forward_order) and self.forward_order[-1] is unit

    def record_post_forward(self, unit) -> None:
        if torch.is_grad_enabled():
            if unit in self.post_forward_order:
                self.post_forward_order.remove(unit)
            self.post_forward_order.append(unit)

    # ------------------------------------------------------------------ backward
    def on_pre_backward(self, unit) -> None:
        if self.config.backward_prefetch_timing == "pre_backward":
            self._prefetch_backward(unit, reason="backward_prefetch")

    def _prefetch_backward(self, unit, *, reason: str) -> None:
        if not unit.backward_prefetch or unit not in self.post_forward_order:
            return
        pos = self.post_forward_order.index(unit)
        budget = self._bwd_budget()
        issued = 0
        for prev in reversed(self.post_forward_order[:pos]):
            if issued >= budget:
                break
            if prev.state.value != "forward_resharded" or prev.flat_buffer.pending_gather is not None:
                continue
            if self._pending_reduces and self.config.owner_backward_prefetch_with_pending_reduce == "never":
                self.counters.prefetch_deferred_pending_reduce += 1
                break
            if not self._caps_allow(prev):
                self.counters.prefetch_blocked_by_caps += 1
                break
            prev._record("backward_prefetch", reason=f"from={unit.name}")
            prev.start_unshard(reason)
            self.counters.backward_prefetch_issued += 1
            issued += 1

    def before_backward_reduce(self, unit) -> None:
        """Bound the reduce-scatters in flight before a new one starts."""
        limit = self.config.max_pending_backward_reduces
        while len(self._pending_reduces) > max(limit - 1, 0) and self._pending_reduces:
            oldest = self._pending_reduces.pop(0)
            self.counters.reduce_waits += 1
            oldest.wait_post_backward_reduce()

    def after_backward_reduce_started(self, unit) -> None:
        if self.config.max_pending_backward_reduces == 0:
            unit.wait_post_backward_reduce()
            return
        self._pending_reduces.append(unit)

    def drop_pending_reduce(self, unit) -> None:
        self._pending_reduces = [u for u in self._pending_reduces if u is not unit]

    def wait_pending_backward_reduce(self) -> None:
        while self._pending_reduces:
            u = self._pending_reduces.pop(0)
            self.counters.reduce_waits += 1
            u.wait_post_backward_reduce()

    # ------------------------------------------------------------------ optimizer boundary
    def prepare_optimizer_step(self) -> None:
        for u in self.units:
            if u.in_no_sync:
                raise RuntimeError(f"{u.name}: optimizer step / zero_grad inside no_sync() is not allowed.")
        self.wait_pending_backward_reduce()
        for u in self.units:
            u.prepare_for_optimizer_step()
        self.wait_pending_backward_reduce()
        for u in self.units:
            u.assert_optimizer_ready()
        self.finish_backward_iteration()

    def finish_backward_iteration(self) -> None:
        if self._pre_forward_seen:
            self.forward_order = list(self._pre_forward_seen)
        self._pre_forward_seen = []
        self.post_forward_order.clear()
        self.counters.iterations += 1
        self._apply_prefetch_policy()

    # ------------------------------------------------------------------ measuring prefetch policies
    def note_unshard_wait(self, unit, host_ms: float, span) -> None:
        """Called by a unit after it waited for its all-gather (``span``: device-timeline record or None)."""
        if self.config.prefetch_policy != "static":
            self._wait_samples.append((host_ms, span))

    def _mean_exposed_wait_ms(self, samples) -> float | None:
        vals = []
        for host_ms, span in samples:
            if span is None:
                vals.append(host_ms)            # blocking transports (CPU): the host wait is the exposed time
            elif span.wait_begin is not None and span.wait_end is not None and span.wait_end.query():
                vals.append(max(span.wait_begin.elapsed_time(span.wait_end), 0.0))
        return sum(vals) / len(vals) if vals else None

    def _apply_prefetch_policy(self) -> None:
        policy = self.config.prefetch_policy
        if policy == "static":
            return
        measured = self._mean_exposed_wait_ms(self._prev_wait_samples)
        self._prev_wait_samples, self._wait_samples = self._wait_samples, []
        if measured is None:
            return
        self.counters.mean_unshard_wait_us = int(measured * 1e3)
        if policy == "adaptive":
            before = (self._fwd_budget(), self._bwd_budget())
            self.adapt_prefetch(measured, threshold_ms=self.config.adaptive_wait_threshold_ms)
            if (self._fwd_budget(), self._bwd_budget()) != before:
                self.counters.policy_adjustments += 1
            return
        # profile_guided: measure each candidate depth for a few iterations, then keep the best
        prof = self._profile
        if prof["done"]:
            return
        if prof["depth"] is None:
            prof["depth"], prof["iters"] = max(self._fwd_budget(), 1), 0
            return
        prof["results"].setdefault(prof["depth"], []).append(measured)
        prof["iters"] += 1
        if prof["iters"] < max(self.config.profile_iterations, 1):
            return
        if prof["depth"] < _POLICY_MAX_DEPTH and self._depth_fits(prof["depth"] + 1):
            prof["depth"] += 1
            prof["iters"] = 0
            self.config.max_forward_prefetch_units = prof["depth"]
            self.config.max_backward_prefetch_units = prof["depth"]
            self.config.max_unsharded_prefetch_units = max(self.config.max_unsharded_prefetch_units, prof["depth"])
            return
        means = {d: sum(v) / len(v) for d, v in prof["results"].items()}
        # the shallowest depth within 10 % (or 10 us) of the best: deeper prefetch costs memory
        best = min(means.values())
        pick = min(d for d, m in means.items() if m <= best * 1.1 + 0.01)
        self.tune_prefetch(PrefetchProfileResult(pick, pick, sum(len(v) for v in prof["results"].values()), means[pick]))
        prof["done"] = True
        self.counters.policy_adjustments += 1

    def _depth_fits(self, depth: int) -> bool:
        """Persistent full-parameter slots bound how many units can be unsharded at once."""
        for u in self.units:
            per_class = getattr(u.flat_buffer.transport, "full_slots_per_class", None)
            if getattr(u.flat_buffer, "full_persistent", False) and per_class is not None and depth + 1 > per_class:
                return False
        return True

    def record_post_optimizer_event(self) -> None:
        dev = self.units[0].flat_buffer.device
        if dev.type == "cuda":
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(dev))
            self._post_optimizer_event = ev
            self._waited_post_optimizer.clear()
        self.maybe_trim_cuda_cache()
        self._prefetch_for_next_step()

    def _prefetch_for_next_step(self) -> None:
        """The parameters are final once the optimizer has run: gather the unit that opens the next
        forward now, behind whatever the host does between two steps."""
        want = self.config.prefetch_first_unit_after_step
        dev = self.units[0].flat_buffer.device
        if want is None:
            want = dev.type == "cuda"
        if not want or not self.forward_order or self._fwd_budget() <= 0:
            return

        def ready(u) -> bool:
            return u.forward_prefetch and u.state.value == "sharded" and u.flat_buffer.pending_gather is None \
                and self._caps_allow(u)

        head = self.forward_order[:max(int(self.config.next_step_prefetch_units), 1)]
        own_events = [getattr(u.flat_buffer, "update_done_event", None) for u in head]
        if len(head) > 1 and all(ev is not None for ev in own_events):
            # in the order their updates finish (the reverse of the forward order): every gather starts as
            # soon as its own unit is final
            for u, ev in reversed(list(zip(head, own_events))):
                if ready(u):
                    u._record("forward_prefetch", reason="after_unit_update")
                    u.start_unshard("next_step_prefetch", after_event=ev)
                    self.counters.next_step_prefetch_issued += 1
            return
        first = head[0]
        if not ready(first):
            return
        first._record("forward_prefetch", reason="after_optimizer_step")
        first.start_unshard("next_step_prefetch")
        self.counters.next_step_prefetch_issued += 1

    def wait_for_post_optimizer_event_before_all_gather(self, unit) -> None:
        ev = self._post_optimizer_event
        if ev is None or self.comm.all_gather_stream is None:
            return
        if 0 not in self._waited_post_optimizer:
            self.comm.all_gather_stream.wait_event(ev)
            self._waited_post_optimizer.add(0)
            self.counters.post_optimizer_waits += 1

    def maybe_trim_cuda_cache(self) -> None:
        c = self.config
        if not c.trim_cuda_cache or not torch.cuda.is_available():
            return
        reserved = torch.cuda.memory_reserved()
        allocated = torch.cuda.memory_allocated()
        if (reserved - allocated) > c.cuda_cache_trim_threshold_mb * 2 ** 20:
            torch.cuda.empty_cache()
            self.counters.cache_trims += 1

    # ------------------------------------------------------------------ policies / diagnostics
    def tune_prefetch(self, result: PrefetchProfileResult) -> None:
        """Apply a profile-guided prefetch depth (``prefetch_policy="profile_guided"``)."""
        self.config.max_forward_prefetch_units = result.forward_prefetch_units
        self.config.max_backward_prefetch_units = result.backward_prefetch_units

    def adapt_prefetch(self, mean_unshard_wait_ms: float, *, threshold_ms: float = 0.05) -> None:
        """``prefetch_policy="adaptive"``: deepen prefetch while waits are visible, within the budget.
        Called by the scheduler itself at the end of every iteration with the measured mean exposed wait."""
        if self.config.prefetch_policy != "adaptive":
            return
        cur = self._fwd_budget()
        if mean_unshard_wait_ms > threshold_ms and cur < max(_POLICY_MAX_DEPTH, self.config.max_unsharded_prefetch_units) \
                and self._depth_fits(cur + 1):
            self.config.max_forward_prefetch_units = cur + 1
            self.config.max_backward_prefetch_units = self._bwd_budget() + 1
            self.config.max_unsharded_prefetch_units = max(self.config.max_unsharded_prefetch_units, cur + 1)

    def validate_unit_order(self) -> None:
        """All ranks must have built the same units in the same order."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return
        sig = tuple((u.name, u.flat_buffer.total_numel) for u in self.units)
        sigs: list = [None] * dist.get_world_size()
        dist.all_gather_object(sigs, sig)
        if any(s != sig for s in sigs):
            raise RuntimeError(f"FSDP unit order differs across ranks: {sigs}")

    def summary(self) -> dict[str, object]:
        return {"num_units": len(self.units), "config": asdict(self.config), "counters": self.counters.as_dict(),
                "pool": self.comm.full_param_pool.stats.as_dict(), "pending_reduces": len(self._pending_reduces),
                "active_full_param_buffers": len(self._active)}
