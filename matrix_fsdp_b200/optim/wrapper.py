"""Optimizer construction and lifecycle glue for FSDP-managed models.

``configure_optimizer(model, kind, **kw)`` builds ``"adamw"`` / ``"sgd"`` (flat fused sharded
optimizers), ``"muon"`` or ``"mixed_muon_adamw"`` (Muon for whole 2-D matrices this rank owns,
AdamW for everything else), accepts scheduler options in the same call and installs the step
prologue: drain pending reduce-scatters, finalise stragglers, drop unused prefetches, require all
units SHARDED; and the epilogue: record the event the next all-gather waits on.

Any plain ``torch.optim.X(model.parameters())`` built *after* sharding also works: a global
optimizer step pre/post hook (``torch.optim.optimizer.register_optimizer_step_pre_hook``)
recognises FSDP-managed parameters and runs the same prologue/epilogue.  The reference gets
that behaviour by monkey-patching ``torch.optim.Optimizer.__init__`` process-wide
(``matrix_fsdp/optim/wrapper.py:271-322``).

Parity: ``matrix_fsdp/optim/wrapper.py:32-1260``.
"""
from __future__ import annotations

from collections.abc import Iterable, Mapping
from dataclasses import dataclass, field
from typing import Any

import torch
from torch import nn
from torch.optim import Optimizer

from ..core.managed_param import ManagedParam
from ..parallel.fsdp_unit import MatrixFSDPNoSync, MatrixFSDPParamGroup
from ..parallel.scheduler import MatrixFSDPScheduler, MatrixFSDPSchedulerConfig
from ..parallel.unit_collection import collect_param_groups
from .flat import FlatShardedAdamW, FlatShardedSGD
from .muon import DEFAULT_MUON_ADJUST_LR_FN, MatrixMuon
from .state import MatrixFSDPOptimizerStateManager

_SCHEDULER_KWARG_NAMES = set(MatrixFSDPSchedulerConfig.__dataclass_fields__) | {
    "scheduler_config", "max_cached_elastic_workspaces_per_key", "flat_adamw_state"}
_AUTO_PREPARE_INSTALLED = False
_AUTO_PREPARE_SUPPRESS = 0


@dataclass(frozen=True)
class MatrixOptimizerConfig:
    optimizer: str = "adamw"
    kwargs: Mapping[str, Any] = field(default_factory=dict)
    default_matrix_optimizer: str = "muon"
    default_other_optimizer: str = "adamw"


@dataclass(frozen=True)
class MatrixOptimizerParamGroupSummary:
    name: str
    optimizer_type: str
    fqns: tuple[str, ...]
    param_numel: int
    local_numel: int


@dataclass(frozen=True)
class ClassifiedMatrixOptimizerParams:
    muon_params: tuple[nn.Parameter, ...]
    adamw_params: tuple[nn.Parameter, ...]
    group_summaries: tuple[MatrixOptimizerParamGroupSummary, ...]
    muon_fqns: tuple[str, ...] = ()
    adamw_fqns: tuple[str, ...] = ()


# --------------------------------------------------------------------------- scheduler plumbing
def _split_scheduler_kwargs(kwargs: Mapping[str, Any]) -> tuple[dict[str, Any], dict[str, Any]]:
    sched = {k: v for k, v in kwargs.items() if k in _SCHEDULER_KWARG_NAMES}
    opt = {k: v for k, v in kwargs.items() if k not in _SCHEDULER_KWARG_NAMES}
    return sched, opt


def _normalize_param_groups(module_or_units) -> list[MatrixFSDPParamGroup]:
    units = collect_param_groups(module_or_units)
    if not units:
        raise ValueError("Expected a module wrapped by matrix_fully_shard().")
    return units


def _ensure_scheduler(units: list[MatrixFSDPParamGroup], scheduler_kwargs: Mapping[str, Any] | None = None):
    kw = dict(scheduler_kwargs or {})
    kw.pop("flat_adamw_state", None)
    if "max_cached_elastic_workspaces_per_key" in kw:
        kw["max_cached_workspaces_per_key"] = kw.pop("max_cached_elastic_workspaces_per_key")
    cfg = kw.pop("scheduler_config", None)
    if cfg is not None and kw:
        raise ValueError(f"Pass either scheduler_config or explicit scheduler kwargs, not both: {', '.join(sorted(kw))}.")
    existing = {id(u.scheduler): u.scheduler for u in units if u.scheduler is not None}
    if len(existing) == 1 and not kw and cfg is None:
        sched = next(iter(existing.values()))
        if len(sched.units) == len(units):
            return sched
    return MatrixFSDPScheduler(units, config=cfg, **kw)


def _units_of_optimizer(optimizer: Optimizer) -> list[MatrixFSDPParamGroup]:
    found: dict[int, MatrixFSDPParamGroup] = {}
    for g in optimizer.param_groups:
        for p in g["params"]:
            ref = getattr(p, "_mfsdp_unit_ref", None)
            unit = ref() if ref is not None else None
            if isinstance(unit, MatrixFSDPParamGroup):      # a unit of this package, not of one that shares the name
                found[id(unit)] = unit
    return sorted(found.values(), key=lambda u: u.metadata.runtime_param_group_id)


def _prepare_matrix_optimizer_step(units, scheduler: MatrixFSDPScheduler | None) -> None:
    if scheduler is not None:
        scheduler.prepare_optimizer_step()
        return
    for u in units:
        u.prepare_for_optimizer_step()
    for u in units:
        u.assert_optimizer_ready()


def _finish_matrix_optimizer_step(units, scheduler: MatrixFSDPScheduler | None) -> None:
    if scheduler is not None:
        scheduler.record_post_optimizer_event()


# --------------------------------------------------------------------------- auto prepare
def install_matrix_optimizer_auto_prepare() -> None:
    """Make any torch optimizer over FSDP-managed params run the lifecycle prologue/epilogue."""
    global _AUTO_PREPARE_INSTALLED
    if _AUTO_PREPARE_INSTALLED:
        return
    from torch.optim.optimizer import register_optimizer_step_post_hook, register_optimizer_step_pre_hook

    def pre(optimizer, args, kwargs):
        if _AUTO_PREPARE_SUPPRESS or getattr(optimizer, "_mfsdp_lifecycle_managed", False):
            return None
        units = getattr(optimizer, "_mfsdp_units", None)
        if units is None:
            units = _units_of_optimizer(optimizer)
            optimizer._mfsdp_units = units
            if units:
                optimizer._mfsdp_scheduler = _ensure_scheduler(units)
        if units:
            _prepare_matrix_optimizer_step(units, getattr(optimizer, "_mfsdp_scheduler", None))
        return None

    def post(optimizer, args, kwargs):
        if _AUTO_PREPARE_SUPPRESS or getattr(optimizer, "_mfsdp_lifecycle_managed", False):
            return None
        units = getattr(optimizer, "_mfsdp_units", None)
        if units:
            for u in units:
                u.flat_buffer.mark_master_updated(lp_written=False)
            sched = getattr(optimizer, "_mfsdp_scheduler", None)
            if sched is not None:
                sched.record_post_optimizer_event()
        return None

    register_optimizer_step_pre_hook(pre)
    register_optimizer_step_post_hook(post)
    _AUTO_PREPARE_INSTALLED = True


class _suppress_auto_prepare:
    def __enter__(self):
        global _AUTO_PREPARE_SUPPRESS
        _AUTO_PREPARE_SUPPRESS += 1

    def __exit__(self, *exc):
        global _AUTO_PREPARE_SUPPRESS
        _AUTO_PREPARE_SUPPRESS -= 1
        return False


# --------------------------------------------------------------------------- wrappers
class MatrixFSDPOptimizer:
    """A torch optimizer plus the FSDP lifecycle around ``step()`` / ``zero_grad()``."""

    def __init__(self, optimizer: Optimizer, units, scheduler: MatrixFSDPScheduler | None = None,
                 **scheduler_kwargs) -> None:
        """``units``: a sharded module, one unit or a list of units (matrix_fsdp/optim/wrapper.py takes the module
        too).  ``optimizer`` may be any element-wise torch optimizer built over ``model.parameters()``: while it
        steps, every parameter is its local shard and ``.grad`` the matching piece of the reduced gradient."""
        self.optimizer = optimizer
        self.fsdp_param_groups = _normalize_param_groups(units)
        sched_kw, extra = _split_scheduler_kwargs(scheduler_kwargs)
        if extra:
            raise TypeError(f"Unknown optimizer wrapper options: {', '.join(sorted(extra))}.")
        self.scheduler = scheduler if scheduler is not None else _ensure_scheduler(self.fsdp_param_groups, sched_kw)
        optimizer._mfsdp_lifecycle_managed = True
        self.state_manager = MatrixFSDPOptimizerStateManager(self.fsdp_param_groups, {"optimizer": optimizer})

    # torch.optim.Optimizer surface
    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def state_dict(self):
        return self.optimizer.state_dict()

    def load_state_dict(self, sd) -> None:
        self.optimizer.load_state_dict(sd)

    def add_param_group(self, group) -> None:
        self.optimizer.add_param_group(group)

    def iter_named_optimizers(self):
        yield "optimizer", self.optimizer

    def step(self, closure=None):
        if closure is not None:
            raise NotImplementedError("Optimizer closures are not supported with sharded parameters.")
        _prepare_matrix_optimizer_step(self.fsdp_param_groups, self.scheduler)
        for u in self.fsdp_param_groups:
            # fused kernels that emit the low-precision copy clear this again
            u.flat_buffer.mark_master_updated(lp_written=False)
        with _suppress_auto_prepare():
            out = self.optimizer.step()
        _finish_matrix_optimizer_step(self.fsdp_param_groups, self.scheduler)
        return out

    def zero_grad(self, set_to_none: bool = True) -> None:
        for u in self.fsdp_param_groups:
            if u.in_no_sync:
                raise RuntimeError("zero_grad() cannot run inside no_sync().")
        self.optimizer.zero_grad(set_to_none=set_to_none)
        for u in self.fsdp_param_groups:
            u.has_accumulated_grads = False
            u.flat_buffer.accumulate_into_local_grad = False
            u.flat_buffer.bucket.accumulating = False
            u.flat_buffer.clear_local_grad_shard()

    def no_sync(self) -> MatrixFSDPNoSync:
        return MatrixFSDPNoSync(self.fsdp_param_groups)

    def local_state_summary(self):
        return self.state_manager.summary()

    def optimizer_group_summary(self) -> tuple[MatrixOptimizerParamGroupSummary, ...]:
        out = []
        for i, g in enumerate(self.optimizer.param_groups):
            fqns, numel, local = [], 0, 0
            for p in g["params"]:
                fqns.append(getattr(p, "_matrix_fsdp_fqn", "<unmanaged>"))
                local += p.numel()
                ref = getattr(p, "_mfsdp_unit_ref", None)
                unit = ref() if ref else None
                numel += unit.registry.param(p._matrix_fsdp_fqn).numel if unit is not None else p.numel()
            out.append(MatrixOptimizerParamGroupSummary(f"group_{i}", type(self.optimizer).__name__.lower(), tuple(fqns),
                                                        numel, local))
        return tuple(out)

    def __getattr__(self, name):
        return getattr(self.__dict__["optimizer"], name)


PreparedMatrixOptimizer = MatrixFSDPOptimizer


def prepare_matrix_optimizer(optimizer: Optimizer, module_or_units=None, **scheduler_kwargs) -> MatrixFSDPOptimizer:
    """Attach lifecycle handling (and scheduler options) to an existing torch optimizer."""
    units = _normalize_param_groups(module_or_units) if module_or_units is not None else _units_of_optimizer(optimizer)
    if not units:
        raise ValueError("The optimizer holds no FSDP-managed parameters.")
    sched, _ = _split_scheduler_kwargs(scheduler_kwargs)
    return MatrixFSDPOptimizer(optimizer, units, _ensure_scheduler(units, sched))


# --------------------------------------------------------------------------- Muon / AdamW split
def _optimizer_type_for_param(mp: ManagedParam, local: torch.Tensor, *, default_matrix_optimizer: str,
                              default_other_optimizer: str) -> str:
    kind = mp.shard_hint.optimizer_type
    if kind == "muon":
        if len(mp.shape) != 2 or local.ndim != 2 or local.numel() != mp.numel:
            raise ValueError(
                f"Param {mp.fqn!r} is marked for Muon, but its local view is not a full 2D matrix. "
                "Use matrix_owner planning for Muon parameters.")
        return "muon"
    if kind == "adamw":
        return "adamw"
    if len(mp.shape) == 2 and local.ndim == 2 and local.numel() == mp.numel:
        return default_matrix_optimizer
    return default_other_optimizer


def classify_matrix_optimizer_params(module_or_units, *, default_matrix_optimizer: str = "muon",
                                     default_other_optimizer: str = "adamw") -> ClassifiedMatrixOptimizerParams:
    """Split the parameters this rank owns into Muon and AdamW sets (hint first, 2-D ⇒ Muon fallback)."""
    units = _normalize_param_groups(module_or_units)
    muon, adamw, summaries = [], [], []
    muon_fqns, adamw_fqns = [], []
    for u in units:
        views = u.flat_buffer.local_param_views()
        m_entries, a_entries = [], []
        for mp in u.registry:
            local = views[mp.fqn]
            if local.numel() == 0:
                continue
            kind = _optimizer_type_for_param(mp, local, default_matrix_optimizer=default_matrix_optimizer,
                                             default_other_optimizer=default_other_optimizer)
            (m_entries if kind == "muon" else a_entries).append((mp, local))
        for name, entries, bucket, fq in (("muon", m_entries, muon, muon_fqns), ("adamw", a_entries, adamw, adamw_fqns)):
            bucket += [mp.param for mp, _ in entries]
            fq += [f"{u.name}.{mp.fqn}" for mp, _ in entries]
            if entries:
                summaries.append(MatrixOptimizerParamGroupSummary(
                    f"{u.name}.{name}", name, tuple(mp.fqn for mp, _ in entries),
                    sum(mp.numel for mp, _ in entries), sum(v.numel() for _, v in entries)))
    return ClassifiedMatrixOptimizerParams(tuple(muon), tuple(adamw), tuple(summaries), tuple(muon_fqns),
                                           tuple(adamw_fqns))


def _common_replicate_group(units):
    """The replicate process group when every unit is hybrid-sharded over the same one, else ``None``.  Replicas
    then own the same matrices with the same reduced gradients, which is what sharing Newton-Schulz needs."""
    groups = {id(u.flat_buffer.replicate_group): u.flat_buffer.replicate_group for u in units
              if u.flat_buffer.replicate_world_size > 1}
    if len(groups) != 1 or any(u.flat_buffer.replicate_world_size <= 1 for u in units):
        return None
    return next(iter(groups.values()))


class MixedMuonAdamWOptimizer:
    """Muon on owned whole matrices + AdamW on the rest, behind one optimizer-like object."""

    def __init__(self, muon_params, adamw_params, *, group_summaries=(), fsdp_param_groups=None, lr: float = 1e-3,
                 weight_decay: float = 0.01, muon_lr: float | None = None, adamw_lr: float | None = None,
                 adamw_betas=(0.9, 0.999), adamw_eps: float = 1e-8, adamw_weight_decay: float | None = None,
                 adamw_foreach: bool | None = None, muon_weight_decay: float | None = None,
                 muon_momentum: float = 0.5, muon_ns_steps: int = 2, muon_nesterov: bool = True,
                 muon_ns_coefficients=None, muon_adjust_lr_fn: str | None = DEFAULT_MUON_ADJUST_LR_FN,
                 lazy_muon_init: bool = True, muon_share_ns_across_replicas: bool = True,
                 **scheduler_kwargs) -> None:
        sched_kw, extra = _split_scheduler_kwargs(scheduler_kwargs)
        if extra:
            raise TypeError(f"Unknown mixed optimizer options: {', '.join(sorted(extra))}.")
        self.fsdp_param_groups = list(fsdp_param_groups or [])
        self.group_summaries = tuple(group_summaries)
        muon_params, adamw_params = list(muon_params), list(adamw_params)
        units = self.fsdp_param_groups
        lp_of = _low_precision_lookup(units)
        muon_kw = dict(lr=lr if muon_lr is None else muon_lr,
                       weight_decay=weight_decay if muon_weight_decay is None else muon_weight_decay,
                       momentum=muon_momentum, nesterov=muon_nesterov, ns_steps=muon_ns_steps,
                       adjust_lr_fn=muon_adjust_lr_fn)
        if muon_ns_coefficients is not None:
            muon_kw["ns_coefficients"] = tuple(muon_ns_coefficients)
        with _suppress_auto_prepare():
            # a rank that owns no matrix still gets a real (empty) Muon optimizer: LR schedulers and state-dict code
            # written against ``opt.muon`` then run unchanged on every rank
            self.muon = MatrixMuon(muon_params or [torch.nn.Parameter(torch.zeros(0, 0), requires_grad=False)],
                                   low_precision_of=lp_of, **muon_kw)
            self.adamw = FlatShardedAdamW(
                adamw_params or [torch.nn.Parameter(torch.zeros(0))], units=None,
                lr=lr if adamw_lr is None else adamw_lr, betas=adamw_betas, eps=adamw_eps,
                weight_decay=weight_decay if adamw_weight_decay is None else adamw_weight_decay)
        self.adamw._low_precision_of = lp_of
        if muon_share_ns_across_replicas and isinstance(self.muon, MatrixMuon):
            self.muon.share_newton_schulz_over(_common_replicate_group(units))
        for opt in (self.muon, self.adamw):
            if isinstance(opt, Optimizer):
                opt._mfsdp_lifecycle_managed = True
        self.scheduler = _ensure_scheduler(units, sched_kw) if units else None
        self.state_manager = MatrixFSDPOptimizerStateManager(units, dict(self.iter_named_optimizers()))

    def iter_named_optimizers(self):
        yield "muon", self.muon
        yield "adamw", self.adamw

    @property
    def param_groups(self):
        return list(self.muon.param_groups) + list(self.adamw.param_groups)

    @property
    def state(self):
        merged = dict(self.muon.state)
        merged.update(self.adamw.state)
        return merged

    def step(self, closure=None):
        if closure is not None:
            raise NotImplementedError("Optimizer closures are not supported with sharded parameters.")
        _prepare_matrix_optimizer_step(self.fsdp_param_groups, self.scheduler)
        with _suppress_auto_prepare():
            self.muon.step()
            self.adamw.step()
            lp_of = getattr(self.adamw, "_low_precision_of", None)
            if lp_of is not None:
                for g in self.adamw.param_groups:
                    for p in g["params"]:
                        if p.grad is not None and p.numel():
                            lp = lp_of(p)
                            if lp is not None:
                                lp.copy_(p.data)
        for u in self.fsdp_param_groups:
            u.flat_buffer.lp_stale = False
        if self.scheduler is not None:
            self.scheduler.record_post_optimizer_event()

    def zero_grad(self, set_to_none: bool = True) -> None:
        for u in self.fsdp_param_groups:
            if u.in_no_sync:
                raise RuntimeError("zero_grad() cannot run inside no_sync().")
        self.muon.zero_grad(set_to_none=set_to_none)
        self.adamw.zero_grad(set_to_none=set_to_none)
        for u in self.fsdp_param_groups:
            u.has_accumulated_grads = False
            u.flat_buffer.accumulate_into_local_grad = False
            u.flat_buffer.clear_local_grad_shard()

    def state_dict(self) -> dict:
        return {"kind": "mixed_muon_adamw", "muon": self.muon.state_dict(), "adamw": self.adamw.state_dict()}

    def load_state_dict(self, sd: Mapping[str, Any]) -> None:
        known = {"muon", "adamw"}
        given = {k for k in sd if k != "kind"}
        if given - known:
            raise ValueError(f"unknown component(s) in mixed optimizer state: {sorted(given - known)}")
        if known - given:
            raise ValueError(f"missing component(s) in mixed optimizer state: {sorted(known - given)}")
        self.muon.load_state_dict(sd["muon"])
        self.adamw.load_state_dict(sd["adamw"])

    def no_sync(self) -> MatrixFSDPNoSync:
        return MatrixFSDPNoSync(self.fsdp_param_groups)

    def local_state_summary(self):
        return self.state_manager.summary()

    def optimizer_group_summary(self) -> tuple[MatrixOptimizerParamGroupSummary, ...]:
        return self.group_summaries


def _low_precision_lookup(units):
    """param -> view of the unit's low-precision shard covering that param (or None)."""
    table: dict[int, tuple] = {}
    for u in units:
        fb = u.flat_buffer
        if fb.local_shard_lp is None:
            continue
        for mp in u.registry:
            piece = fb.pieces.get(mp.fqn)
            if piece is not None:
                table[id(mp.param)] = (fb, piece)

    def lookup(p):
        hit = table.get(id(p))
        if hit is None:
            return None
        fb, piece = hit
        return fb.local_shard_lp[piece.local_start:piece.local_end].view(piece.shape)

    return lookup


def make_mixed_muon_adamw_optimizer(module_or_units, *, default_matrix_optimizer: str = "muon",
                                    default_other_optimizer: str = "adamw", manage_matrix_lifecycle: bool = True,
                                    **optimizer_kwargs) -> MixedMuonAdamWOptimizer:
    units = _normalize_param_groups(module_or_units)
    classified = classify_matrix_optimizer_params(units, default_matrix_optimizer=default_matrix_optimizer,
                                                  default_other_optimizer=default_other_optimizer)
    return MixedMuonAdamWOptimizer(classified.muon_params, classified.adamw_params,
                                   group_summaries=classified.group_summaries,
                                   fsdp_param_groups=units if manage_matrix_lifecycle else None, **optimizer_kwargs)


def _optimizer_params_from_module_or_units(module_or_units) -> tuple[nn.Parameter, ...]:
    if isinstance(module_or_units, nn.Module):
        # parameters that a unit was told to ignore belong to the upper stack (tensor / expert parallel owners)
        # and its optimizer; unmanaged parameters that nobody claimed are still stepped here
        ignored: set[int] = set()
        managed: set[int] = set()
        for u in _normalize_param_groups(module_or_units):
            ignored |= {id(p) for p in (u.ignored_params or ())}
            managed |= {id(mp.param) for mp in u.registry}
        return tuple(p for p in module_or_units.parameters() if id(p) in managed or id(p) not in ignored)
    seen, out = set(), []
    for u in _normalize_param_groups(module_or_units):
        for mp in u.registry:
            if id(mp.param) not in seen:
                seen.add(id(mp.param))
                out.append(mp.param)
    return tuple(out)


def configure_optimizer(module_or_units, optimizer: str | MatrixOptimizerConfig = "adamw", **kwargs):
    """Build an optimizer for an FSDP-managed module (see module docstring)."""
    install_matrix_optimizer_auto_prepare()
    default_matrix, default_other = "muon", "adamw"
    opt_kwargs: dict[str, Any] = {}
    if isinstance(optimizer, MatrixOptimizerConfig):
        kind = optimizer.optimizer
        opt_kwargs.update(dict(optimizer.kwargs))
        default_matrix, default_other = optimizer.default_matrix_optimizer, optimizer.default_other_optimizer
    else:
        kind = optimizer
    opt_kwargs.update(kwargs)
    default_matrix = opt_kwargs.pop("default_matrix_optimizer", default_matrix)
    default_other = opt_kwargs.pop("default_other_optimizer", default_other)
    sched_kw, opt_kwargs = _split_scheduler_kwargs(opt_kwargs)
    kind = kind.lower()
    if kind in ("mixed_muon_adamw", "muon_adamw", "mixed"):
        return make_mixed_muon_adamw_optimizer(module_or_units, default_matrix_optimizer=default_matrix,
                                               default_other_optimizer=default_other, **opt_kwargs, **sched_kw)
    units = collect_param_groups(module_or_units)
    params = _optimizer_params_from_module_or_units(module_or_units)
    with _suppress_auto_prepare():
        if kind == "adamw":
            opt_kwargs.pop("foreach", None)
            opt_kwargs.pop("fused", None)
            inner: Optimizer = FlatShardedAdamW(params, units=units, **opt_kwargs)
        elif kind == "sgd":
            inner = FlatShardedSGD(params, units=units, **opt_kwargs)
        elif kind == "muon":
            owned = [p for p in params if p.ndim == 2 and p.numel() > 0]
            if len(owned) != len([p for p in params if p.numel() > 0]):
                raise ValueError("Muon only supports 2D parameters; use 'mixed_muon_adamw' for models with "
                                 "norms, biases or embeddings.")
            share = opt_kwargs.pop("share_ns_across_replicas", True)
            inner = MatrixMuon(owned or [torch.nn.Parameter(torch.zeros(0, 0))],
                               low_precision_of=_low_precision_lookup(units), **opt_kwargs)
            if share and units:
                inner.share_newton_schulz_over(_common_replicate_group(units))
        else:
            raise ValueError("optimizer must be one of 'adamw', 'sgd', 'muon', or 'mixed_muon_adamw', "
                             f"got {kind!r}.")
    if not units:
        return inner
    return MatrixFSDPOptimizer(inner, units, _ensure_scheduler(units, sched_kw))


configure_matrix_optimizer = configure_optimizer
