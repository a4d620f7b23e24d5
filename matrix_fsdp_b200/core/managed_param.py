"""Registry of the parameters one FSDP unit manages, plus per-parameter shard hints.

Parity: ``matrix_fsdp/core/managed_param.py:16-205`` (hint fields, validation rules and
error wording).  Difference: tied parameters can be admitted once under their first FQN
(``allow_shared=True``) so a root unit can own a tied embedding / LM head; the default keeps
the reference's rejection.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping

import torch
from torch import nn


class ParamRuntimeKind:
    FSDP_GATHER = "fsdp_gather"
    EP_LOCAL_FSDP = "ep_local_fsdp"
    EXPERT_OWNER = "expert_owner"


_GRANULARITIES = (None, "parameter", "matrix_owner", "row_block", "block")
_RUNTIME_KINDS = (None, ParamRuntimeKind.FSDP_GATHER, ParamRuntimeKind.EP_LOCAL_FSDP, ParamRuntimeKind.EXPERT_OWNER)
_PARALLEL_ROLES = (None, "dense", "embedding", "norm", "router", "routed_expert", "shared_expert")


@dataclass(frozen=True)
class ParamShardHint:
    optimizer_type: str | None = None
    split_granularity: str | None = None
    block_shape: tuple[int, ...] | None = None
    runtime_kind: str | None = None
    parallel_role: str | None = None
    expert_id: int | None = None
    expert_group_id: str | None = None
    owner_rank: int | None = None
    owner_replica_ranks: tuple[int, ...] = ()


@dataclass
class ManagedParam:
    fqn: str
    param: nn.Parameter
    shape: torch.Size
    dtype: torch.dtype
    device: torch.device
    numel: int
    offset: int
    end: int
    shard_hint: ParamShardHint = field(default_factory=ParamShardHint)
    aliases: tuple[str, ...] = ()

    @property
    def local_name(self) -> str:
        return self.fqn.rsplit(".", 1)[-1]


@dataclass
class ManagedParamRegistry:
    params: tuple[ManagedParam, ...]
    _by_fqn: dict[str, ManagedParam] = field(init=False, repr=False)

    def __post_init__(self) -> None:
        self._by_fqn = {}
        for mp in self.params:
            if mp.fqn in self._by_fqn:
                raise ValueError(f"Duplicate managed parameter fqn: {mp.fqn}.")
            self._by_fqn[mp.fqn] = mp

    def __iter__(self):
        return iter(self.params)

    def __len__(self) -> int:
        return len(self.params)

    def __getitem__(self, index: int) -> ManagedParam:
        return self.params[index]

    @property
    def total_numel(self) -> int:
        return self.params[-1].end if self.params else 0

    @property
    def fqns(self) -> tuple[str, ...]:
        return tuple(mp.fqn for mp in self.params)

    def param(self, fqn: str) -> ManagedParam:
        try:
            return self._by_fqn[fqn]
        except KeyError:
            raise KeyError(f"Unknown managed parameter fqn: {fqn}") from None

    def as_list(self) -> list[ManagedParam]:
        return list(self.params)

    def reassign_offsets(self, order: list[str]) -> None:
        """Re-lay the flat space in ``order`` (used when a layout is packed rank-major)."""
        if sorted(order) != sorted(self.fqns):
            raise ValueError("reassign_offsets needs a permutation of the managed fqns")
        off = 0
        new = []
        for fqn in order:
            mp = self._by_fqn[fqn]
            mp.offset, mp.end = off, off + mp.numel
            off = mp.end
            new.append(mp)
        self.params = tuple(new)

    @classmethod
    def from_module(
        cls,
        module: nn.Module,
        *,
        shard_hints: Mapping[str, ParamShardHint] | None = None,
        ignored_params: set[nn.Parameter] | None = None,
        allow_shared: bool = False,
    ) -> "ManagedParamRegistry":
        """One walk over every (name, parameter) pair of the module, aliases included.  The first name a
        tensor shows up under becomes its FQN and fixes its place in the flat space; later names of the
        same tensor are aliases (rejected unless ``allow_shared``)."""
        skip = {id(p) for p in ignored_params or ()}
        slots: dict[int, _Slot] = {}
        for name, tensor in module.named_parameters(recurse=True, remove_duplicate=False):
            if id(tensor) in skip:
                continue
            slot = slots.get(id(tensor))
            if slot is None:
                slots[id(tensor)] = _Slot(name, tensor)
            else:
                slot.other_names.append(name)
        tied = [slot for slot in slots.values() if slot.other_names]
        if tied and not allow_shared:
            listing = "; ".join(",".join([slot.name, *slot.other_names]) for slot in tied)
            raise NotImplementedError(
                "MatrixFSDP does not support shared parameters yet. " f"Shared parameter aliases: {listing}."
            )
        wanted = dict(shard_hints or {})
        unclaimed = set(wanted)
        managed: list[ManagedParam] = []
        cursor = 0
        for slot in slots.values():                      # dicts keep first-seen order = registration order
            t = slot.tensor
            hint = wanted.get(slot.name, _NO_HINT)
            unclaimed.difference_update([slot.name, *slot.other_names])
            validate_param_shard_hint(slot.name, t.shape, t.numel(), hint)
            managed.append(ManagedParam(fqn=slot.name, param=t, shape=t.shape, dtype=t.dtype, device=t.device,
                                        numel=t.numel(), offset=cursor, end=cursor + t.numel(), shard_hint=hint,
                                        aliases=tuple(slot.other_names)))
            cursor += t.numel()
        if unclaimed:
            raise ValueError(f"Shard hints refer to unknown parameters: {', '.join(sorted(unclaimed))}.")
        return cls(tuple(managed))


class _Slot:
    """A distinct parameter tensor met during the module walk, with every name it goes by."""

    __slots__ = ("name", "tensor", "other_names")

    def __init__(self, name: str, tensor: nn.Parameter) -> None:
        self.name, self.tensor, self.other_names = name, tensor, []


_NO_HINT = ParamShardHint()


def _fmt(values) -> str:
    return ", ".join(repr(v) for v in sorted(values, key=str))


# ---------------------------------------------------------------------------- hint validation
# The checks are data: each rule is (applies?, broken?, message) over one context object, evaluated in
# table order; the first broken rule raises.  Rules that only make sense for one granularity carry that
# condition in their ``applies`` part, so there is no branching in the driver.
class _HintCheck:
    __slots__ = ("fqn", "shape", "numel", "h", "g", "bs", "rows", "cols")

    def __init__(self, fqn: str, shape, numel: int, hint: ParamShardHint) -> None:
        self.fqn, self.shape, self.numel, self.h = fqn, tuple(shape), int(numel), hint
        self.g, self.bs = hint.split_granularity, hint.block_shape
        self.rows, self.cols = (self.shape + (None, None))[:2] if len(self.shape) == 2 else (None, None)


def _member(attr: str, allowed) -> tuple:
    return (lambda c: True,
            lambda c: getattr(c.h, attr) not in allowed,
            lambda c: f"Param {c.fqn} has unknown {attr}={getattr(c.h, attr)!r}; expected {_fmt(allowed)}.")


def _non_negative(attr: str) -> tuple:
    return (lambda c: getattr(c.h, attr) is not None,
            lambda c: getattr(c.h, attr) < 0,
            lambda c: f"Param {c.fqn} {attr} must be non-negative, got {getattr(c.h, attr)}.")


_WHOLE = (None, "parameter", "matrix_owner")

_HINT_RULES: tuple[tuple, ...] = (
    _member("split_granularity", _GRANULARITIES),
    _member("runtime_kind", _RUNTIME_KINDS),
    _member("parallel_role", _PARALLEL_ROLES),
    _non_negative("expert_id"),
    _non_negative("owner_rank"),
    (lambda c: bool(c.h.owner_replica_ranks),
     lambda c: min(c.h.owner_replica_ranks) < 0,
     lambda c: f"Param {c.fqn} owner_replica_ranks must be non-negative, got {c.h.owner_replica_ranks}."),
    (lambda c: c.h.runtime_kind == ParamRuntimeKind.EXPERT_OWNER,
     lambda c: not c.h.expert_group_id,
     lambda c: f"Param {c.fqn} runtime_kind='expert_owner' requires expert_group_id metadata."),
    # ---- block_shape on its own
    (lambda c: c.bs is not None,
     lambda c: len(c.bs) == 0,
     lambda c: f"Param {c.fqn} block_shape cannot be empty."),
    (lambda c: c.bs is not None,
     lambda c: min(c.bs) <= 0,
     lambda c: f"Param {c.fqn} block_shape dims must be positive, got {c.bs}."),
    # ---- whole-parameter granularities take no block shape
    (lambda c: c.g in _WHOLE,
     lambda c: c.bs is not None,
     lambda c: f"Param {c.fqn} split_granularity={c.g!r} does not accept block_shape."),
    (lambda c: c.g == "matrix_owner",
     lambda c: len(c.shape) != 2,
     lambda c: f"Param {c.fqn} matrix_owner split_granularity expects a 2D tensor, got shape={c.shape}."),
    # ---- flat blocks
    (lambda c: c.g == "block",
     lambda c: c.bs is None or len(c.bs) != 1,
     lambda c: f"Param {c.fqn} block split_granularity expects a 1D block_shape."),
    (lambda c: c.g == "block",
     lambda c: c.numel % c.bs[0] != 0,
     lambda c: f"Param {c.fqn} numel={c.numel} is not divisible by block_shape={c.bs}."),
    # ---- row blocks of a matrix
    (lambda c: c.g == "row_block",
     lambda c: len(c.shape) != 2,
     lambda c: f"Param {c.fqn} row_block split_granularity expects a 2D tensor, got shape={c.shape}."),
    (lambda c: c.g == "row_block",
     lambda c: c.bs is None or len(c.bs) not in (1, 2),
     lambda c: f"Param {c.fqn} row_block split_granularity expects a 1D or 2D block_shape."),
    (lambda c: c.g == "row_block" and len(c.bs) == 2,
     lambda c: c.bs[1] != c.cols,
     lambda c: f"Param {c.fqn} row_block block_shape second dim={c.bs[1]} must match cols={c.cols}."),
    (lambda c: c.g == "row_block",
     lambda c: c.rows % c.bs[0] != 0,
     lambda c: f"Param {c.fqn} rows={c.rows} is not divisible by row block={c.bs[0]}."),
)


def validate_param_shard_hint(fqn: str, shape, numel: int, hint: ParamShardHint) -> None:
    """Raise ``ValueError`` for the first rule of the table that the hint breaks."""
    ctx = _HintCheck(fqn, shape, numel, hint)
    for applies, broken, message in _HINT_RULES:
        if applies(ctx) and broken(ctx):
            raise ValueError(message(ctx))


def hint_block_units(mp: ManagedParam) -> int | None:
    """Smallest indivisible run of elements for a parameter, or ``None`` for whole-param."""
    h = mp.shard_hint
    if not h.block_shape:
        return None
    per_row = {"block": 1, "row_block": int(mp.shape[1]) if len(mp.shape) == 2 else 0}.get(h.split_granularity, 0)
    return int(h.block_shape[0]) * per_row or None
