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
        hints = dict(shard_hints or {})
        ignored = {id(p) for p in ignored_params or ()}
        names: dict[int, list[str]] = {}
        for fqn, p in module.named_parameters(recurse=True, remove_duplicate=False):
            if id(p) not in ignored:
                names.setdefault(id(p), []).append(fqn)
        shared = [v for v in names.values() if len(v) > 1]
        if shared and not allow_shared:
            listing = "; ".join(",".join(v) for v in shared)
            raise NotImplementedError(
                "MatrixFSDP does not support shared parameters yet. " f"Shared parameter aliases: {listing}."
            )
        out: list[ManagedParam] = []
        offset = 0
        for fqn, p in module.named_parameters(recurse=True, remove_duplicate=True):
            if id(p) in ignored:
                continue
            hint = hints.get(fqn, ParamShardHint())
            validate_param_shard_hint(fqn, p.shape, p.numel(), hint)
            aliases = tuple(n for n in names[id(p)] if n != fqn)
            out.append(ManagedParam(fqn, p, p.shape, p.dtype, p.device, p.numel(), offset, offset + p.numel(), hint, aliases))
            offset += p.numel()
        known = {mp.fqn for mp in out} | {a for mp in out for a in mp.aliases}
        unknown = set(hints) - known
        if unknown:
            raise ValueError(f"Shard hints refer to unknown parameters: {', '.join(sorted(unknown))}.")
        return cls(tuple(out))


def _fmt(values) -> str:
    return ", ".join(repr(v) for v in sorted(values, key=str))


def validate_param_shard_hint(fqn: str, shape, numel: int, hint: ParamShardHint) -> None:
    shape = tuple(shape)
    if hint.split_granularity not in _GRANULARITIES:
        raise ValueError(
            f"Param {fqn} has unknown split_granularity={hint.split_granularity!r}; expected {_fmt(_GRANULARITIES)}.")
    if hint.runtime_kind not in _RUNTIME_KINDS:
        raise ValueError(f"Param {fqn} has unknown runtime_kind={hint.runtime_kind!r}; expected {_fmt(_RUNTIME_KINDS)}.")
    if hint.parallel_role not in _PARALLEL_ROLES:
        raise ValueError(
            f"Param {fqn} has unknown parallel_role={hint.parallel_role!r}; expected {_fmt(_PARALLEL_ROLES)}.")
    if hint.expert_id is not None and hint.expert_id < 0:
        raise ValueError(f"Param {fqn} expert_id must be non-negative, got {hint.expert_id}.")
    if hint.owner_rank is not None and hint.owner_rank < 0:
        raise ValueError(f"Param {fqn} owner_rank must be non-negative, got {hint.owner_rank}.")
    if any(r < 0 for r in hint.owner_replica_ranks):
        raise ValueError(f"Param {fqn} owner_replica_ranks must be non-negative, got {hint.owner_replica_ranks}.")
    if hint.runtime_kind == ParamRuntimeKind.EXPERT_OWNER and not hint.expert_group_id:
        raise ValueError(f"Param {fqn} runtime_kind='expert_owner' requires expert_group_id metadata.")
    bs = hint.block_shape
    if bs is not None:
        if len(bs) == 0:
            raise ValueError(f"Param {fqn} block_shape cannot be empty.")
        if any(d <= 0 for d in bs):
            raise ValueError(f"Param {fqn} block_shape dims must be positive, got {bs}.")
    g = hint.split_granularity
    if g in (None, "parameter", "matrix_owner"):
        if bs is not None:
            raise ValueError(f"Param {fqn} split_granularity={g!r} does not accept block_shape.")
        if g == "matrix_owner" and len(shape) != 2:
            raise ValueError(f"Param {fqn} matrix_owner split_granularity expects a 2D tensor, got shape={shape}.")
        return
    if g == "block":
        if bs is None or len(bs) != 1:
            raise ValueError(f"Param {fqn} block split_granularity expects a 1D block_shape.")
        if numel % bs[0] != 0:
            raise ValueError(f"Param {fqn} numel={numel} is not divisible by block_shape={bs}.")
        return
    # row_block
    if len(shape) != 2:
        raise ValueError(f"Param {fqn} row_block split_granularity expects a 2D tensor, got shape={shape}.")
    if bs is None or len(bs) not in (1, 2):
        raise ValueError(f"Param {fqn} row_block split_granularity expects a 1D or 2D block_shape.")
    rows, cols = shape
    if len(bs) == 2 and bs[1] != cols:
        raise ValueError(f"Param {fqn} row_block block_shape second dim={bs[1]} must match cols={cols}.")
    if rows % bs[0] != 0:
        raise ValueError(f"Param {fqn} rows={rows} is not divisible by row block={bs[0]}.")


def hint_block_units(mp: ManagedParam) -> int | None:
    """Smallest indivisible run of elements for a parameter, or ``None`` for whole-param."""
    h = mp.shard_hint
    if h.split_granularity == "block" and h.block_shape:
        return int(h.block_shape[0])
    if h.split_granularity == "row_block" and h.block_shape:
        return int(h.block_shape[0]) * int(mp.shape[1])
    return None
