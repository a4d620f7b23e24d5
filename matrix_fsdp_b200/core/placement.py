"""``MatrixShard``: a DTensor ``Placement`` for rank-ordered contiguous cuts of a flattened tensor.

The placement stores only *proportions*: ``local_units[r]`` is rank r's share of the flat tensor
in gcd-reduced units, so a loader can recompute every rank's range from the total size alone
(checkpoint metadata stores exactly this).  Internally the class keeps the running sum of the
units (``_cuts``), so every query (length, offset, range, split) is a lookup into one table
scaled by ``total_numel / sum(units)``.

Capability parity: ``matrix_fsdp/core/placement.py:25-238`` (same public names and semantics).
"""
from __future__ import annotations

from dataclasses import dataclass
from itertools import accumulate
from math import gcd

import torch

from .layout import MatrixGroupLayout, ShardPlan

try:  # the Placement base class moved between torch releases
    from torch.distributed.tensor.placement_types import Placement as _PlacementBase
except Exception:  # pragma: no cover
    _PlacementBase = object


def is_matrix_shard_placement(placement: object) -> bool:
    probe = getattr(placement, "is_matrix_shard", None)
    return bool(probe()) if callable(probe) else False


def _require(ok: bool, message: str) -> None:
    if not ok:
        raise ValueError(message)


class MatrixShard(_PlacementBase):
    """Flatten over ``dims`` and cut into one chunk per rank, chunk r taking ``local_units[r]`` parts."""

    __slots__ = ("dims", "local_units", "_cuts")

    def __init__(self, dims: tuple[int, ...], local_units: tuple[int, ...]) -> None:
        super().__init__()
        dims = tuple(int(d) for d in dims)
        units = tuple(int(u) for u in local_units)
        _require(len(units) > 0, "local_units cannot be empty.")
        _require(min(units) >= 0, f"local_units must be non-negative, got {units}.")
        _require(sum(units) > 0, "local_units cannot all be zero.")
        _require(all(d >= 0 for d in dims), f"dims must be non-negative, got {dims}.")
        for name, value in (("dims", dims), ("local_units", units), ("_cuts", (0, *accumulate(units)))):
            object.__setattr__(self, name, value)

    # immutable value object ------------------------------------------------------------
    def __setattr__(self, key, value):
        raise AttributeError("MatrixShard is immutable")

    def _identity(self) -> tuple:
        return ("MatrixShard", self.dims, self.local_units)

    def __eq__(self, other: object) -> bool:
        return isinstance(other, MatrixShard) and self._identity() == other._identity()

    def __hash__(self) -> int:
        return hash(self._identity())

    def __repr__(self) -> str:
        return f"MatrixShard(dims={self.dims}, local_units={self.local_units})"

    __str__ = __repr__

    def is_matrix_shard(self) -> bool:
        return True

    # geometry --------------------------------------------------------------------------
    @property
    def world_size(self) -> int:
        return len(self.local_units)

    @property
    def total_units(self) -> int:
        return self._cuts[-1]

    def _boundaries(self, total_numel: int) -> tuple[int, ...]:
        """Element offsets of all cuts (``world_size + 1`` values, first 0, last ``total_numel``)."""
        _require(total_numel >= 0, f"total_numel must be non-negative, got {total_numel}.")
        per_unit, rest = divmod(total_numel, self.total_units)
        _require(rest == 0, f"total_numel={total_numel} must be divisible by sum(local_units)={self.total_units}.")
        return tuple(c * per_unit for c in self._cuts)

    def _check_rank(self, rank: int) -> int:
        _require(0 <= rank < self.world_size, f"rank={rank} is out of range for world_size={self.world_size}.")
        return rank

    def shard_range(self, rank: int, total_numel: int) -> tuple[int, int]:
        cuts = self._boundaries(total_numel)
        r = self._check_rank(rank)
        return cuts[r], cuts[r + 1]

    def shard_offset(self, rank: int, total_numel: int) -> int:
        return self.shard_range(rank, total_numel)[0]

    def shard_lengths(self, total_numel: int) -> tuple[int, ...]:
        cuts = self._boundaries(total_numel)
        return tuple(b - a for a, b in zip(cuts, cuts[1:]))

    # tensors ---------------------------------------------------------------------------
    def split_tensor(self, tensor: torch.Tensor, *, num_chunks: int | None = None) -> tuple[torch.Tensor, ...]:
        """Views of ``tensor`` (contiguous), one per rank, in rank order."""
        _require(tensor.is_contiguous(), "MatrixShard expects a contiguous tensor.")
        _require(num_chunks in (None, self.world_size),
                 f"num_chunks={num_chunks} must equal len(local_units)={self.world_size}.")
        flat = tensor.view(-1)
        cuts = self._boundaries(flat.numel())
        return tuple(flat[a:b] for a, b in zip(cuts, cuts[1:]))

    def local_shard(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        return self.split_tensor(tensor)[self._check_rank(rank)]

    def reconstruct_tensor_from_flat(self, flat_tensor: torch.Tensor, shape: tuple[int, ...]) -> torch.Tensor:
        _require(flat_tensor.ndim == 1, f"flat_tensor must be 1D, got shape={tuple(flat_tensor.shape)}.")
        lead = len(self.dims)
        _require(self.dims == tuple(range(lead)), f"dims must be a prefix tuple like (0, 1, ...), got {self.dims}.")
        tail = tuple(shape[lead:])
        tail_numel = int(torch.Size(tail).numel()) if tail else 1
        _require(flat_tensor.numel() % tail_numel == 0,
                 f"flat_tensor.numel()={flat_tensor.numel()} must be divisible by trailing shape product={tail_numel}.")
        return flat_tensor.view(-1, *tail)


MatrixShardPlacement = MatrixShard


@dataclass(frozen=True)
class PlacementCompatibility:
    compatible: bool
    reason: str | None = None
    requires_flat_reorder: bool = False
    requires_multi_segment_runtime: bool = False


def shard_sizes_to_matrix_local_units(shard_sizes: tuple[int, ...]) -> tuple[int, ...]:
    _require(len(shard_sizes) > 0, "shard_sizes cannot be empty.")
    _require(min(shard_sizes) >= 0, f"shard_sizes must be non-negative, got {shard_sizes}.")
    _require(any(shard_sizes), "Matrix local_units cannot represent an all-empty shard plan.")
    common = gcd(*shard_sizes)
    return tuple(s // common for s in shard_sizes)


def explain_matrix_shard_compatibility(layout_or_plan: MatrixGroupLayout | ShardPlan) -> PlacementCompatibility:
    """A plan fits a ``MatrixShard`` exactly when it *is* the canonical cut: rank r holds the single run
    ``[sum(sizes[:r]), sum(sizes[:r+1]))`` at local offset 0.  The plan's segments are compared with that
    canonical picture rank by rank; the first difference becomes the reason, together with what kind of
    runtime support (a rank-major re-lay of the flat space, several segments per rank) would lift it."""
    plan = layout_or_plan.to_shard_plan() if isinstance(layout_or_plan, MatrixGroupLayout) else layout_or_plan
    if plan.total_numel <= 0:
        return PlacementCompatibility(False, "an empty plan has no proportions to record")
    if plan.rank_segments is None:
        return PlacementCompatibility(False, "the plan carries no per-rank segments")
    if sum(plan.shard_sizes) != plan.total_numel:
        return PlacementCompatibility(
            False, f"shard sizes add up to {sum(plan.shard_sizes)}, the flat space has {plan.total_numel} elements")
    starts = (0, *accumulate(plan.shard_sizes))
    for rank, (size, begin, segs) in enumerate(zip(plan.shard_sizes, starts, plan.rank_segments)):
        held = [(s.global_start, s.global_end, s.local_start) for s in segs if s.numel]
        want = [(begin, begin + size, 0)] if size else []
        if held == want:
            continue
        if len(held) > 1:
            return PlacementCompatibility(False, f"rank {rank} holds {len(held)} separate runs, a MatrixShard holds one",
                                          requires_flat_reorder=True, requires_multi_segment_runtime=True)
        if not want or not held:
            return PlacementCompatibility(False, f"rank {rank}: shard size {size} does not match its segments {held}")
        (g0, g1, l0), = held
        if g1 - g0 != size:
            return PlacementCompatibility(False, f"rank {rank}: its run has {g1 - g0} elements, its shard {size}")
        if l0 != 0:
            return PlacementCompatibility(False, f"rank {rank}: its run is stored at local offset {l0}, not 0")
        return PlacementCompatibility(False, f"rank {rank}: its run starts at {g0}; in rank order it would start at {begin}",
                                      requires_flat_reorder=True)
    return PlacementCompatibility(True)


def is_matrix_shard_compatible_plan(layout_or_plan: MatrixGroupLayout | ShardPlan) -> bool:
    return explain_matrix_shard_compatibility(layout_or_plan).compatible


def matrix_shard_from_plan(plan: ShardPlan, *, dims: tuple[int, ...] = (0,)) -> MatrixShard:
    verdict = explain_matrix_shard_compatibility(plan)
    _require(verdict.compatible,
             "MatrixShard can directly represent only contiguous rank-ordered flat shard plans. "
             f"Reason: {verdict.reason}.")
    return MatrixShard(dims=dims, local_units=shard_sizes_to_matrix_local_units(plan.shard_sizes))


def matrix_shard_from_layout(layout: MatrixGroupLayout, *, dims: tuple[int, ...] = (0,)) -> MatrixShard:
    return matrix_shard_from_plan(layout.to_shard_plan(), dims=dims)
