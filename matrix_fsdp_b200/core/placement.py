"""``MatrixShard``: a DTensor ``Placement`` describing rank-ordered contiguous flat chunks.

A logical tensor is flattened and cut into one contiguous chunk per rank, chunk sizes being
proportional to ``local_units`` (the gcd-reduced shard sizes).  Checkpoint metadata stores
this placement so a loader can recompute every rank's range from the total size alone.

Parity: ``matrix_fsdp/core/placement.py:25-238``.
"""
from __future__ import annotations

from dataclasses import dataclass
from functools import reduce
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


class MatrixShard(_PlacementBase):
    """Placement: flatten over ``dims`` and split into chunks proportional to ``local_units``."""

    __slots__ = ("dims", "local_units")

    def __init__(self, dims: tuple[int, ...], local_units: tuple[int, ...]) -> None:
        super().__init__()
        object.__setattr__(self, "dims", tuple(int(d) for d in dims))
        object.__setattr__(self, "local_units", tuple(int(u) for u in local_units))
        if not self.local_units:
            raise ValueError("local_units cannot be empty.")
        if any(u < 0 for u in self.local_units):
            raise ValueError(f"local_units must be non-negative, got {self.local_units}.")
        if sum(self.local_units) == 0:
            raise ValueError("local_units cannot all be zero.")
        if any(d < 0 for d in self.dims):
            raise ValueError(f"dims must be non-negative, got {self.dims}.")

    def __setattr__(self, key, value):  # frozen
        raise AttributeError("MatrixShard is immutable")

    def __eq__(self, other: object) -> bool:
        return isinstance(other, MatrixShard) and self.dims == other.dims and self.local_units == other.local_units

    def __hash__(self) -> int:
        return hash(("MatrixShard", self.dims, self.local_units))

    def __repr__(self) -> str:
        return f"MatrixShard(dims={self.dims}, local_units={self.local_units})"

    __str__ = __repr__

    @property
    def world_size(self) -> int:
        return len(self.local_units)

    @property
    def total_units(self) -> int:
        return sum(self.local_units)

    def _ratio(self, total_numel: int) -> int:
        if total_numel < 0:
            raise ValueError(f"total_numel must be non-negative, got {total_numel}.")
        if total_numel % self.total_units != 0:
            raise ValueError(
                f"total_numel={total_numel} must be divisible by sum(local_units)={self.total_units}.")
        return total_numel // self.total_units

    def _validate_rank(self, rank: int) -> None:
        if not 0 <= rank < self.world_size:
            raise ValueError(f"rank={rank} is out of range for world_size={self.world_size}.")

    def shard_lengths(self, total_numel: int) -> tuple[int, ...]:
        ratio = self._ratio(total_numel)
        return tuple(u * ratio for u in self.local_units)

    def shard_offset(self, rank: int, total_numel: int) -> int:
        self._validate_rank(rank)
        return sum(self.local_units[:rank]) * self._ratio(total_numel)

    def shard_range(self, rank: int, total_numel: int) -> tuple[int, int]:
        start = self.shard_offset(rank, total_numel)
        return start, start + self.shard_lengths(total_numel)[rank]

    def split_tensor(self, tensor: torch.Tensor, *, num_chunks: int | None = None) -> tuple[torch.Tensor, ...]:
        """Views of ``tensor`` (contiguous), one per rank, in rank order."""
        if not tensor.is_contiguous():
            raise ValueError("MatrixShard expects a contiguous tensor.")
        if num_chunks is not None and num_chunks != self.world_size:
            raise ValueError(f"num_chunks={num_chunks} must equal len(local_units)={self.world_size}.")
        flat = tensor.view(-1)
        out, start = [], 0
        for n in self.shard_lengths(flat.numel()):
            out.append(flat.narrow(0, start, n))
            start += n
        return tuple(out)

    def local_shard(self, tensor: torch.Tensor, rank: int) -> torch.Tensor:
        self._validate_rank(rank)
        return self.split_tensor(tensor)[rank]

    def is_matrix_shard(self) -> bool:
        return True

    def reconstruct_tensor_from_flat(self, flat_tensor: torch.Tensor, shape: tuple[int, ...]) -> torch.Tensor:
        if flat_tensor.ndim != 1:
            raise ValueError(f"flat_tensor must be 1D, got shape={tuple(flat_tensor.shape)}.")
        nd = len(self.dims)
        if self.dims != tuple(range(nd)):
            raise ValueError(f"dims must be a prefix tuple like (0, 1, ...), got {self.dims}.")
        trailing = 1
        for s in shape[nd:]:
            trailing *= s
        if flat_tensor.numel() % trailing != 0:
            raise ValueError(
                f"flat_tensor.numel()={flat_tensor.numel()} must be divisible by trailing shape product={trailing}.")
        return flat_tensor.view(-1, *shape[nd:])


MatrixShardPlacement = MatrixShard


@dataclass(frozen=True)
class PlacementCompatibility:
    compatible: bool
    reason: str | None = None
    requires_flat_reorder: bool = False
    requires_multi_segment_runtime: bool = False


def shard_sizes_to_matrix_local_units(shard_sizes: tuple[int, ...]) -> tuple[int, ...]:
    if not shard_sizes:
        raise ValueError("shard_sizes cannot be empty.")
    if any(s < 0 for s in shard_sizes):
        raise ValueError(f"shard_sizes must be non-negative, got {shard_sizes}.")
    if sum(shard_sizes) == 0:
        raise ValueError("Matrix local_units cannot represent an all-empty shard plan.")
    div = max(reduce(gcd, shard_sizes, 0), 1)
    return tuple(s // div for s in shard_sizes)


def _to_shard_plan(layout_or_plan: MatrixGroupLayout | ShardPlan) -> ShardPlan:
    return layout_or_plan.to_shard_plan() if isinstance(layout_or_plan, MatrixGroupLayout) else layout_or_plan


def explain_matrix_shard_compatibility(layout_or_plan: MatrixGroupLayout | ShardPlan) -> PlacementCompatibility:
    """A plan is MatrixShard-representable iff each rank holds one chunk and chunks are rank-ordered."""
    plan = _to_shard_plan(layout_or_plan)
    if plan.total_numel <= 0:
        return PlacementCompatibility(False, "empty shard plans cannot be represented as matrix placements")
    if plan.rank_segments is None:
        return PlacementCompatibility(False, "missing rank segment metadata")
    cursor = 0
    for rank, segs in enumerate(plan.rank_segments):
        if plan.shard_sizes[rank] == 0:
            if any(s.numel for s in segs):
                return PlacementCompatibility(False, f"rank {rank} has segments for an empty shard")
            continue
        if len(segs) != 1:
            return PlacementCompatibility(
                False, f"rank {rank} has {len(segs)} local segments, expected exactly one",
                requires_flat_reorder=True, requires_multi_segment_runtime=True)
        seg = segs[0]
        if seg.local_start != 0:
            return PlacementCompatibility(False, f"rank {rank} segment local_start={seg.local_start}, expected 0")
        if seg.global_start != cursor:
            return PlacementCompatibility(
                False, f"rank {rank} segment starts at {seg.global_start}, expected rank-ordered cursor {cursor}",
                requires_flat_reorder=True)
        if seg.numel != plan.shard_sizes[rank]:
            return PlacementCompatibility(
                False, f"rank {rank} segment size={seg.numel}, expected shard size={plan.shard_sizes[rank]}")
        cursor = seg.global_end
    if cursor != plan.total_numel:
        return PlacementCompatibility(False, f"rank segments cover {cursor} elements, expected {plan.total_numel}")
    return PlacementCompatibility(True)


def is_matrix_shard_compatible_plan(layout_or_plan: MatrixGroupLayout | ShardPlan) -> bool:
    return explain_matrix_shard_compatibility(layout_or_plan).compatible


def matrix_shard_from_plan(plan: ShardPlan, *, dims: tuple[int, ...] = (0,)) -> MatrixShard:
    compat = explain_matrix_shard_compatibility(plan)
    if not compat.compatible:
        raise ValueError(
            "MatrixShard can directly represent only contiguous rank-ordered flat shard plans. "
            f"Reason: {compat.reason}.")
    return MatrixShard(dims=dims, local_units=shard_sizes_to_matrix_local_units(plan.shard_sizes))


def matrix_shard_from_layout(layout: MatrixGroupLayout, *, dims: tuple[int, ...] = (0,)) -> MatrixShard:
    return matrix_shard_from_plan(layout.to_shard_plan(), dims=dims)
