"""Structural validation of planner output and classification of how the runtime executes it.

Checks: every element of the group is held by exactly one rank, local packing is gap-free,
parameter segments agree with rank segments, and shard-hint constraints hold (whole-param
owners, block / row-block alignment, one owner per expert group).

Runtime modes: ``matrix_shard`` (one rank-ordered chunk per rank: equal-chunk collectives
apply), ``segment_runtime`` (arbitrary per-rank segment lists: the peer pull kernels take a
(peer, offset, length) table, so no padding or reordering is needed), ``flat_reorder``
(whole-parameter owner layouts re-packed rank-major on request).

Parity: ``matrix_fsdp/planning/layout_validator.py:12-359``.
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

from ..core.layout import LayoutSegment, MatrixGroupLayout, ParamSegment
from ..core.managed_param import ManagedParam, ParamRuntimeKind
from ..core.placement import explain_matrix_shard_compatibility


@dataclass(frozen=True)
class RuntimeLayoutCompatibility:
    compatible: bool
    mode: str
    reason: str | None = None
    requires_flat_reorder: bool = False
    matrix_shard_compatible: bool = False
    matrix_shard_reason: str | None = None


def _check_range(start: int, end: int, total: int, ctx: str) -> None:
    if start < 0 or end > total or start > end:
        raise ValueError(f"{ctx} range [{start}, {end}) is outside [0, {total}).")


def _check_exact_cover(intervals: list[tuple[int, int, str]], total: int, what: str) -> None:
    cursor = 0
    for start, end, ctx in sorted(intervals):
        if start == end:
            continue
        if start < cursor:
            raise ValueError(f"{what} overlap at offset {start} ({ctx}).")
        if start > cursor:
            raise ValueError(f"{what} leave a gap [{cursor}, {start}) before {ctx}.")
        cursor = end
    if cursor != total:
        raise ValueError(f"{what} cover {cursor} elements, expected {total}.")


def validate_group_layout(layout: MatrixGroupLayout, params: Sequence[ManagedParam], world_size: int) -> None:
    total = sum(p.numel for p in params)
    if layout.world_size != world_size:
        raise ValueError(f"Layout world_size={layout.world_size} does not match world_size={world_size}.")
    if layout.total_numel != total:
        raise ValueError(f"Layout total_numel={layout.total_numel} does not match parameter total {total}.")
    if {p.fqn for p in layout.params} != {p.fqn for p in params}:
        raise ValueError("Layout parameter set does not match the managed parameters.")
    # rank segments: in range, locally packed, exact global cover
    cover = []
    for rl in layout.ranks:
        local = sorted(rl.segments, key=lambda s: s.local_start)
        cur = 0
        for seg in local:
            _check_range(seg.global_start, seg.global_end, total, f"rank {rl.rank} segment")
            if seg.local_start != cur:
                raise ValueError(
                    f"rank {rl.rank} segment {seg} breaks local packing (expected local_start={cur}).")
            cur = seg.local_end
            cover.append((seg.global_start, seg.global_end, f"rank {rl.rank}"))
        if cur != rl.local_units:
            raise ValueError(f"rank {rl.rank} local_units={rl.local_units} but segments pack {cur} elements.")
    _check_exact_cover(cover, total, "Rank segments")
    # param segments: exact cover of each param and containment in a rank segment
    by_fqn = {p.fqn: p for p in params}
    for pl in layout.params:
        mp = by_fqn[pl.fqn]
        if (pl.global_start, pl.global_end) != (mp.offset, mp.end):
            raise ValueError(f"Param {pl.fqn} layout range does not match its managed offset range.")
        pcover = []
        for ps in pl.segments:
            if ps.fqn != pl.fqn:
                raise ValueError(f"Param segment {ps} is filed under {pl.fqn}.")
            _check_range(ps.global_start, ps.global_end, total, f"param {pl.fqn} segment")
            pcover.append((ps.global_start - mp.offset, ps.global_end - mp.offset, f"rank {ps.rank}"))
            if not _rank_contains(layout.ranks[ps.rank].segments, ps):
                raise ValueError(f"Param segment {ps} is not contained in a segment of rank {ps.rank}.")
        _check_exact_cover(pcover, mp.numel, f"Param {pl.fqn} segments")
    _validate_hints(layout, params)


def _rank_contains(rank_segments: tuple[LayoutSegment, ...], ps: ParamSegment) -> bool:
    for seg in rank_segments:
        if seg.global_start <= ps.global_start and ps.global_end <= seg.global_end:
            return ps.local_start == seg.local_start + (ps.global_start - seg.global_start)
    return False


def _check_alignment(segments, offset: int, units: int, fqn: str) -> None:
    for s in segments:
        if (s.global_start - offset) % units or (s.global_end - offset) % units:
            raise ValueError(f"Param {fqn} segment {s} is not aligned to block_units={units}.")


def _validate_hints(layout: MatrixGroupLayout, params: Sequence[ManagedParam]) -> None:
    by_fqn = {pl.fqn: pl for pl in layout.params}
    expert_owners: dict[str, set[int]] = {}
    for mp in params:
        h, pl = mp.shard_hint, by_fqn[mp.fqn]
        if h.split_granularity in ("parameter", "matrix_owner") and len(pl.segments) != 1:
            raise ValueError(
                f"Param {mp.fqn} split_granularity={h.split_granularity!r} "
                "requires a single whole-parameter owner segment.")
        if h.split_granularity == "block" and h.block_shape is not None:
            _check_alignment(pl.segments, mp.offset, h.block_shape[0], mp.fqn)
        if h.split_granularity == "row_block" and h.block_shape is not None:
            _check_alignment(pl.segments, mp.offset, h.block_shape[0] * tuple(mp.shape)[1], mp.fqn)
        if h.runtime_kind == ParamRuntimeKind.EXPERT_OWNER:
            if len(pl.segments) != 1:
                raise ValueError(f"Param {mp.fqn} runtime_kind='expert_owner' requires one whole owner segment.")
            expert_owners.setdefault(h.expert_group_id or mp.fqn, set()).add(pl.segments[0].rank)
    for gid, ranks in expert_owners.items():
        if len(ranks) != 1:
            raise ValueError(f"Expert group {gid!r} must have one owner rank, got {tuple(sorted(ranks))}.")


def _is_whole_param_layout(layout: MatrixGroupLayout) -> bool:
    return all(len(pl.segments) == 1 and pl.segments[0].numel == pl.numel for pl in layout.params)


def explain_runtime_layout_compatibility(layout: MatrixGroupLayout, params: Sequence[ManagedParam], world_size: int, *,
                                         allow_flat_reorder: bool = True,
                                         allow_segment_runtime: bool = True) -> RuntimeLayoutCompatibility:
    validate_group_layout(layout, params, world_size)
    pc = explain_matrix_shard_compatibility(layout)
    if pc.compatible:
        return RuntimeLayoutCompatibility(True, "matrix_shard", matrix_shard_compatible=True)
    if allow_segment_runtime:
        return RuntimeLayoutCompatibility(True, "segment_runtime", reason=pc.reason, matrix_shard_reason=pc.reason)
    if allow_flat_reorder and _is_whole_param_layout(layout):
        return RuntimeLayoutCompatibility(True, "flat_reorder", reason=pc.reason, requires_flat_reorder=True,
                                          matrix_shard_reason=pc.reason)
    return RuntimeLayoutCompatibility(
        False, "unsupported",
        reason="layout requires segment_runtime, but segment runtime layouts are disabled",
        requires_flat_reorder=pc.requires_flat_reorder, matrix_shard_reason=pc.reason)


def validate_runtime_layout(layout: MatrixGroupLayout, params: Sequence[ManagedParam], world_size: int, *,
                            allow_flat_reorder: bool = True,
                            allow_segment_runtime: bool = True) -> RuntimeLayoutCompatibility:
    compat = explain_runtime_layout_compatibility(layout, params, world_size, allow_flat_reorder=allow_flat_reorder,
                                                  allow_segment_runtime=allow_segment_runtime)
    if not compat.compatible:
        raise ValueError(f"MatrixFSDP runtime cannot execute planner layout. Reason: {compat.reason}.")
    return compat


def flat_reorder_order(layout: MatrixGroupLayout) -> list[str]:
    """Rank-major parameter order that turns a whole-param owner layout into rank-contiguous chunks."""
    order: list[str] = []
    for rank in range(layout.world_size):
        for ps in layout.param_segments_for_rank(rank):
            order.append(ps.fqn)
    return order
