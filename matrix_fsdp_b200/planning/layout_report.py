"""Metrics of a group layout: balance, fragmentation, split parameters, traffic estimates.

Parity: ``matrix_fsdp/planning/layout_report.py:12-165``.
"""
from __future__ import annotations

from collections import Counter
from collections.abc import Sequence
from dataclasses import asdict, dataclass

from ..core.layout import MatrixGroupLayout
from .planner import ParamBlock


@dataclass(frozen=True)
class MatrixGroupLayoutReport:
    total_numel: int
    world_size: int
    rank_units: tuple[int, ...]
    max_rank_units: int
    min_rank_units: int
    avg_rank_units: float
    imbalance_units: int
    imbalance_ratio: float
    non_empty_ranks: int
    num_params: int
    num_whole_params: int
    whole_param_fqns: tuple[str, ...]
    num_split_params: int
    split_param_fqns: tuple[str, ...]
    split_param_units: int
    num_blocks: int
    blocks_by_kind: dict[str, int]
    params_by_rank: tuple[tuple[str, ...], ...]
    rank_segment_counts: tuple[int, ...]
    num_rank_segments: int
    max_rank_segments: int
    fragmented_rank_segments: int
    fragmented_rank_units: int
    param_segment_counts: dict[str, int]
    num_param_segments: int
    split_param_segments: int
    max_param_segments: int
    total_comm_units: int
    max_rank_comm_units: int
    estimated_padding_units: int
    estimated_collectives: int

    def as_metadata(self) -> dict[str, object]:
        return asdict(self)


def _padding_units(rank_units: Sequence[int], alignment: int | None) -> int:
    if alignment is None:
        return 0
    if alignment <= 0:
        raise ValueError(f"padding_alignment must be positive, got {alignment}.")
    return sum((-u) % alignment for u in rank_units)


def report_group_layout(layout: MatrixGroupLayout, blocks: Sequence[ParamBlock] = (), *,
                        padding_alignment: int | None = None,
                        collectives_per_segmented_exchange: int = 2) -> MatrixGroupLayoutReport:
    if collectives_per_segmented_exchange < 0:
        raise ValueError(
            f"collectives_per_segmented_exchange must be non-negative, got {collectives_per_segmented_exchange}.")
    units = layout.shard_sizes
    mx, mn = max(units, default=0), min(units, default=0)
    avg = sum(units) / len(units) if units else 0
    whole = tuple(p.fqn for p in layout.params if len(p.segments) == 1)
    split = tuple(p.fqn for p in layout.params if len(p.segments) > 1)
    seg_counts = tuple(len(r.segments) for r in layout.ranks)
    pseg = {p.fqn: len(p.segments) for p in layout.params}
    nseg = sum(seg_counts)
    return MatrixGroupLayoutReport(
        total_numel=layout.total_numel, world_size=layout.world_size, rank_units=units, max_rank_units=mx,
        min_rank_units=mn, avg_rank_units=avg, imbalance_units=mx - mn,
        imbalance_ratio=(mx / avg) if avg else 0.0, non_empty_ranks=sum(1 for u in units if u > 0),
        num_params=len(layout.params), num_whole_params=len(whole), whole_param_fqns=whole,
        num_split_params=len(split), split_param_fqns=split,
        split_param_units=sum(p.numel for p in layout.params if len(p.segments) > 1),
        num_blocks=len(blocks), blocks_by_kind=dict(Counter(b.kind for b in blocks)),
        params_by_rank=tuple(layout.params_for_rank(r) for r in range(layout.world_size)),
        rank_segment_counts=seg_counts, num_rank_segments=nseg, max_rank_segments=max(seg_counts, default=0),
        fragmented_rank_segments=sum(max(0, c - 1) for c in seg_counts),
        fragmented_rank_units=sum(r.local_units for r in layout.ranks if len(r.segments) > 1),
        param_segment_counts=pseg, num_param_segments=sum(pseg.values()),
        split_param_segments=sum(max(0, c - 1) for c in pseg.values()),
        max_param_segments=max(pseg.values(), default=0),
        total_comm_units=layout.total_numel * layout.world_size, max_rank_comm_units=mx * layout.world_size,
        estimated_padding_units=_padding_units(units, padding_alignment),
        estimated_collectives=collectives_per_segmented_exchange if nseg else 0)
