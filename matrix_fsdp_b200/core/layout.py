"""Group-local layout data model: who holds which slice of a unit's flat parameter space.

All offsets are *group-local*: element indices into the flat concatenation of one FSDP
unit's managed parameters (not whole-model offsets).  A rank's shard is the ordered list of
:class:`LayoutSegment` it holds; ``local_start`` says where the segment sits inside that
rank's packed local shard.

Behavioural parity: ``matrix_fsdp/core/layout.py:15-224`` (same class and field names so
planner outputs, checkpoints and user code carry over); the implementation here is written
around interval arithmetic helpers that the peer-memory runtime reuses to build its
(peer, offset, length) pull tables.
"""
from __future__ import annotations

from bisect import bisect_right
from dataclasses import dataclass
from typing import Iterable, Protocol, Sequence


class LayoutParam(Protocol):
    fqn: str
    offset: int
    end: int


class _Span:
    """Interval arithmetic shared by the segment records: ``[global_start, global_end)`` of the flat space, packed
    at ``local_start`` of the holder's shard."""

    __slots__ = ()

    numel = property(lambda self: self.global_end - self.global_start)
    local_end = property(lambda self: self.local_start + (self.global_end - self.global_start))

    def intersects(self, start: int, end: int) -> bool:
        return self.global_start < end and start < self.global_end


@dataclass(frozen=True)
class LayoutSegment(_Span):
    global_start: int
    global_end: int
    local_start: int

    def __post_init__(self) -> None:
        if self.global_end < self.global_start:
            raise ValueError(f"segment end {self.global_end} < start {self.global_start}")
        if self.global_start < 0 or self.local_start < 0:
            raise ValueError("segment offsets must be non-negative")


@dataclass(frozen=True)
class ParamSegment(_Span):
    fqn: str
    rank: int
    global_start: int
    global_end: int
    local_start: int

    def to_layout_segment(self) -> LayoutSegment:
        return LayoutSegment(self.global_start, self.global_end, self.local_start)


def _exclusive_offsets(sizes: Sequence[int]) -> tuple[int, ...]:
    out, acc = [], 0
    for s in sizes:
        out.append(acc)
        acc += int(s)
    return tuple(out)


@dataclass(frozen=True)
class ShardPlan:
    """Per-rank shard sizes plus (optionally) the exact segments each rank holds."""

    total_numel: int
    shard_sizes: tuple[int, ...]
    shard_offsets: tuple[int, ...]
    rank_segments: tuple[tuple[LayoutSegment, ...], ...] | None = None

    def __post_init__(self) -> None:
        if len(self.shard_sizes) != len(self.shard_offsets):
            raise ValueError("shard_sizes and shard_offsets must have one entry per rank")
        if self.rank_segments is None:
            segs = tuple(
                (LayoutSegment(off, off + size, 0),) for off, size in zip(self.shard_offsets, self.shard_sizes)
            )
            object.__setattr__(self, "rank_segments", segs)

    @property
    def world_size(self) -> int:
        return len(self.shard_sizes)

    def local_range(self, rank: int) -> tuple[int, int]:
        off = self.shard_offsets[rank]
        return off, off + self.shard_sizes[rank]

    def local_segments(self, rank: int) -> tuple[LayoutSegment, ...]:
        assert self.rank_segments is not None
        return self.rank_segments[rank]


@dataclass(frozen=True)
class RankLayout:
    rank: int
    local_units: int
    segments: tuple[LayoutSegment, ...]


@dataclass(frozen=True)
class ParamLayout:
    fqn: str
    global_start: int
    global_end: int
    segments: tuple[ParamSegment, ...]

    @property
    def numel(self) -> int:
        return self.global_end - self.global_start


def split_segments_by_params(
    rank: int, segments: Iterable[LayoutSegment], params: Sequence[LayoutParam]
) -> list[ParamSegment]:
    """Cut a rank's segments at parameter boundaries (params must be offset-sorted)."""
    starts = [p.offset for p in params]
    out: list[ParamSegment] = []
    for seg in segments:
        if seg.numel == 0:
            continue
        i = max(bisect_right(starts, seg.global_start) - 1, 0)
        while i < len(params) and params[i].offset < seg.global_end:
            p = params[i]
            lo, hi = max(seg.global_start, p.offset), min(seg.global_end, p.end)
            if lo < hi:
                out.append(ParamSegment(p.fqn, rank, lo, hi, seg.local_start + (lo - seg.global_start)))
            i += 1
    return out


@dataclass(frozen=True)
class MatrixGroupLayout:
    """Layout of one planner/runtime communication group (one FSDP unit)."""

    total_numel: int
    ranks: tuple[RankLayout, ...]
    params: tuple[ParamLayout, ...] = ()

    @classmethod
    def from_rank_segments(
        cls,
        total_numel: int,
        rank_segments: Sequence[Sequence[LayoutSegment]],
        params: Sequence[LayoutParam] = (),
    ) -> "MatrixGroupLayout":
        ordered = sorted(params, key=lambda p: p.offset)
        ranks = []
        per_param: dict[str, list[ParamSegment]] = {p.fqn: [] for p in ordered}
        for rank, segs in enumerate(rank_segments):
            segs = tuple(segs)
            ranks.append(RankLayout(rank, sum(s.numel for s in segs), segs))
            for ps in split_segments_by_params(rank, segs, ordered):
                per_param[ps.fqn].append(ps)
        playouts = tuple(
            ParamLayout(p.fqn, p.offset, p.end, tuple(sorted(per_param[p.fqn], key=lambda s: s.global_start)))
            for p in params
        )
        return cls(int(total_numel), tuple(ranks), playouts)

    @classmethod
    def from_shard_plan(cls, plan: ShardPlan, params: Sequence[LayoutParam] = ()) -> "MatrixGroupLayout":
        assert plan.rank_segments is not None
        return cls.from_rank_segments(plan.total_numel, plan.rank_segments, params)

    @property
    def world_size(self) -> int:
        return len(self.ranks)

    @property
    def shard_sizes(self) -> tuple[int, ...]:
        return tuple(r.local_units for r in self.ranks)

    @property
    def rank_segments(self) -> tuple[tuple[LayoutSegment, ...], ...]:
        return tuple(r.segments for r in self.ranks)

    def param(self, fqn: str) -> ParamLayout:
        for p in self.params:
            if p.fqn == fqn:
                return p
        raise KeyError(f"Unknown parameter fqn: {fqn}")

    def owner_ranks(self, fqn: str) -> tuple[int, ...]:
        return tuple(sorted({s.rank for s in self.param(fqn).segments}))

    def param_segments_for_rank(self, rank: int) -> tuple[ParamSegment, ...]:
        segs = [s for p in self.params for s in p.segments if s.rank == rank]
        return tuple(sorted(segs, key=lambda s: s.local_start))

    def rank_segments_for_param(self, rank: int, fqn: str) -> tuple[ParamSegment, ...]:
        return tuple(s for s in self.param(fqn).segments if s.rank == rank)

    def params_for_rank(self, rank: int) -> tuple[str, ...]:
        return tuple(p.fqn for p in self.params if any(s.rank == rank for s in p.segments))

    def to_shard_plan(self) -> ShardPlan:
        sizes = self.shard_sizes
        offsets = tuple(r.segments[0].global_start if r.segments else 0 for r in self.ranks)
        if not rank_segments_are_rank_contiguous_chunks(self.rank_segments):
            offsets = _exclusive_offsets(sizes)
        return ShardPlan(self.total_numel, sizes, offsets, self.rank_segments)


def rank_segments_are_rank_contiguous_chunks(rank_segments: Sequence[Sequence[LayoutSegment]]) -> bool:
    """True when rank r holds exactly one chunk and chunks follow each other in rank order."""
    cursor = 0
    for segs in rank_segments:
        segs = [s for s in segs if s.numel > 0]
        if len(segs) > 1:
            return False
        if segs:
            s = segs[0]
            if s.global_start != cursor or s.local_start != 0:
                return False
            cursor = s.global_end
    return True


def contiguous_shard_plan(total_numel: int, shard_sizes: Sequence[int]) -> ShardPlan:
    sizes = tuple(int(s) for s in shard_sizes)
    if sum(sizes) != total_numel:
        raise ValueError(f"shard sizes sum to {sum(sizes)}, expected {total_numel}")
    return ShardPlan(int(total_numel), sizes, _exclusive_offsets(sizes))


def coalesce_segments(segments: Iterable[LayoutSegment]) -> tuple[LayoutSegment, ...]:
    """Merge neighbours that are contiguous both globally and locally.

    Parity: ``matrix_fsdp/kernels/segment_fusion.py:1-29``.
    """
    out: list[LayoutSegment] = []
    for seg in segments:
        if seg.numel == 0:
            continue
        if out and out[-1].global_end == seg.global_start and out[-1].local_end == seg.local_start:
            prev = out.pop()
            out.append(LayoutSegment(prev.global_start, seg.global_end, prev.local_start))
        else:
            out.append(seg)
    return tuple(out)
