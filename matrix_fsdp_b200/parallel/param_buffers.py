"""Descriptors of how a unit's parameter buffer is communicated (not transports themselves).

``StaticParamBuffer`` describes equal / padded layouts (one collective on rank-major chunks);
``ElasticParamBuffer`` describes owner / uneven layouts: it precomputes the communication plan
(coalesced per-rank segments, whether every rank's shard is one chunk in rank order) and a
workspace plan.  For library collectives the workspace is the padded ``[W, max_shard]`` staging
buffer; the peer kernels need none, since they read ``(peer, offset, length)`` ranges in place —
the plan's ``peer_pull_table`` is exactly what those kernels consume.

Parity: ``matrix_fsdp/runtime/static_param_buffer.py:1-207`` and
``runtime/elastic_param_buffer.py:1-578``.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..core.layout import LayoutSegment, coalesce_segments, rank_segments_are_rank_contiguous_chunks
from .workspace_cache import CommWorkspaceCache, CommWorkspaceLease


def _segments_from_sizes(sizes: tuple[int, ...]) -> tuple[tuple[LayoutSegment, ...], ...]:
    out, cur = [], 0
    for s in sizes:
        out.append((LayoutSegment(cur, cur + s, 0),) if s else ())
        cur += s
    return tuple(out)


@dataclass(frozen=True)
class _LayoutStats:
    shard_sizes: tuple[int, ...]
    rank_segments: tuple[tuple[LayoutSegment, ...], ...] | None = None

    def __post_init__(self) -> None:
        if self.rank_segments is None:
            object.__setattr__(self, "rank_segments", _segments_from_sizes(self.shard_sizes))

    world_size = property(lambda s: len(s.shard_sizes))
    total_shard_numel = property(lambda s: sum(s.shard_sizes))
    max_shard_size = property(lambda s: max(s.shard_sizes, default=0))
    min_shard_size = property(lambda s: min(s.shard_sizes, default=0))
    padded_numel = property(lambda s: s.world_size * s.max_shard_size)
    padding_waste_numel = property(lambda s: max(s.padded_numel - s.total_shard_numel, 0))
    segment_count = property(lambda s: sum(len(r) for r in s.rank_segments))
    max_segments_per_rank = property(lambda s: max((len(r) for r in s.rank_segments), default=0))

    @property
    def padding_waste_ratio(self) -> float:
        return self.padding_waste_numel / self.total_shard_numel if self.total_shard_numel else 0.0

    @property
    def owner_imbalance_ratio(self) -> float:
        mean = self.total_shard_numel / self.world_size if self.world_size else 0.0
        return self.max_shard_size / mean if mean else 0.0

    @property
    def rank_chunk_fast_path(self) -> bool:
        return all(len(r) <= 1 for r in self.rank_segments)

    @property
    def packed_rank_shards_are_full_tensor_order(self) -> bool:
        return rank_segments_are_rank_contiguous_chunks(self.rank_segments)

    def as_summary(self) -> dict[str, object]:
        return {
            "world_size": self.world_size, "total_shard_numel": self.total_shard_numel,
            "max_shard_size": self.max_shard_size, "min_shard_size": self.min_shard_size,
            "padded_numel": self.padded_numel, "padding_waste_numel": self.padding_waste_numel,
            "padding_waste_ratio": self.padding_waste_ratio, "owner_imbalance_ratio": self.owner_imbalance_ratio,
            "segment_count": self.segment_count, "max_segments_per_rank": self.max_segments_per_rank,
            "rank_chunk_fast_path": self.rank_chunk_fast_path,
            "packed_rank_shards_are_full_tensor_order": self.packed_rank_shards_are_full_tensor_order,
        }


class StaticParamBufferLayout(_LayoutStats):
    pass


class ElasticParamBufferLayout(_LayoutStats):
    def build_communication_plan(self) -> "ElasticCommunicationPlan":
        coalesced = tuple(coalesce_segments(r) for r in self.rank_segments)
        chunks = tuple(
            ElasticRankChunk(rank, seg.global_start, seg.global_end, seg.local_start)
            for rank, segs in enumerate(coalesced) for seg in segs)
        fast = all(len(r) <= 1 for r in coalesced)
        return ElasticCommunicationPlan(self.rank_segments, coalesced, chunks,
                                        tuple(self.shard_sizes) if fast else None)


@dataclass(frozen=True)
class ElasticRankChunk:
    rank: int
    global_start: int
    global_end: int
    local_start: int

    @property
    def numel(self) -> int:
        return self.global_end - self.global_start

    def as_segment(self) -> LayoutSegment:
        return LayoutSegment(self.global_start, self.global_end, self.local_start)


@dataclass(frozen=True)
class ElasticCommunicationPlan:
    rank_segments: tuple[tuple[LayoutSegment, ...], ...]
    coalesced_rank_segments: tuple[tuple[LayoutSegment, ...], ...]
    rank_chunks: tuple[ElasticRankChunk, ...]
    rank_chunk_shard_sizes: tuple[int, ...] | None

    world_size = property(lambda s: len(s.rank_segments))
    segment_count = property(lambda s: sum(len(r) for r in s.rank_segments))
    coalesced_segment_count = property(lambda s: sum(len(r) for r in s.coalesced_rank_segments))
    max_segments_per_rank = property(lambda s: max((len(r) for r in s.rank_segments), default=0))
    max_coalesced_segments_per_rank = property(lambda s: max((len(r) for r in s.coalesced_rank_segments), default=0))
    rank_chunk_count = property(lambda s: len(s.rank_chunks))
    nonempty_rank_chunk_count = property(lambda s: sum(1 for c in s.rank_chunks if c.numel))

    def peer_pull_table(self) -> tuple[tuple[int, int, int, int], ...]:
        """(peer, peer_local_offset, global_offset, numel) rows: what an all-gather pull kernel reads."""
        return tuple((c.rank, c.local_start, c.global_start, c.numel) for c in self.rank_chunks if c.numel)

    def as_summary(self) -> dict[str, object]:
        return {
            "communication_segment_count": self.segment_count,
            "communication_coalesced_segment_count": self.coalesced_segment_count,
            "communication_max_segments_per_rank": self.max_segments_per_rank,
            "communication_max_coalesced_segments_per_rank": self.max_coalesced_segments_per_rank,
            "communication_rank_chunk_count": self.rank_chunk_count,
            "communication_nonempty_rank_chunk_count": self.nonempty_rank_chunk_count,
            "communication_rank_chunk_fast_path": self.rank_chunk_shard_sizes is not None,
        }


@dataclass(frozen=True)
class _WorkspacePlan:
    total_numel: int
    padded_numel: int
    needs_workspace: bool
    kind: str

    @property
    def preferred_workspace_kind(self) -> str:
        return self.kind

    @property
    def preferred_workspace_numel(self) -> int:
        if not self.needs_workspace:
            return 0
        return self.padded_numel if self.kind == "padded_rank_chunks" else self.total_numel

    @property
    def padding_waste_ratio(self) -> float:
        return max(self.padded_numel - self.total_numel, 0) / self.total_numel if self.total_numel else 0.0

    def as_summary(self) -> dict[str, object]:
        return {"workspace_kind": self.kind, "workspace_needed": self.needs_workspace,
                "workspace_preferred_numel": self.preferred_workspace_numel,
                "workspace_padding_waste_ratio": self.padding_waste_ratio}


class StaticParamBufferWorkspacePlan(_WorkspacePlan):
    pass


class ElasticParamBufferWorkspacePlan(_WorkspacePlan):
    pass


ElasticParamBufferWorkspace = CommWorkspaceCache
ElasticParamBufferWorkspaceLease = CommWorkspaceLease


def _effective_gather_backend(strategy: str, transport_kind: str, can_direct: bool) -> str:
    if transport_kind == "peer":
        return "peer_pull"
    if transport_kind == "local":
        return "local_copy"
    if strategy not in ("auto", "all_gather"):
        return strategy
    return "all_gather_into_tensor" if can_direct else "padded_all_gather"


@dataclass(frozen=True)
class StaticParamBuffer:
    layout: StaticParamBufferLayout
    total_numel: int

    def workspace_plan(self, *, can_direct_all_gather: bool) -> StaticParamBufferWorkspacePlan:
        return StaticParamBufferWorkspacePlan(self.total_numel, self.layout.padded_numel, not can_direct_all_gather,
                                              "none" if can_direct_all_gather else "padded_rank_chunks")

    def effective_param_gather_backend(self, *, param_gather_strategy: str, can_direct_all_gather: bool,
                                       transport_kind: str = "torch_dist") -> str:
        return _effective_gather_backend(param_gather_strategy, transport_kind, can_direct_all_gather)

    def communication_summary(self, *, param_gather_strategy: str, matrix_collective_backend: str,
                              can_direct_all_gather: bool, transport_kind: str = "torch_dist") -> dict[str, object]:
        return {
            "param_buffer_type": "static", "param_gather_strategy": param_gather_strategy,
            "matrix_collective_backend": matrix_collective_backend,
            "effective_param_gather_backend": self.effective_param_gather_backend(
                param_gather_strategy=param_gather_strategy, can_direct_all_gather=can_direct_all_gather,
                transport_kind=transport_kind),
            "effective_grad_reduce_backend": {"peer": "peer_pull_reduce", "local": "local_copy"}.get(
                transport_kind, "reduce_scatter_tensor" if can_direct_all_gather else "padded_reduce_scatter"),
            "owner_segment_collectives": False,
            **self.layout.as_summary(),
            **self.workspace_plan(can_direct_all_gather=can_direct_all_gather).as_summary(),
        }


@dataclass(frozen=True)
class ElasticParamBuffer:
    layout: ElasticParamBufferLayout
    total_numel: int
    workspace: CommWorkspaceCache = field(default_factory=CommWorkspaceCache)
    communication_plan: ElasticCommunicationPlan = field(init=False)

    def __post_init__(self) -> None:
        object.__setattr__(self, "communication_plan", self.layout.build_communication_plan())

    def rank_chunk_workspace_numel(self, *, compact: bool) -> int:
        return self.total_numel if compact else self.layout.padded_numel

    def acquire_rank_chunk_workspace(self, *, dtype: torch.dtype, device: torch.device,
                                     compact: bool = False) -> CommWorkspaceLease:
        return self.workspace.lease(self.rank_chunk_workspace_numel(compact=compact), dtype, device)

    def workspace_plan(self, *, can_direct_all_gather: bool, transport_kind: str = "torch_dist",
                       compact: bool = False) -> ElasticParamBufferWorkspacePlan:
        needs = not can_direct_all_gather and transport_kind == "torch_dist"
        kind = "none" if not needs else ("compact_rank_chunks" if compact else "padded_rank_chunks")
        return ElasticParamBufferWorkspacePlan(self.total_numel, self.layout.padded_numel, needs, kind)

    def effective_param_gather_backend(self, *, param_gather_strategy: str, can_direct_all_gather: bool,
                                       transport_kind: str = "torch_dist") -> str:
        return _effective_gather_backend(param_gather_strategy, transport_kind, can_direct_all_gather)

    def communication_summary(self, *, param_gather_strategy: str, matrix_collective_backend: str,
                              can_direct_all_gather: bool, transport_kind: str = "torch_dist",
                              reduce_impl: str = "auto") -> dict[str, object]:
        reduce_backend = {"peer": "peer_pull_reduce", "local": "local_copy"}.get(
            transport_kind, "owner_reduce" if reduce_impl in ("owner_reduce", "reduce") else "padded_reduce_scatter")
        return {
            "param_buffer_type": "elastic", "param_gather_strategy": param_gather_strategy,
            "matrix_collective_backend": matrix_collective_backend,
            "effective_param_gather_backend": self.effective_param_gather_backend(
                param_gather_strategy=param_gather_strategy, can_direct_all_gather=can_direct_all_gather,
                transport_kind=transport_kind),
            "effective_grad_reduce_backend": reduce_backend,
            "owner_segment_collectives": transport_kind != "local",
            **self.layout.as_summary(), **self.communication_plan.as_summary(),
            **self.workspace_plan(can_direct_all_gather=can_direct_all_gather, transport_kind=transport_kind).as_summary(),
            **{f"workspace_{k}": v for k, v in self.workspace.stats().items()},
        }


def describe_unit_param_buffer(unit) -> StaticParamBuffer | ElasticParamBuffer:
    """The descriptor the unit's transports work from (built with its segment tables): static for equal
    rank-ordered chunks, elastic otherwise."""
    fb = unit.flat_buffer
    if getattr(fb.tables, "param_buffer", None) is not None:
        return fb.tables.param_buffer
    if fb.tables.equal_contiguous or fb.world_size == 1:
        return StaticParamBuffer(StaticParamBufferLayout(fb.tables.shard_sizes, fb.tables.rank_segments), fb.total_numel)
    return ElasticParamBuffer(ElasticParamBufferLayout(fb.tables.shard_sizes, fb.tables.rank_segments), fb.total_numel)
