"""Segment collectives over ``torch.distributed`` (NCCL or Gloo) with async handles.

These are the portable transport: they serve CPU/Gloo runs, multi-node NCCL runs and act
as the functional baseline for the peer-memory kernels in
:mod:`matrix_fsdp_b200.parallel.peer`.  Every function also has a single-rank branch
(``group is None``) that degenerates to local copies so the whole lifecycle runs in one
process.

Async pattern: when a CUDA ``stream`` is given the blocking collective is enqueued on that
stream (after it has waited for the caller's stream) and the handle's ``wait()`` makes the
current stream wait for the recorded event; without a stream the ``async_op`` work handle
is kept.  Parity: ``matrix_fsdp/runtime/collectives.py:26-1046``.
"""
from __future__ import annotations

import os
from collections.abc import Sequence
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..core.layout import LayoutSegment, rank_segments_are_rank_contiguous_chunks

VALIDATE_SIGNATURE_ENV = "MFSDP_VALIDATE_OWNER_COLLECTIVE_SIGNATURE"


class MatrixCollectiveHandle:
    """Completion handle of one enqueued collective (or a batch of them)."""

    def __init__(self, works=(), event=None, post=None, info: dict | None = None) -> None:
        self._works = [w for w in works if w is not None]
        self._event = event
        self._post = post
        self.info = info or {}
        self.done = False
        self.span = None          # device-timeline record (device_timeline.CollectiveSpan) when enabled

    def wait(self) -> None:
        if self.done:
            return
        if self.span is not None:
            from . import device_timeline as _tl

            _tl.begin_wait(self.span)
        for w in self._works:
            w.wait()
        if self._event is not None:
            torch.cuda.current_stream().wait_event(self._event)
        if self.span is not None:
            _tl.end_wait(self.span)
        if self._post is not None:
            self._post()
        self.done = True

    def is_completed(self) -> bool:
        if self.done:
            return True
        if self._event is not None:
            return self._event.query()
        return all(w.is_completed() for w in self._works)


class MatrixTensorCollectiveHandle(MatrixCollectiveHandle):
    """Handle that also names the tensor the collective produces."""

    def __init__(self, tensor: torch.Tensor, **kw) -> None:
        super().__init__(**kw)
        self.tensor = tensor


def _world(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _rank(group) -> int:
    return 0 if group is None else dist.get_rank(group)


def _run(fn, *, stream, info) -> MatrixCollectiveHandle:
    """Run ``fn`` (which issues blocking collectives) on ``stream`` and return its handle."""
    from . import device_timeline as _tl

    if stream is not None:
        stream.wait_stream(torch.cuda.current_stream())
        span = _tl.open_span("", info.get("kind", ""), stream, impl=info.get("impl", ""), nbytes=info.get("bytes", 0))
        with torch.cuda.stream(stream):
            fn()
            _tl.close_span(span, stream)
            ev = torch.cuda.Event()
            ev.record(stream)
        info["sync_mode"] = "stream_event"
        h = MatrixCollectiveHandle(event=ev, info=info)
        h.span = span
        return h
    fn()
    info["sync_mode"] = "blocking"
    return MatrixCollectiveHandle(info=info)


@dataclass
class SegmentTables:
    """Everything a transport needs about one unit's layout, precomputed once."""

    total_numel: int
    world_size: int
    rank: int
    rank_segments: tuple[tuple[LayoutSegment, ...], ...]
    shard_sizes: tuple[int, ...]
    max_shard: int = 0
    equal_contiguous: bool = False
    rank_contiguous: bool = False
    signature: tuple = field(default=(), repr=False)
    # Descriptor of how this layout is communicated (param_buffers.StaticParamBuffer for equal rank-ordered
    # chunks, ElasticParamBuffer otherwise): the transports take their copy tables and workspace sizes from it.
    param_buffer: object = field(default=None, repr=False, compare=False)

    @classmethod
    def build(cls, total_numel: int, rank_segments: Sequence[Sequence[LayoutSegment]], rank: int) -> "SegmentTables":
        from .param_buffers import (ElasticParamBuffer, ElasticParamBufferLayout, StaticParamBuffer,
                                    StaticParamBufferLayout)

        segs = tuple(tuple(s for s in rs if s.numel > 0) for rs in rank_segments)
        sizes = tuple(sum(s.numel for s in rs) for rs in segs)
        contiguous = rank_segments_are_rank_contiguous_chunks(segs)
        equal = contiguous and len(set(sizes)) == 1 and sizes[0] * len(sizes) == total_numel
        sig = (total_numel, tuple(tuple((s.global_start, s.global_end, s.local_start) for s in rs) for rs in segs))
        if equal or len(segs) == 1:
            desc = StaticParamBuffer(StaticParamBufferLayout(sizes, segs), int(total_numel))
        else:
            desc = ElasticParamBuffer(ElasticParamBufferLayout(sizes, segs), int(total_numel))
        return cls(int(total_numel), len(segs), int(rank), segs, sizes, max(sizes, default=0), equal, contiguous, sig,
                   desc)

    @property
    def my_segments(self) -> tuple[LayoutSegment, ...]:
        return self.rank_segments[self.rank]

    def pull_rows(self) -> tuple[tuple[int, int, int, int], ...]:
        """(owner rank, offset in the owner's shard, offset in the flat space, numel) of every run an
        all-gather copies, adjacent runs merged: the elastic descriptor's communication plan, or one row
        per rank for equal chunks."""
        plan = getattr(self.param_buffer, "communication_plan", None)
        if plan is not None:
            return plan.peer_pull_table()
        return tuple((r, s.local_start, s.global_start, s.numel) for r, rs in enumerate(self.rank_segments) for s in rs)

    def staging_numel(self, transport_kind: str = "torch_dist") -> int:
        """Elements of the rank-major staging buffer a library collective needs for this layout (0: none)."""
        if self.param_buffer is None:
            return 0 if self.equal_contiguous else self.world_size * self.max_shard
        kw = {"can_direct_all_gather": self.equal_contiguous}
        if hasattr(self.param_buffer, "communication_plan"):
            kw["transport_kind"] = transport_kind
        return self.param_buffer.workspace_plan(**kw).preferred_workspace_numel


def validate_layout_signature(tables: SegmentTables, group) -> None:
    """Debug aid: all ranks must agree on the layout before issuing per-owner collectives."""
    if group is None or os.environ.get(VALIDATE_SIGNATURE_ENV, "0") in ("", "0"):
        return
    sigs: list = [None] * _world(group)
    dist.all_gather_object(sigs, hash(tables.signature), group=group)
    if len(set(sigs)) != 1:
        raise RuntimeError(f"Layout signature differs across ranks: {sigs}")


# --------------------------------------------------------------------------- local copies
def scatter_local_segments(shard: torch.Tensor, full: torch.Tensor, segments: Sequence[LayoutSegment]) -> None:
    """``full[g0:g1] = shard[l0:l1]`` for every segment."""
    for s in segments:
        full[s.global_start:s.global_end].copy_(shard[s.local_start:s.local_end])


def gather_local_segments(full: torch.Tensor, shard: torch.Tensor, segments: Sequence[LayoutSegment]) -> None:
    """``shard[l0:l1] = full[g0:g1]`` for every segment."""
    for s in segments:
        shard[s.local_start:s.local_end].copy_(full[s.global_start:s.global_end])


# --------------------------------------------------------------------------- all-gather
def all_gather_equal_1d_into_async(shard: torch.Tensor, full: torch.Tensor, group, *, stream=None) -> MatrixCollectiveHandle:
    """Equal rank-ordered shards straight into the full buffer (no staging)."""
    info = {"kind": "all_gather", "impl": "all_gather_into_tensor", "bytes": full.numel() * full.element_size(), "count": 1}
    if group is None:
        full.copy_(shard)
        return MatrixCollectiveHandle(info={**info, "impl": "local_copy", "sync_mode": "local"})
    return _run(lambda: dist.all_gather_into_tensor(full, shard, group=group), stream=stream, info=info)


def all_gather_matrix_1d_into_async(shard: torch.Tensor, full: torch.Tensor, tables: SegmentTables, group, *,
                                    stream=None, workspace: torch.Tensor | None = None) -> MatrixCollectiveHandle:
    """Uneven layouts: pad shards to the largest, gather, then unpad into the full buffer."""
    W, mx = tables.world_size, tables.max_shard
    info = {"kind": "all_gather", "impl": "padded_all_gather", "bytes": W * mx * full.element_size(), "count": 1}
    if group is None:
        scatter_local_segments(shard, full, tables.my_segments)
        return MatrixCollectiveHandle(info={**info, "impl": "local_copy", "sync_mode": "local"})

    def body():
        ws = workspace if workspace is not None else torch.empty(W * mx, dtype=full.dtype, device=full.device)
        send = ws.new_zeros(mx) if shard.numel() != mx else shard
        if shard.numel() != mx:
            send[: shard.numel()].copy_(shard)
        dist.all_gather_into_tensor(ws[: W * mx], send, group=group)
        for r in range(W):
            scatter_local_segments(ws[r * mx:(r + 1) * mx], full, tables.rank_segments[r])

    return _run(body, stream=stream, info=info)


def broadcast_rank_segments_1d_into_async(shard: torch.Tensor, full: torch.Tensor, tables: SegmentTables, group, *,
                                          stream=None) -> MatrixCollectiveHandle:
    """Owner broadcast: every rank broadcasts its packed shard; receivers scatter it into place."""
    W = tables.world_size
    info = {"kind": "all_gather", "impl": "owner_broadcast", "bytes": full.numel() * full.element_size(),
            "count": sum(1 for s in tables.shard_sizes if s)}
    if group is None:
        scatter_local_segments(shard, full, tables.my_segments)
        return MatrixCollectiveHandle(info={**info, "impl": "local_copy", "sync_mode": "local"})
    validate_layout_signature(tables, group)

    def body():
        for r in range(W):
            n = tables.shard_sizes[r]
            if n == 0:
                continue
            contiguous_one = len(tables.rank_segments[r]) == 1
            if contiguous_one:
                seg = tables.rank_segments[r][0]
                view = full[seg.global_start:seg.global_end]
                if r == tables.rank:
                    view.copy_(shard[:n])
                dist.broadcast(view, src=dist.get_global_rank(group, r), group=group)
            else:
                buf = shard[:n] if r == tables.rank else torch.empty(n, dtype=full.dtype, device=full.device)
                dist.broadcast(buf, src=dist.get_global_rank(group, r), group=group)
                scatter_local_segments(buf, full, tables.rank_segments[r])

    return _run(body, stream=stream, info=info)


def _is_nccl(group) -> bool:
    try:
        return dist.get_backend(group) == "nccl"
    except Exception:  # noqa: BLE001
        return False


def all_gather_uneven_rank_segments_1d_into_async(shard: torch.Tensor, full: torch.Tensor, tables: SegmentTables, group,
                                                  *, stream=None, workspace: torch.Tensor | None = None,
                                                  ) -> MatrixCollectiveHandle:
    """Uneven list all-gather: ``dist.all_gather`` with one output tensor per rank, each of that rank's
    size.  With rank-contiguous chunks the outputs are views of the full buffer (nothing is staged or
    padded); multi-segment shards land in per-rank staging tensors and are scattered afterwards.

    The list form with unequal sizes exists for NCCL only and cannot carry an empty tensor, so other
    backends take the padded gather and layouts with an empty rank take the owner broadcast
    (``matrix_fsdp/runtime/collectives.py:330-410`` has the same two fall-backs)."""
    if group is None:
        scatter_local_segments(shard, full, tables.my_segments)
        return MatrixCollectiveHandle(info={"kind": "all_gather", "impl": "local_copy", "bytes": 0, "count": 0,
                                            "sync_mode": "local"})
    if any(n == 0 for n in tables.shard_sizes):
        return broadcast_rank_segments_1d_into_async(shard, full, tables, group, stream=stream)
    if not _is_nccl(group):
        return all_gather_matrix_1d_into_async(shard, full, tables, group, stream=stream, workspace=workspace)
    info = {"kind": "all_gather", "impl": "uneven_all_gather", "bytes": full.numel() * full.element_size(), "count": 1}

    def body():
        direct = tables.rank_contiguous
        outs = []
        for r in range(tables.world_size):
            n = tables.shard_sizes[r]
            if direct:
                seg = tables.rank_segments[r][0]
                outs.append(full[seg.global_start:seg.global_end])
            else:
                outs.append(torch.empty(n, dtype=full.dtype, device=full.device))
        dist.all_gather(outs, shard[: tables.shard_sizes[tables.rank]], group=group)
        if not direct:
            for r, buf in enumerate(outs):
                scatter_local_segments(buf, full, tables.rank_segments[r])

    return _run(body, stream=stream, info=info)


def all_gather_by_all_reduce_1d_into_async(shard: torch.Tensor, full: torch.Tensor, tables: SegmentTables, group, *,
                                           stream=None) -> MatrixCollectiveHandle:
    """Diagnostic gather: zero the full buffer, drop the own segments in, sum over ranks.  Moves W times
    the bytes of a real gather; useful to tell a layout problem from a collective problem
    (``matrix_fsdp/kernels/custom_collectives.py:803-838``)."""
    info = {"kind": "all_gather", "impl": "all_reduce_gather", "bytes": full.numel() * full.element_size(), "count": 1}
    if group is None:
        scatter_local_segments(shard, full, tables.my_segments)
        return MatrixCollectiveHandle(info={**info, "impl": "local_copy", "sync_mode": "local"})

    def body():
        full.zero_()
        scatter_local_segments(shard, full, tables.my_segments)
        dist.all_reduce(full, group=group)

    return _run(body, stream=stream, info=info)


def all_gatherv_rank_segments_1d_into_async(shard: torch.Tensor, full: torch.Tensor, tables: SegmentTables, group, *,
                                            stream=None, impl: str = "auto",
                                            workspace: torch.Tensor | None = None) -> MatrixCollectiveHandle:
    """Dispatch on layout shape and ``impl``: equal chunks, padded gather, uneven list gather, owner
    broadcast, or the all-reduce diagnostic."""
    if impl in ("equal", "equal_all_gather") and not tables.equal_contiguous:
        raise RuntimeError("param_gather_strategy='equal_all_gather' requires equal rank-ordered shards.")
    if tables.equal_contiguous and impl in ("auto", "equal", "equal_all_gather"):
        return all_gather_equal_1d_into_async(shard, full, group, stream=stream)
    if impl in ("owner_broadcast", "broadcast"):
        return broadcast_rank_segments_1d_into_async(shard, full, tables, group, stream=stream)
    if impl in ("uneven_all_gather", "uneven"):
        return all_gather_uneven_rank_segments_1d_into_async(shard, full, tables, group, stream=stream,
                                                             workspace=workspace)
    if impl in ("all_reduce", "all_reduce_gather"):
        return all_gather_by_all_reduce_1d_into_async(shard, full, tables, group, stream=stream)
    return all_gather_matrix_1d_into_async(shard, full, tables, group, stream=stream, workspace=workspace)


# --------------------------------------------------------------------------- reduce-scatter
def pack_rank_major_padded(full_grad: torch.Tensor, tables: SegmentTables, out: torch.Tensor | None = None) -> torch.Tensor:
    """``[W, max_shard]`` reduce-scatter input: row r is rank r's packed shard, zero padded."""
    W, mx = tables.world_size, tables.max_shard
    if out is None:
        out = torch.zeros(W * mx, dtype=full_grad.dtype, device=full_grad.device)
    else:
        out.zero_()
    for r in range(W):
        gather_local_segments(full_grad, out[r * mx:(r + 1) * mx], tables.rank_segments[r])
    return out


def reduce_scatter_padded_rank_chunks_1d_async(full_grad: torch.Tensor, out_shard: torch.Tensor,
                                               tables: SegmentTables, group, *, scale: float | None = None,
                                               stream=None, workspace: torch.Tensor | None = None,
                                               ) -> MatrixCollectiveHandle:
    """Sum over ranks of each rank's segments, result on the owning rank, then ``* scale``."""
    W, mx = tables.world_size, tables.max_shard
    n_local = tables.shard_sizes[tables.rank]
    info = {"kind": "reduce_scatter", "impl": "padded_reduce_scatter", "bytes": W * mx * full_grad.element_size(), "count": 1}
    if group is None:
        gather_local_segments(full_grad, out_shard, tables.my_segments)
        if scale is not None and scale != 1.0:
            out_shard.mul_(scale)
        return MatrixCollectiveHandle(info={**info, "impl": "local_copy", "sync_mode": "local"})

    def body():
        if tables.equal_contiguous and out_shard.dtype == full_grad.dtype:
            dist.reduce_scatter_tensor(out_shard[:n_local], full_grad, group=group)
            info["impl"] = "reduce_scatter_tensor"
        else:
            packed = pack_rank_major_padded(full_grad, tables, workspace)
            recv = torch.empty(mx, dtype=full_grad.dtype, device=full_grad.device)
            dist.reduce_scatter_tensor(recv, packed[: W * mx], group=group)
            out_shard[:n_local].copy_(recv[:n_local])
        if scale is not None and scale != 1.0:
            out_shard[:n_local].mul_(scale)

    return _run(body, stream=stream, info=info)


def reduce_owner_rank_chunks_1d_async(full_grad: torch.Tensor, out_shard: torch.Tensor, tables: SegmentTables, group, *,
                                      scale: float | None = None, stream=None) -> MatrixCollectiveHandle:
    """One ``reduce`` per owner rank (no padding); the owner keeps its packed result."""
    W = tables.world_size
    info = {"kind": "reduce_scatter", "impl": "owner_reduce", "bytes": full_grad.numel() * full_grad.element_size(),
            "count": sum(1 for s in tables.shard_sizes if s)}
    if group is None:
        return reduce_scatter_padded_rank_chunks_1d_async(full_grad, out_shard, tables, None, scale=scale)
    validate_layout_signature(tables, group)

    def body():
        for r in range(W):
            n = tables.shard_sizes[r]
            if n == 0:
                continue
            buf = torch.empty(n, dtype=full_grad.dtype, device=full_grad.device)
            gather_local_segments(full_grad, buf, tables.rank_segments[r])
            dist.reduce(buf, dst=dist.get_global_rank(group, r), group=group)
            if r == tables.rank:
                out_shard[:n].copy_(buf)
                if scale is not None and scale != 1.0:
                    out_shard[:n].mul_(scale)

    return _run(body, stream=stream, info=info)


def reduce_scatter_uneven_rank_chunks_1d_async(full_grad: torch.Tensor, out_shard: torch.Tensor, tables: SegmentTables,
                                               group, *, scale: float | None = None, stream=None,
                                               workspace: torch.Tensor | None = None) -> MatrixCollectiveHandle:
    """Uneven list reduce-scatter: ``dist.reduce_scatter(out, [one view per rank])`` on the compact flat
    gradient, no padding.  NCCL only and every rank needs at least one element; otherwise the padded
    path runs (``matrix_fsdp/runtime/collectives.py:609-675``)."""
    if group is None or not _is_nccl(group) or any(n == 0 for n in tables.shard_sizes) \
            or out_shard.dtype != full_grad.dtype:
        return reduce_scatter_padded_rank_chunks_1d_async(full_grad, out_shard, tables, group, scale=scale,
                                                          stream=stream, workspace=workspace)
    info = {"kind": "reduce_scatter", "impl": "uneven_reduce_scatter",
            "bytes": full_grad.numel() * full_grad.element_size(), "count": 1}
    n_local = tables.shard_sizes[tables.rank]

    def body():
        ins = []
        for r in range(tables.world_size):
            if tables.rank_contiguous:
                seg = tables.rank_segments[r][0]
                ins.append(full_grad[seg.global_start:seg.global_end])
            else:
                buf = torch.empty(tables.shard_sizes[r], dtype=full_grad.dtype, device=full_grad.device)
                gather_local_segments(full_grad, buf, tables.rank_segments[r])
                ins.append(buf)
        dist.reduce_scatter(out_shard[:n_local], ins, group=group)
        if scale is not None and scale != 1.0:
            out_shard[:n_local].mul_(scale)

    return _run(body, stream=stream, info=info)


def param_segment_tables(tables: SegmentTables, start: int, end: int) -> tuple[SegmentTables, int]:
    """Tables of the sub-range ``[start, end)`` of the flat space (one parameter), with offsets relative
    to ``start`` and each rank's pieces packed from local offset 0; also returns where this rank's first
    piece sits in its full local shard."""
    per_rank, my_local = [], None
    for r, segs in enumerate(tables.rank_segments):
        out, cursor = [], 0
        for sg in segs:
            a, b = max(sg.global_start, start), min(sg.global_end, end)
            if a >= b:
                continue
            if r == tables.rank and my_local is None:
                my_local = sg.local_start + (a - sg.global_start)
            out.append(LayoutSegment(a - start, b - start, cursor))
            cursor += b - a
        per_rank.append(out)
    return SegmentTables.build(end - start, per_rank, tables.rank), (my_local if my_local is not None else 0)


def reduce_scatter_per_param_async(full_grad: torch.Tensor, out_shard: torch.Tensor, tables: SegmentTables,
                                  param_ranges: Sequence[tuple[int, int]], group, *, scale: float | None = None,
                                  stream=None) -> MatrixCollectiveHandle:
    """One reduce-scatter per parameter (``param_ranges``: [start, end) of each parameter in the flat
    space), each over that parameter's own rank chunks.  A diagnostic strategy: it isolates one
    parameter's gradient traffic and costs one collective per parameter
    (``matrix_fsdp/runtime/flat_buffer.py:522-552``, ``runtime/collectives.py:993-1029``)."""
    info = {"kind": "reduce_scatter", "impl": "per_param_reduce_scatter",
            "bytes": full_grad.numel() * full_grad.element_size(), "count": len(param_ranges)}

    def one(start: int, end: int) -> None:
        sub, _ = param_segment_tables(tables, start, end)
        n_mine = sub.shard_sizes[sub.rank]
        piece = torch.empty(max(n_mine, 1), dtype=full_grad.dtype, device=full_grad.device)[:n_mine]
        src = full_grad[start:end]
        if group is None:
            gather_local_segments(src, piece, sub.my_segments)
        else:
            W, mx = sub.world_size, max(sub.max_shard, 1)
            packed = pack_rank_major_padded(src, sub) if sub.max_shard else src.new_zeros(W * mx)
            recv = torch.empty(mx, dtype=full_grad.dtype, device=full_grad.device)
            dist.reduce_scatter_tensor(recv, packed[: W * mx], group=group)
            piece.copy_(recv[:n_mine])
        # the parameter's pieces go back to where the unit-wide layout keeps them in the local shard
        cursor = 0
        for sg in tables.my_segments:
            a, b = max(sg.global_start, start), min(sg.global_end, end)
            if a >= b:
                continue
            dst = out_shard[sg.local_start + (a - sg.global_start): sg.local_start + (b - sg.global_start)]
            dst.copy_(piece[cursor:cursor + (b - a)])
            if scale is not None and scale != 1.0:
                dst.mul_(scale)
            cursor += b - a

    def body():
        for start, end in param_ranges:
            one(int(start), int(end))

    if group is None:
        body()
        return MatrixCollectiveHandle(info={**info, "sync_mode": "local"})
    return _run(body, stream=stream, info=info)


def reduce_scatterv_owner_rank_chunks_1d_async(full_grad, out_shard, tables, group, *, scale=None, stream=None,
                                               impl: str = "auto", workspace=None) -> MatrixCollectiveHandle:
    if impl in ("owner_reduce", "reduce", "native_reduce"):
        return reduce_owner_rank_chunks_1d_async(full_grad, out_shard, tables, group, scale=scale, stream=stream)
    if impl in ("uneven_reduce_scatter", "uneven"):
        return reduce_scatter_uneven_rank_chunks_1d_async(full_grad, out_shard, tables, group, scale=scale,
                                                          stream=stream, workspace=workspace)
    return reduce_scatter_padded_rank_chunks_1d_async(full_grad, out_shard, tables, group, scale=scale,
                                                      stream=stream, workspace=workspace)


def all_reduce_full_grad(tensor: torch.Tensor, group, *, scale: float | None = None) -> torch.Tensor:
    """In-place sum over ``group`` (HSDP replicate step and diagnostics), then ``* scale``."""
    if group is not None and _world(group) > 1:
        dist.all_reduce(tensor, group=group)
    if scale is not None and scale != 1.0:
        tensor.mul_(scale)
    return tensor
