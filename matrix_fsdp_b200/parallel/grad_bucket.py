"""Gradient bucket of one unit: full-size gradients laid out in the unit's flat order.

The bucket is the reduce-scatter source.  Gradients get into it in one of two ways:

* *direct write*: ops of this package (``ops.functional.linear`` and friends) write their
  weight gradient straight into ``grad_view(fqn)`` from the wgrad GEMM epilogue, so there is
  no copy-in at all;
* *copy-in*: for arbitrary ``nn.Module`` code the post-accumulate-grad hook hands the
  autograd-produced ``param.grad`` to :meth:`copy_in`, which uses one fused call when the
  layout allows (``torch.cat(out=)`` for whole buckets, ``torch._foreach_copy_`` otherwise).

For transports that need a rank-major ``[W, max_shard]`` input, :meth:`pack_rank_major`
produces it with the fast paths ``flat_contiguous`` (plain view), ``fsdp2_chunk``
(``torch._chunk_cat``) and ``foreach_copy``, else zero + per-segment copies.

Parity: ``matrix_fsdp/runtime/grad_bucket.py:1-225``.
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import torch

from ..core.layout import LayoutSegment
from .collectives import SegmentTables, gather_local_segments


@dataclass(frozen=True)
class BucketParam:
    fqn: str
    offset: int
    numel: int

    @property
    def end(self) -> int:
        return self.offset + self.numel


def classify_bucket_layout(tables: SegmentTables, params: Sequence[BucketParam]) -> str:
    """Name of the cheapest packing path for this layout."""
    if tables.equal_contiguous or tables.world_size == 1:
        return "flat_contiguous"
    W = tables.world_size
    # fsdp2_chunk: every param cut into W equal chunks, rank r's row = [p0 chunk r, p1 chunk r, ...]
    ok = all(p.numel % W == 0 for p in params)
    if ok:
        for r in range(W):
            want, local = [], 0
            for p in params:
                c = p.numel // W
                want.append(LayoutSegment(p.offset + r * c, p.offset + (r + 1) * c, local))
                local += c
            if tuple(want) != tuple(tables.rank_segments[r]):
                ok = False
                break
        if ok:
            return "fsdp2_chunk"
    # foreach_copy: every segment covers whole params only
    starts = {p.offset for p in params}
    ends = {p.end for p in params}
    if all(s.global_start in starts and s.global_end in ends for rs in tables.rank_segments for s in rs):
        return "foreach_copy"
    return "segment_copy"


class MatrixGradBucket:
    def __init__(self, tables: SegmentTables, params: Sequence[BucketParam], dtype: torch.dtype,
                 device: torch.device) -> None:
        self.tables = tables
        self.params = tuple(params)
        self.dtype = dtype
        self.device = device
        self.layout_class = classify_bucket_layout(tables, self.params)
        self.buffer: torch.Tensor | None = None
        self.accumulating = False
        self._by_fqn = {p.fqn: p for p in self.params}

    # -- storage ---------------------------------------------------------------
    def attach(self, buffer: torch.Tensor) -> None:
        assert buffer.numel() >= self.tables.total_numel
        self.buffer = buffer[: self.tables.total_numel]

    def ensure(self) -> torch.Tensor:
        if self.buffer is None:
            self.buffer = torch.empty(self.tables.total_numel, dtype=self.dtype, device=self.device)
        return self.buffer

    def release(self) -> None:
        self.buffer = None
        self.accumulating = False

    def grad_view(self, fqn: str, shape=None) -> torch.Tensor:
        p = self._by_fqn[fqn]
        v = self.ensure()[p.offset:p.end]
        return v.view(shape) if shape is not None else v

    # -- copy-in -----------------------------------------------------------------
    def copy_in(self, grads: Sequence[torch.Tensor | None], *, accumulate: bool = False) -> str:
        """Write one full-size gradient per param (``None`` = zero) into the bucket."""
        buf = self.ensure()
        assert len(grads) == len(self.params)
        if accumulate:
            for p, g in zip(self.params, grads):
                if g is not None:
                    buf[p.offset:p.end].add_(g.reshape(-1).to(buf.dtype))
            return "accumulate"
        if all(g is not None and g.dtype == buf.dtype for g in grads):
            flat = [g.reshape(-1) for g in grads]
            contiguous = all(a.end == b.offset for a, b in zip(self.params, self.params[1:]))
            if contiguous and self.params and self.params[0].offset == 0:
                torch.cat(flat, out=buf)
                return "cat"
            torch._foreach_copy_([buf[p.offset:p.end] for p in self.params], flat)
            return "foreach_copy"
        for p, g in zip(self.params, grads):
            if g is None:
                buf[p.offset:p.end].zero_()
            else:
                buf[p.offset:p.end].copy_(g.reshape(-1))
        return "slice_copy"

    # -- rank-major packing -------------------------------------------------------
    def pack_rank_major(self, grads: Sequence[torch.Tensor] | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
        """``[W * max_shard]`` reduce-scatter input (row r = rank r's packed shard, zero padded)."""
        t = self.tables
        W, mx = t.world_size, t.max_shard
        if grads is not None and self.layout_class == "fsdp2_chunk":
            out = out if out is not None else torch.empty(W * mx, dtype=self.dtype, device=self.device)
            torch._chunk_cat([g.reshape(-1) for g in grads], dim=0, num_chunks=W, out=out.view(W, mx))
            return out
        if grads is not None:
            self.copy_in(grads)
        buf = self.ensure()
        if self.layout_class == "flat_contiguous":
            return buf
        out = out if out is not None else torch.empty(W * mx, dtype=self.dtype, device=self.device)
        out.zero_()
        for r in range(W):
            gather_local_segments(buf, out[r * mx:(r + 1) * mx], t.rank_segments[r])
        return out
