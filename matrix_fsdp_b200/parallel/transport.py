"""Transports: how a unit's shards and gradients move between ranks.

A transport owns the *data plane* of one shard group.  The flat-buffer runtime only ever
calls ``gather`` (shards → full parameters), ``reduce`` (full gradients → owned shard of the
mean) and the two allocation hooks, so the same lifecycle code runs on:

* :class:`LocalTransport`      – one rank: copies (or pure aliasing);
* :class:`TorchDistTransport`  – NCCL / Gloo collectives (portable baseline, CPU tests);
* ``PeerTransport`` (:mod:`matrix_fsdp_b200.parallel.peer`) – hand-written sm_100a kernels
  that pull peer shards / reduce peer gradients over NVLink from IPC-mapped memory.

The reference hard-wires ``torch.distributed`` calls into its flat buffer
(``matrix_fsdp/runtime/flat_buffer.py:304-382,629-818``) and selects implementations through
environment variables (``kernels/custom_collectives.py:24-52``); here that choice is one
object picked at construction.
"""
from __future__ import annotations

import os

import torch

from .collectives import (MatrixCollectiveHandle, SegmentTables, all_gatherv_rank_segments_1d_into_async,
                          all_reduce_full_grad, gather_local_segments,
                          reduce_scatterv_owner_rank_chunks_1d_async, scatter_local_segments)
from .workspace_cache import CommWorkspaceCache

GATHER_IMPL_ENV = "MFSDP_ALLGATHERV_IMPL"
REDUCE_IMPL_ENV = "MFSDP_REDUCE_SCATTERV_IMPL"
TRANSPORT_ENV = "MFSDP_TRANSPORT"


class LocalTransport:
    kind = "local"
    needs_symmetric_buffers = False
    accumulates_fp32 = True   # a single rank only copies; copy_ converts dtypes on the way

    def __init__(self) -> None:
        self.group = None

    def alloc_persistent(self, numel: int, dtype: torch.dtype, device: torch.device, tag: str = "",
                         symmetric_numel: int | None = None) -> torch.Tensor:
        return torch.empty(numel, dtype=dtype, device=device)

    def acquire_grad_buffer(self, unit_key, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        return torch.empty(numel, dtype=dtype, device=device)

    def release_grad_buffer(self, unit_key, buf: torch.Tensor) -> None:
        pass

    def gather(self, shard, full, tables: SegmentTables, *, stream=None, unit_key=None) -> MatrixCollectiveHandle:
        scatter_local_segments(shard, full, tables.my_segments)
        return MatrixCollectiveHandle(info={"kind": "all_gather", "impl": "local_copy", "backend": self.kind,
                                            "bytes": full.numel() * full.element_size(), "count": 0,
                                            "sync_mode": "local"})

    def reduce(self, full_grad, out_shard, tables: SegmentTables, *, scale=None, stream=None,
               unit_key=None) -> MatrixCollectiveHandle:
        gather_local_segments(full_grad, out_shard, tables.my_segments)
        if scale is not None and scale != 1.0:
            out_shard.mul_(scale)
        return MatrixCollectiveHandle(info={"kind": "reduce_scatter", "impl": "local_copy", "backend": self.kind,
                                            "bytes": 0, "count": 0, "sync_mode": "local"})

    def all_reduce(self, tensor, group, *, scale=None):
        return all_reduce_full_grad(tensor, group, scale=scale)

    def local_update(self, grad: torch.Tensor, update: dict, *, scale=None, stream=None) -> MatrixCollectiveHandle:
        """One rank: the gradient bucket already is the reduced gradient, so the AdamW update of a unit can run
        as soon as its backward has finished -- on ``stream``, beside the backward GEMMs of the next unit (a
        bandwidth-bound kernel next to compute-bound ones) instead of after the whole backward pass.  ``update``
        holds master / moments / bf16 shard and the hyper-parameters (``optim.flat.FlatShardedAdamW``)."""
        from ..ops import kernels

        cur = torch.cuda.current_stream(grad.device)
        run = stream if stream is not None else cur
        if stream is not None:
            stream.wait_stream(cur)
        with torch.cuda.stream(run):
            kernels.adamw_flat_(update["p"], update["m"], update["v"], grad, lr=float(update["lr"]),
                                beta1=update["beta1"], beta2=update["beta2"], eps=update["eps"],
                                weight_decay=update["weight_decay"], step=int(update["step"]),
                                grad_scale=float(1.0 if scale is None else scale), p_lp=update.get("p_lp"))
        ev = None
        if stream is not None:
            ev = torch.cuda.Event()
            ev.record(run)
        return MatrixCollectiveHandle(event=ev, info={
            "kind": "reduce_scatter", "impl": "local_adamw", "backend": self.kind, "bytes": 0, "count": 0,
            "sync_mode": "stream_event" if stream is not None else "stream_order"})


class TorchDistTransport(LocalTransport):
    kind = "torch_dist"
    accumulates_fp32 = False  # library collectives reduce in the dtype of the buffer they are given

    def __init__(self, group, *, gather_impl: str | None = None, reduce_impl: str | None = None,
                 workspace_cache: CommWorkspaceCache | None = None) -> None:
        super().__init__()
        self.group = group
        self.gather_impl = gather_impl or os.environ.get(GATHER_IMPL_ENV, "auto")
        self.reduce_impl = reduce_impl or os.environ.get(REDUCE_IMPL_ENV, "auto")
        self.workspace_cache = workspace_cache or CommWorkspaceCache(max_cached_per_key=1)

    def _workspace(self, tables: SegmentTables, like: torch.Tensor):
        numel = tables.staging_numel(self.kind)      # the layout's descriptor knows what staging it needs
        if numel <= 0:
            return None
        return self.workspace_cache.lease(numel, like.dtype, like.device)

    def gather(self, shard, full, tables, *, stream=None, unit_key=None, impl: str | None = None):
        impl = impl or self.gather_impl
        lease = self._workspace(tables, full) if impl not in ("owner_broadcast", "broadcast", "all_reduce",
                                                              "all_reduce_gather") else None
        h = all_gatherv_rank_segments_1d_into_async(shard, full, tables, self.group, stream=stream, impl=impl,
                                                    workspace=lease.tensor if lease else None)
        h.info["backend"] = self.kind
        if lease is not None:
            h.info["workspace_numel"] = lease.tensor.numel()
            h.info["workspace_reused"] = lease.reused
            prev = h._post
            h._post = (lambda: (prev() if prev else None, lease.release()))
        return h

    def reduce(self, full_grad, out_shard, tables, *, scale=None, stream=None, unit_key=None, impl: str | None = None):
        impl = impl or self.reduce_impl
        lease = self._workspace(tables, full_grad) if impl not in ("owner_reduce", "reduce") else None
        h = reduce_scatterv_owner_rank_chunks_1d_async(full_grad, out_shard, tables, self.group, scale=scale,
                                                       stream=stream, impl=impl,
                                                       workspace=lease.tensor if lease else None)
        h.info["backend"] = self.kind
        if lease is not None:
            h.info["workspace_numel"] = lease.tensor.numel()
            h.info["workspace_reused"] = lease.reused
            prev = h._post
            h._post = (lambda: (prev() if prev else None, lease.release()))
        return h


def make_transport(group, world_size: int, device: torch.device, *, prefer: str | None = None):
    """Pick the transport for a shard group.

    ``prefer``: ``"peer"`` | ``"torch_dist"`` | ``None`` (auto: peer kernels on CUDA when every
    rank of the group sits on this node and the IPC mapping succeeds, else torch.distributed).
    """
    if world_size <= 1 or group is None:
        return LocalTransport()
    prefer = prefer or os.environ.get(TRANSPORT_ENV, "auto")
    if device.type == "cuda" and prefer in ("auto", "peer"):
        try:
            from .peer import PeerTransport

            t = PeerTransport.create(group, device)
            if t is not None:
                return t
            if prefer == "peer":
                raise RuntimeError("peer transport requested but unavailable")
        except Exception:
            if prefer == "peer":
                raise
    return TorchDistTransport(group)
