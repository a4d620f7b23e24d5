"""Flat-buffer storage of one FSDP unit.

Owns, for one unit:

``local_shard``       this rank's packed slice of the flat parameter space, in the model's
                      original ("master") dtype;
``local_shard_lp``    the same slice in the compute dtype when mixed precision is on (the
                      all-gather source; written by the fused optimizer kernels, refreshed by
                      a cast otherwise);
``full_buffer``       a persistent tensor object of the unit's full size whose *storage* is
                      materialised on unshard and shrunk to 0 bytes on reshard, so views saved
                      by autograd stay valid across reshard / re-gather;
``bucket``            full-size gradients in flat order (reduce-scatter source);
``local_grad_shard``  the reduced, averaged gradient slice the optimizer consumes.

``param.data`` is swapped between cached views of ``local_shard`` and cached views of
``full_buffer``; parameters stay ordinary ``nn.Parameter`` objects.

Parity: ``matrix_fsdp/runtime/flat_buffer.py:95-1502``.  One-time init differs: the reference
materialises ``torch.cat`` of all params plus a packed copy (2× the unit transiently,
``flat_buffer.py:240-243``); here every rank copies only the pieces it owns.
"""
from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass

import os

import torch

from ..core.layout import LayoutSegment, MatrixGroupLayout
from ..core.managed_param import ManagedParam, ManagedParamRegistry
from ..core.placement import MatrixShard, explain_matrix_shard_compatibility, shard_sizes_to_matrix_local_units
from .collectives import MatrixCollectiveHandle, SegmentTables
from .grad_bucket import BucketParam, MatrixGradBucket


@dataclass
class LocalParamPiece:
    """The part of one parameter that lives in this rank's shard."""

    fqn: str
    param_start: int      # offset of the piece inside the parameter (elements)
    numel: int
    local_start: int      # offset inside local_shard
    shape: tuple[int, ...]

    @property
    def local_end(self) -> int:
        return self.local_start + self.numel


def _piece_shape(mp: ManagedParam, start: int, numel: int) -> tuple[int, ...]:
    if numel == mp.numel:
        return tuple(mp.shape)
    if numel == 0:
        return (0,)
    if len(mp.shape) >= 2:
        inner = mp.numel // int(mp.shape[0])
        if start % inner == 0 and numel % inner == 0:
            return (numel // inner, *tuple(mp.shape)[1:])
    return (numel,)


def _poison_enabled() -> bool:
    return os.environ.get("MFSDP_DEBUG_POISON", "0") not in ("", "0")


class MatrixFlatBuffer:
    def __init__(self, registry: ManagedParamRegistry, layout: MatrixGroupLayout, *, rank: int, world_size: int,
                 transport, replicate_group=None, replicate_world_size: int = 1, param_dtype: torch.dtype | None = None,
                 reduce_dtype: torch.dtype | None = None, divide_grads_by_world: bool = True,
                 unit_key: str = "", exclusive_full_buffer: bool = False, gather_impl: str | None = None,
                 reduce_impl: str | None = None, shard_group=None) -> None:
        self.registry = registry
        self.layout = layout
        self.rank, self.world_size = rank, world_size
        self.transport = transport
        self.replicate_group = replicate_group
        self.replicate_world_size = replicate_world_size
        self.divide_grads_by_world = divide_grads_by_world
        self.unit_key = unit_key
        # explicit collective variants (``param_gather_strategy`` / ``backward_reduce_strategy``): they are
        # library collectives, run through a torch.distributed transport even when the unit's own
        # transport is the peer-kernel one
        self.gather_impl, self.reduce_impl = gather_impl, reduce_impl
        self.shard_group = shard_group
        self._library_transport = None
        params = registry.params
        if not params:
            raise ValueError("An FSDP unit needs at least one managed parameter.")
        dtypes = {p.dtype for p in params}
        if len(dtypes) != 1:
            raise ValueError(f"All managed parameters of a unit must share one dtype, got {sorted(map(str, dtypes))}.")
        devices = {p.device for p in params}
        if len(devices) != 1:
            raise ValueError(f"All managed parameters of a unit must share one device, got {sorted(map(str, devices))}.")
        self.device = params[0].device
        self.shard_dtype = params[0].dtype
        self.param_dtype = param_dtype or self.shard_dtype
        self.reduce_dtype = reduce_dtype or self.param_dtype
        self.mixed = self.param_dtype != self.shard_dtype
        self.total_numel = registry.total_numel
        self.tables = SegmentTables.build(self.total_numel, layout.rank_segments, rank)
        self.local_numel = self.tables.shard_sizes[rank]
        compat = explain_matrix_shard_compatibility(layout)
        self.matrix_shard: MatrixShard | None = (
            MatrixShard((0,), shard_sizes_to_matrix_local_units(layout.shard_sizes)) if compat.compatible else None)

        # ---- local shard: copy only the owned pieces out of the original parameters
        self.local_shard = transport.alloc_persistent(self.local_numel, self.shard_dtype, self.device, "shard",
                                                      symmetric_numel=self.tables.max_shard) \
            if not self.mixed else torch.empty(self.local_numel, dtype=self.shard_dtype, device=self.device)
        self.pieces: dict[str, LocalParamPiece] = {}
        with torch.no_grad():
            for ps in layout.param_segments_for_rank(rank):
                mp = registry.param(ps.fqn)
                if ps.fqn in self.pieces:
                    raise ValueError(
                        f"rank {rank} owns multiple local segments of parameter {ps.fqn!r}; "
                        "such layouts cannot be exposed as local views.")
                start = ps.global_start - mp.offset
                self.local_shard[ps.local_start:ps.local_end].copy_(
                    mp.param.detach().reshape(-1)[start:start + ps.numel])
                self.pieces[ps.fqn] = LocalParamPiece(ps.fqn, start, ps.numel, ps.local_start,
                                                      _piece_shape(mp, start, ps.numel))
        self.local_shard_lp: torch.Tensor | None = None
        self.lp_stale = True
        if self.mixed:
            self.local_shard_lp = transport.alloc_persistent(self.local_numel, self.param_dtype, self.device, "shard_lp",
                                                             symmetric_numel=self.tables.max_shard)

        # ---- aliasing: a single rank that holds the whole space in flat order needs no gather copy
        segs = self.tables.my_segments
        self.full_aliases_shard = (world_size == 1 and len(segs) == 1 and segs[0].global_start == 0
                                   and segs[0].numel == self.total_numel)

        # ---- full buffer object (storage materialised lazily) and cached views
        # ``full_persistent``: the transport handed out a persistent (symmetric, multicast-mapped) slot that
        # this unit shares with units it is never unsharded together with; nothing is resized then.
        self.full_persistent = False
        self.full_pool = None
        self._pooled: torch.Tensor | None = None
        if self.full_aliases_shard:
            self.full_buffer = self._gather_source_tensor()
        else:
            slot = None
            alloc_full = getattr(transport, "alloc_full_buffer", None)
            if alloc_full is not None and gather_impl is None:
                slot = alloc_full(unit_key, self.total_numel, self.param_dtype, self.tables,
                                  exclusive=exclusive_full_buffer)
            self.full_persistent = slot is not None
            self.full_buffer = slot if slot is not None else \
                torch.empty(self.total_numel, dtype=self.param_dtype, device=self.device)
        # views are created while the storage exists; they stay valid across resize_(0) / resize_(n)
        self._full_views = {mp.fqn: self.full_buffer[mp.offset:mp.end].view(mp.shape) for mp in params}
        if not self.full_aliases_shard:
            self._shrink_full()
        self._local_views: dict[str, torch.Tensor] = {}
        self._rebuild_local_views()
        self.full_materialized = self.full_aliases_shard
        self.params_use_full = False

        # ---- gradient side
        self.bucket = MatrixGradBucket(self.tables, [BucketParam(p.fqn, p.offset, p.numel) for p in params],
                                       self._bucket_dtype(), self.device)
        self.local_grad_shard: torch.Tensor | None = None
        self._local_grad_views: dict[str, torch.Tensor] = {}
        # True from the moment a reduction into ``local_grad_shard`` was issued until ``zero_grad``:
        # the buffer itself outlives the step, so optimizers must not read it without this flag
        # (a unit that got no backward in a step has no gradient, like ``param.grad is None``).
        self.local_grad_valid = False
        self.pending_gather: MatrixCollectiveHandle | None = None
        self.pending_reduce: MatrixCollectiveHandle | None = None
        self.grad_bucket_acquired = False
        self.accumulate_into_local_grad = False
        self.fused_optimizer_consumes_bucket = False
        # Set by an optimizer that wants the reduce-scatter to apply its update (peer transport only):
        # a callable returning the update arguments for this reduction, or None to reduce normally.
        self.fused_reduce_update = None
        self.fused_update_applied = False
        self.update_done_event = None     # CUDA event after which this step's fused update of the unit is complete
        self.deferred_gather = None          # plan of the all-gather rows left to the first consumer GEMM

    # ------------------------------------------------------------------ helpers
    def _bucket_dtype(self) -> torch.dtype:
        # Peer kernels accumulate in fp32 registers whatever the wire dtype, so they keep the
        # compute dtype on the wire; library collectives reduce in the bucket's dtype.
        if getattr(self.transport, "accumulates_fp32", False):
            return self.param_dtype
        return self.reduce_dtype

    def _gather_source_tensor(self) -> torch.Tensor:
        return self.local_shard_lp if self.mixed else self.local_shard

    def library_transport(self):
        """torch.distributed transport of this unit's shard group (the unit's own one when it already is)."""
        if getattr(self.transport, "kind", "") in ("torch_dist", "local"):
            return self.transport
        if self._library_transport is None:
            from .transport import TorchDistTransport

            self._library_transport = TorchDistTransport(self.shard_group)
        return self._library_transport

    def _rebuild_local_views(self) -> None:
        self._local_views = {}
        for mp in self.registry.params:
            piece = self.pieces.get(mp.fqn)
            if piece is None:
                self._local_views[mp.fqn] = self.local_shard.new_empty(0)
            else:
                self._local_views[mp.fqn] = self.local_shard[piece.local_start:piece.local_end].view(piece.shape)

    def local_param_views(self) -> dict[str, torch.Tensor]:
        return dict(self._local_views)

    def owned_fqns(self) -> tuple[str, ...]:
        return tuple(self.pieces)

    # ------------------------------------------------------------------ param.data swapping
    def use_local_shards(self) -> None:
        for mp in self.registry.params:
            mp.param.data = self._local_views[mp.fqn]
        self.params_use_full = False

    def use_full_param_buffer(self) -> None:
        for mp in self.registry.params:
            mp.param.data = self._full_views[mp.fqn]
        self.params_use_full = True

    # ------------------------------------------------------------------ full buffer storage
    def _full_nbytes(self) -> int:
        return self.total_numel * self.full_buffer.element_size()

    # ---- pooled mode: with saved-tensor hooks the autograd graph keeps no view of the unsharded buffer, so
    # the buffer may be a different allocation every time; it then comes from a shared pool and goes back
    # to it at reshard, reusable once the kernels that read it have finished (CUDA event).
    def use_full_param_pool(self, pool) -> None:
        if self.full_aliases_shard or self.full_persistent or self.full_materialized:
            return
        if self.full_pool is None:
            self.full_buffer.untyped_storage().resize_(0)
        self.full_pool = pool

    def _shrink_full(self) -> None:
        if self.full_aliases_shard:
            return
        if self.full_persistent:
            self.transport.release_full_buffer(self.unit_key)   # peers may refill the slot from here on
            return
        if self.full_pool is not None:
            if self._pooled is not None:
                event = None
                if self.device.type == "cuda":
                    event = torch.cuda.Event()
                    event.record(torch.cuda.current_stream(self.device))
                self.full_pool.release(self._pooled, event)
                self._pooled = None
            return
        self.full_buffer.untyped_storage().resize_(0)

    def _materialize_full(self) -> None:
        if self.full_persistent:
            return
        if self.full_pool is not None:
            if self._pooled is None:
                self._pooled = self.full_pool.acquire(self.total_numel, self.param_dtype, self.device)
                self.full_buffer = self._pooled
                self._full_views = {mp.fqn: self.full_buffer[mp.offset:mp.end].view(mp.shape)
                                    for mp in self.registry.params}
                if _poison_enabled() and self.full_buffer.is_floating_point():
                    self.full_buffer.fill_(float("nan"))
            return
        st = self.full_buffer.untyped_storage()
        if st.size() != self._full_nbytes():
            st.resize_(self._full_nbytes())
            if _poison_enabled() and self.full_buffer.is_floating_point():
                # debug aid: a read of gathered parameters before they arrived shows up as NaN
                # (ordered before the gather by the gather stream's wait on the current stream)
                self.full_buffer.fill_(float("nan"))

    def full_storage_nbytes(self) -> int:
        if self.full_aliases_shard:
            return 0
        if self.full_persistent:
            return self._full_nbytes() if self.full_materialized else 0
        if self.full_pool is not None:
            return self._full_nbytes() if self._pooled is not None else 0
        return self.full_buffer.untyped_storage().size()

    def full_slot_available(self) -> bool:
        """False while another unit's parameters occupy the slot this unit's full buffer lives in."""
        probe = getattr(self.transport, "full_slot_available", None)
        return True if (probe is None or not self.full_persistent) else bool(probe(self.unit_key))

    # ------------------------------------------------------------------ all-gather
    def refresh_low_precision_shard(self) -> None:
        """Cast master → compute dtype when the optimizer did not already emit it."""
        if self.mixed and self.lp_stale:
            if self.device.type == "cuda" and self.param_dtype == torch.bfloat16 \
                    and self.shard_dtype == torch.float32 and _native_ok():
                from ..ops import kernels

                kernels.cast_f32_bf16(self.local_shard, self.local_shard_lp)
            else:
                self.local_shard_lp.copy_(self.local_shard)
            self.lp_stale = False

    def start_all_gather_full_params(self, *, stream=None, defer: tuple | None = None,
                                     ordered_by_caller: bool = False) -> MatrixCollectiveHandle:
        """``defer`` = (lo, hi, row_len): leave that range of the full buffer to the GEMM that reads it
        first (transports that can; the plan is then in ``self.deferred_gather``).  ``ordered_by_caller``: the
        caller made ``stream`` wait for the event after which this unit's shard is final, so the gather need
        not wait for the rest of the current stream (only with a persistent full-parameter slot: a buffer from
        the caching allocator is tied to the current stream)."""
        if self.pending_gather is not None:
            return self.pending_gather
        self.refresh_low_precision_shard()
        if self.full_aliases_shard:
            h = MatrixCollectiveHandle(info={"kind": "all_gather", "impl": "alias", "backend": "local", "bytes": 0,
                                             "count": 0, "sync_mode": "local", "materialization": "alias"})
        else:
            self._materialize_full()
            if defer is not None and getattr(self.transport, "supports_deferred_gather", False) \
                    and self.full_buffer.dtype == torch.bfloat16:
                h = self.transport.gather(self._gather_source_tensor(), self.full_buffer, self.tables, stream=stream,
                                          unit_key=self.unit_key, defer=defer)
                self.deferred_gather = getattr(h, "deferred", None)
            elif self.gather_impl is not None and self.world_size > 1:
                if self.gather_impl == "equal_all_gather" and not self.tables.equal_contiguous:
                    raise RuntimeError("param_gather_strategy='equal_all_gather' requires equal rank-ordered shards.")
                if self.gather_impl == "owner_broadcast" and not self._whole_param_owners():
                    raise RuntimeError("param_gather_strategy='owner_broadcast' requires whole-parameter owner shards.")
                h = self.library_transport().gather(self._gather_source_tensor(), self.full_buffer, self.tables,
                                                    stream=stream, unit_key=self.unit_key, impl=self.gather_impl)
            elif ordered_by_caller and self.full_persistent and stream is not None:
                h = self.transport.gather(self._gather_source_tensor(), self.full_buffer, self.tables, stream=stream,
                                          unit_key=self.unit_key, wait_current=False)
            else:
                h = self.transport.gather(self._gather_source_tensor(), self.full_buffer, self.tables, stream=stream,
                                          unit_key=self.unit_key)
            h.info.setdefault("materialization", "persistent_slot" if self.full_persistent else "storage_resize")
        self.full_materialized = True
        self.pending_gather = h
        return h

    def _whole_param_owners(self) -> bool:
        return all(len(self.layout.owner_ranks(mp.fqn)) == 1 for mp in self.registry.params)

    def wait_all_gather(self, *, keep_deferred: bool = False) -> MatrixCollectiveHandle | None:
        h, self.pending_gather = self.pending_gather, None
        if h is not None:
            h.wait()
        if not keep_deferred:
            self.complete_deferred_gather()
        return h

    def complete_deferred_gather(self) -> None:
        """Nobody will fuse the deferred rows into a GEMM: copy them now (current stream)."""
        plan, self.deferred_gather = self.deferred_gather, None
        if plan is not None:
            plan.complete()

    def take_deferred_gather(self, weight: torch.Tensor):
        """Hand the deferred plan to the GEMM whose B operand is exactly the deferred weight."""
        plan = self.deferred_gather
        if plan is None:
            return None
        if weight.data_ptr() != plan.b_ptr or weight.numel() != plan.hi - plan.lo or not weight.is_contiguous():
            self.complete_deferred_gather()
            return None
        self.deferred_gather = None
        return plan

    def clear_full_params(self, *, keep_storage: bool = False) -> None:
        """Drop the unsharded storage (params must already point at local views)."""
        if self.pending_gather is not None:
            self.wait_all_gather()
        if self.deferred_gather is not None:
            self.deferred_gather = None
            raise RuntimeError("rows of the all-gather were left to a fused GEMM that never ran")
        if not keep_storage:
            self._shrink_full()
        self.full_materialized = self.full_aliases_shard

    # ------------------------------------------------------------------ gradients
    def prepare_grad_bucket(self) -> torch.Tensor:
        """Make sure the bucket has storage (direct-write ops need it before backward compute)."""
        if self.bucket.buffer is None:
            buf = self.transport.acquire_grad_buffer(self.unit_key, self.total_numel, self.bucket.dtype, self.device)
            self.bucket.attach(buf)
            self.grad_bucket_acquired = True
        return self.bucket.buffer

    def collect_param_grads(self, *, accumulate: bool, written_direct: set[str] | None = None) -> str:
        """Move autograd-produced ``param.grad`` tensors into the bucket and clear them."""
        self.prepare_grad_bucket()
        written_direct = written_direct or set()
        grads = []
        any_missing = False
        for mp in self.registry.params:
            g = mp.param.grad
            if mp.fqn in written_direct:
                grads.append("direct")
            elif g is None:
                grads.append(None)
                any_missing = True
            else:
                grads.append(g.detach())
            mp.param.grad = None
        if written_direct:
            how = "direct"
            for mp, g in zip(self.registry.params, grads):
                if isinstance(g, str):
                    continue
                view = self.bucket.buffer[mp.offset:mp.end]
                if g is None:
                    if not accumulate:
                        view.zero_()
                elif accumulate:
                    view.add_(g.reshape(-1).to(view.dtype))
                else:
                    view.copy_(g.reshape(-1))
            return how
        if accumulate:
            return self.bucket.copy_in(grads, accumulate=True)
        if any_missing:
            return self.bucket.copy_in(grads)
        return self.bucket.copy_in(grads)

    def _ensure_local_grad_shard(self) -> torch.Tensor:
        if self.local_grad_shard is None:
            self.local_grad_shard = torch.empty(self.local_numel, dtype=self.shard_dtype, device=self.device)
            self._local_grad_views = {}
            for fqn, piece in self.pieces.items():
                self._local_grad_views[fqn] = self.local_grad_shard[piece.local_start:piece.local_end].view(piece.shape)
        return self.local_grad_shard

    def stash_local_grads_for_accumulation(self) -> None:
        """A new forward starts while reduced gradients are still attached: detach them from the
        parameters (shapes differ once unsharded) and fold the next reduction into them."""
        attached = False
        for mp in self.registry.params:
            if mp.param.grad is not None:
                attached = True
                mp.param.grad = None
        if attached and self.local_grad_shard is not None:
            if self.bucket.buffer is not None and \
                    self.local_grad_shard.untyped_storage().data_ptr() == self.bucket.buffer.untyped_storage().data_ptr():
                self.local_grad_shard = self.local_grad_shard.clone()
                self._local_grad_views = {
                    fqn: self.local_grad_shard[p.local_start:p.local_end].view(p.shape)
                    for fqn, p in self.pieces.items()}
                self.bucket.release()
            self.accumulate_into_local_grad = True

    def grad_scale(self) -> float:
        if not self.divide_grads_by_world:
            return 1.0
        return 1.0 / float(self.world_size * self.replicate_world_size)

    def start_reduce_grad_bucket_to_local_shard(self, *, stream=None, strategy: str = "bucket_reduce_scatter",
                                                ) -> MatrixCollectiveHandle:
        """Reduce the bucket over the shard group (then the replicate group) into ``local_grad_shard``.

        ``strategy``: ``bucket_reduce_scatter`` (the transport's own reduction), ``flat`` (one library
        reduce-scatter over the flat gradient) or ``per_param`` (one library reduce-scatter per parameter)."""
        out = self._ensure_local_grad_shard()
        src = self.bucket.ensure()
        scale = self.grad_scale()
        self.update_done_event = None
        if self.world_size == 1 and self.replicate_world_size == 1 and self.full_aliases_shard \
                and self.fused_reduce_update is not None and src.is_cuda and scale == 1.0 \
                and strategy == "bucket_reduce_scatter" and not self.accumulate_into_local_grad \
                and type(self.transport).__name__ == "LocalTransport":
            # single rank with the update fused into the "reduce": the bucket is the gradient, AdamW runs now
            update = self.fused_reduce_update()
            if update is not None:
                h = self.transport.local_update(src, update, stream=stream)
                self.fused_update_applied = True
                self.update_done_event = getattr(h, "_event", None)
                self.pending_reduce = h
                return h
        if self.world_size == 1 and self.replicate_world_size == 1 and self.full_aliases_shard \
                and (src.dtype == out.dtype or self.fused_optimizer_consumes_bucket) and scale == 1.0 \
                and not self.accumulate_into_local_grad:
            # single rank, same dtype: the bucket *is* the local gradient
            self.local_grad_shard = src
            self._local_grad_views = {
                fqn: src[p.local_start:p.local_end].view(p.shape) for fqn, p in self.pieces.items()}
            h = MatrixCollectiveHandle(info={"kind": "reduce_scatter", "impl": "alias", "backend": "local",
                                             "bytes": 0, "count": 0, "sync_mode": "local"})
            self.pending_reduce = h
            self.local_grad_valid = True
            return h
        if self.fused_reduce_update is not None and self.replicate_world_size == 1 \
                and strategy == "bucket_reduce_scatter" and self.reduce_impl is None \
                and not self.accumulate_into_local_grad and hasattr(self.transport, "reduce_update"):
            update = self.fused_reduce_update()
            if update is not None:
                h = self.transport.reduce_update(src, self.tables, update, scale=scale, stream=stream,
                                                 unit_key=self.unit_key)
                self.fused_update_applied = True
                self.update_done_event = getattr(h, "_event", None)
                self.pending_reduce = h
                return h
        library = (strategy in ("flat", "per_param") or self.reduce_impl is not None) and self.world_size > 1
        reducer = self.library_transport() if library else self.transport
        needs_cast = out.dtype != src.dtype and not getattr(reducer, "accumulates_fp32", False)
        accumulate = self.accumulate_into_local_grad
        self.accumulate_into_local_grad = False
        if accumulate and out.dtype != self.shard_dtype:
            out = out.to(self.shard_dtype)
        if needs_cast or accumulate:
            target = torch.empty(self.local_numel, dtype=src.dtype if needs_cast else out.dtype, device=self.device)
        else:
            target = out
        shard_scale = scale if self.replicate_world_size == 1 else 1.0 / float(self.world_size) \
            if self.divide_grads_by_world else 1.0
        if library and strategy == "per_param":
            from .collectives import reduce_scatter_per_param_async

            h = reduce_scatter_per_param_async(src, target, self.tables,
                                               [(mp.offset, mp.end) for mp in self.registry.params],
                                               self.shard_group, scale=shard_scale, stream=stream)
            h.info["backend"] = reducer.kind
        elif library:
            h = reducer.reduce(src, target, self.tables, scale=shard_scale, stream=stream, unit_key=self.unit_key,
                               impl=self.reduce_impl or "padded")
        else:
            h = self.transport.reduce(src, target, self.tables, scale=shard_scale, stream=stream,
                                      unit_key=self.unit_key)
        replicate_group, rworld = self.replicate_group, self.replicate_world_size
        divide = self.divide_grads_by_world
        prev_post = h._post

        def post():
            if prev_post is not None:
                prev_post()
            if rworld > 1:
                self.transport.all_reduce(target, replicate_group, scale=(1.0 / rworld) if divide else None)
            if accumulate:
                out.add_(target.to(out.dtype))
            elif needs_cast:
                out.copy_(target)

        h._post = post
        self.pending_reduce = h
        self.local_grad_valid = True
        return h

    def wait_reduce(self) -> MatrixCollectiveHandle | None:
        h, self.pending_reduce = self.pending_reduce, None
        if h is not None:
            h.wait()
        return h

    def use_local_grad_shard(self) -> None:
        """``param.grad`` := view of the reduced local gradient (owned pieces only)."""
        assert not self.params_use_full
        for mp in self.registry.params:
            v = self._local_grad_views.get(mp.fqn)
            if v is not None and v.numel() > 0 and v.dtype == mp.param.dtype:
                mp.param.grad = v
            else:
                mp.param.grad = None

    def release_grad_bucket(self) -> None:
        if self.bucket.buffer is not None:
            keep = self.local_grad_shard is not None and \
                self.local_grad_shard.untyped_storage().data_ptr() == self.bucket.buffer.untyped_storage().data_ptr()
            if not keep and self.grad_bucket_acquired:
                self.transport.release_grad_buffer(self.unit_key, self.bucket.buffer)
            self.bucket.release()
            self.grad_bucket_acquired = False

    def clear_local_grad_shard(self) -> None:
        self.local_grad_valid = False
        for mp in self.registry.params:
            mp.param.grad = None
        if self.local_grad_shard is not None and self.world_size == 1 and self.full_aliases_shard:
            self.local_grad_shard = None
            self._local_grad_views = {}

    # ------------------------------------------------------------------ optimizer notifications
    def mark_master_updated(self, lp_written: bool = False) -> None:
        """Call after the optimizer changed ``local_shard`` (``lp_written``: the kernel emitted the lp copy)."""
        if self.mixed:
            self.lp_stale = not lp_written

    # ------------------------------------------------------------------ accounting
    def memory_snapshot(self) -> dict[str, int]:
        es = self.full_buffer.element_size()
        bucket = self.bucket.buffer
        lg = self.local_grad_shard
        return {
            "full_param_buffer_numel": self.total_numel if self.full_materialized else 0,
            "full_param_buffer_bytes": self.total_numel * es if self.full_materialized and not self.full_aliases_shard else 0,
            "grad_bucket_numel": bucket.numel() if bucket is not None else 0,
            "grad_bucket_bytes": bucket.numel() * bucket.element_size() if bucket is not None else 0,
            "local_grad_shard_numel": lg.numel() if lg is not None else 0,
            "local_grad_shard_bytes": lg.numel() * lg.element_size() if lg is not None else 0,
            "local_shard_bytes": self.local_shard.numel() * self.local_shard.element_size(),
        }


def _native_ok() -> bool:
    from ..ops import lib

    return lib.available() and not lib.disabled_by_env()
