"""Pool of full-parameter (unsharded) buffers keyed by (device, dtype, numel).

Used by units that run with ``use_saved_tensor_hooks=True``: their autograd graph holds no view
of the unsharded buffer, so the buffer may be a different allocation at every unshard and is
acquired here at unshard and released here at reshard (``MatrixFlatBuffer._materialize_full`` /
``_shrink_full``).  Units without the hooks keep one tensor whose storage is resized instead,
because views saved by autograd have to stay valid.

A released buffer may still be read by kernels in flight, so release takes the CUDA event
that marks the last use; the buffer returns to the free list only once that event has
completed (checked lazily at the next acquire).  With the default
``max_cached_per_key=2`` the steady state is two live slots per size class (the unit being
computed and the one being prefetched) and no allocator traffic per step; the reference's
default of 0 frees and reallocates every time (``matrix_fsdp/runtime/buffer_pool.py:1-202``).
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass

import torch


@dataclass
class BufferPoolStats:
    acquires: int = 0
    allocations: int = 0
    reuses: int = 0
    releases: int = 0
    deferred_releases: int = 0
    dropped: int = 0
    high_water_bytes: int = 0
    live_bytes: int = 0

    def as_dict(self) -> dict[str, int]:
        return dict(self.__dict__)


class FullParamBufferPool:
    def __init__(self, max_cached_per_key: int = 2) -> None:
        self.max_cached_per_key = int(max_cached_per_key)
        self._free: dict[tuple, list[torch.Tensor]] = defaultdict(list)
        self._pending: list[tuple[tuple, torch.Tensor, object]] = []
        self.stats = BufferPoolStats()

    @staticmethod
    def _key(device: torch.device, dtype: torch.dtype, numel: int) -> tuple:
        return (str(device), dtype, int(numel))

    def _drain_pending(self) -> None:
        still = []
        for key, buf, event in self._pending:
            if event is None or event.query():
                self._park(key, buf)
            else:
                still.append((key, buf, event))
        self._pending = still

    def _park(self, key: tuple, buf: torch.Tensor) -> None:
        if len(self._free[key]) < self.max_cached_per_key:
            self._free[key].append(buf)
        else:
            self.stats.dropped += 1
            self.stats.live_bytes -= buf.numel() * buf.element_size()

    def acquire(self, numel: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
        self.stats.acquires += 1
        self._drain_pending()
        key = self._key(device, dtype, numel)
        if self._free[key]:
            self.stats.reuses += 1
            return self._free[key].pop()
        self.stats.allocations += 1
        buf = torch.empty(numel, dtype=dtype, device=device)
        self.stats.live_bytes += numel * buf.element_size()
        self.stats.high_water_bytes = max(self.stats.high_water_bytes, self.stats.live_bytes)
        return buf

    def release(self, buf: torch.Tensor, event=None) -> None:
        """Give a buffer back; ``event`` (a recorded CUDA event) defers reuse until it completes."""
        self.stats.releases += 1
        key = self._key(buf.device, buf.dtype, buf.numel())
        if event is not None and not event.query():
            self.stats.deferred_releases += 1
            self._pending.append((key, buf, event))
            return
        self._park(key, buf)

    def clear(self) -> None:
        self._free.clear()
        self._pending.clear()
        self.stats.live_bytes = 0

    def cached_buffers(self) -> int:
        return sum(len(v) for v in self._free.values()) + len(self._pending)


_GLOBAL_POOL: FullParamBufferPool | None = None


def global_full_param_buffer_pool() -> FullParamBufferPool:
    global _GLOBAL_POOL
    if _GLOBAL_POOL is None:
        _GLOBAL_POOL = FullParamBufferPool()
    return _GLOBAL_POOL


def clear_global_full_param_buffer_pool() -> None:
    if _GLOBAL_POOL is not None:
        _GLOBAL_POOL.clear()
