"""Lease-based cache of communication scratch buffers keyed by (device, dtype, numel).

Parity: ``matrix_fsdp/runtime/workspace_cache.py:1-118``.
"""
from __future__ import annotations

from collections import defaultdict
from dataclasses import dataclass

import torch


@dataclass
class CommWorkspaceLease:
    cache: "CommWorkspaceCache"
    key: tuple
    tensor: torch.Tensor
    reused: bool
    released: bool = False

    def release(self) -> None:
        if not self.released:
            self.released = True
            self.cache._give_back(self)

    def __enter__(self) -> torch.Tensor:
        return self.tensor

    def __exit__(self, *exc) -> None:
        self.release()


class CommWorkspaceCache:
    def __init__(self, max_cached_per_key: int = 1) -> None:
        self.max_cached_per_key = int(max_cached_per_key)
        self._free: dict[tuple, list[torch.Tensor]] = defaultdict(list)
        self.allocations = 0
        self.reuses = 0
        self.leases = 0

    def lease(self, numel: int, dtype: torch.dtype, device: torch.device) -> CommWorkspaceLease:
        key = (str(device), dtype, int(numel))
        self.leases += 1
        if self._free[key]:
            self.reuses += 1
            return CommWorkspaceLease(self, key, self._free[key].pop(), True)
        self.allocations += 1
        return CommWorkspaceLease(self, key, torch.empty(numel, dtype=dtype, device=device), False)

    def _give_back(self, lease: CommWorkspaceLease) -> None:
        if len(self._free[lease.key]) < self.max_cached_per_key:
            self._free[lease.key].append(lease.tensor)

    def clear(self) -> None:
        self._free.clear()

    def stats(self) -> dict[str, int]:
        return {"allocations": self.allocations, "reuses": self.reuses, "leases": self.leases,
                "cached": sum(len(v) for v in self._free.values())}
