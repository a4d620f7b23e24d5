"""Runtime identifiers and the per-unit event log record.

Parity: ``matrix_fsdp/runtime/runtime.py:1-53`` and ``runtime/runtime_event.py:14-59``.
Events carry the host enqueue time and, when the unit records CUDA events, the device
duration of the span (``device_ms``), which the reference does not measure.
"""
from __future__ import annotations

import itertools
import threading
from dataclasses import asdict, dataclass, field
from typing import Any

RuntimeParamGroupId = int
PlannerGroupId = int
CommBufferId = int
RuntimeUnitId = int

_counter = itertools.count()
_seq = itertools.count()
_lock = threading.Lock()


def next_runtime_param_group_id() -> int:
    with _lock:
        return next(_counter)


def next_event_sequence() -> int:
    with _lock:
        return next(_seq)


def reset_runtime_ids() -> None:
    """Restart numbering (tests build many independent models in one process)."""
    global _counter
    with _lock:
        _counter = itertools.count()


@dataclass(frozen=True)
class RuntimeUnitMetadata:
    runtime_param_group_id: int
    planner_group_id: int
    comm_buffer_id: int

    @property
    def name(self) -> str:
        return f"param_group_{self.runtime_param_group_id}"

    def as_dict(self) -> dict[str, int]:
        return asdict(self)


@dataclass(frozen=True)
class RuntimeEvent:
    name: str
    unit: str
    sequence: int
    lifecycle_state: str
    duration_ms: float = 0.0
    device_ms: float | None = None
    reason: str | None = None
    collective_kind: str | None = None
    collective_backend: str | None = None
    collective_impl: str | None = None
    collective_bytes: int = 0
    collective_count: int = 0
    collective_sync_mode: str | None = None
    collective_phase_ms: tuple[tuple[str, float], ...] = ()
    active_full_param_buffers: int = 0
    active_full_param_numel: int = 0
    active_full_param_bytes: int = 0
    full_param_buffer_numel: int = 0
    full_param_buffer_bytes: int = 0
    grad_bucket_numel: int = 0
    grad_bucket_bytes: int = 0
    reduce_scatter_input_numel: int = 0
    reduce_scatter_input_bytes: int = 0
    local_grad_shard_numel: int = 0
    local_grad_shard_bytes: int = 0
    pending_reduce_scatter_count: int = 0
    grad_bucket_aliases_full_grad: bool = False
    local_grad_aliases_bucket: bool = False
    workspace_kind: str | None = None
    workspace_numel: int = 0
    workspace_reused: bool = False
    materialization: str | None = None
    prefetched: bool = False
    recompute: bool = False
    extra: dict[str, Any] = field(default_factory=dict)

    def as_dict(self) -> dict[str, Any]:
        return asdict(self)


class nvtx_range:
    """NVTX range around a runtime phase (``MFSDP_NVTX=1`` on a CUDA build; otherwise free).

    The reference has no NVTX / profiler integration (its event log carries host durations only)."""

    _enabled: bool | None = None

    def __init__(self, name: str) -> None:
        self.name = name

    @classmethod
    def enabled(cls) -> bool:
        if cls._enabled is None:
            import os

            import torch

            cls._enabled = os.environ.get("MFSDP_NVTX", "0") not in ("", "0") and torch.cuda.is_available()
        return cls._enabled

    def __enter__(self):
        if self.enabled():
            import torch

            torch.cuda.nvtx.range_push(self.name)
        return self

    def __exit__(self, *exc):
        if self.enabled():
            import torch

            torch.cuda.nvtx.range_pop()
        return False
