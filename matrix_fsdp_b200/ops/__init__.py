"""The sm_100a kernel library and its Python bindings.

``native_kernel_status()`` answers "will the CUDA kernels run here?" without touching a device: whether
``libmfsdp_kernels.so`` was built, whether it loads, whether it exports every entry point the Python side binds,
and whether an environment switch turned it off.  Counterpart of ``matrix_fsdp/kernels/native.py:41-59``
(``NativeKernelStatus``, ``native_kernel_status``, ``native_kernel_available``); the segment-fusion helpers of
``matrix_fsdp/kernels/segment_fusion.py`` live in ``core/layout.py`` and are re-exported here under their names.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class NativeKernelStatus:
    available: bool
    library: str
    reason: str | None = None
    entry_points: int = 0
    missing_entry_points: tuple[str, ...] = ()
    disabled_by_env: bool = False


def native_kernel_status() -> NativeKernelStatus:
    from . import lib

    path = str(lib.lib_path())
    if lib.disabled_by_env():
        return NativeKernelStatus(False, path, reason="MFSDP_DISABLE_NATIVE_KERNELS is set", disabled_by_env=True)
    handle = lib.load()
    if handle is None:
        return NativeKernelStatus(False, path, reason=f"{type(lib._LIB_ERR).__name__}: {lib._LIB_ERR}")
    # the modules that declare further launchers (attention, MoE, peer collectives) register them on import
    from . import attention, moe_kernels  # noqa: F401
    from ..parallel import peer  # noqa: F401

    missing = tuple(name for name in lib._SIGNATURES if not hasattr(handle, name))
    reason = f"library lacks {len(missing)} entry point(s): rebuild with `python -m matrix_fsdp_b200.ops.build`" \
        if missing else None
    return NativeKernelStatus(not missing, path, reason=reason, entry_points=len(lib._SIGNATURES),
                              missing_entry_points=missing)


def native_kernel_available() -> bool:
    return native_kernel_status().available


def coalesce_contiguous_segments(segments):
    """Merge neighbours that are contiguous in the flat space and in the local shard."""
    from ..core.layout import coalesce_segments

    return coalesce_segments(segments)


def coalesce_rank_segments(rank_segments):
    """:func:`coalesce_contiguous_segments` for every rank of a layout."""
    return tuple(coalesce_contiguous_segments(segs) for segs in rank_segments)


__all__ = ["NativeKernelStatus", "coalesce_contiguous_segments", "coalesce_rank_segments", "native_kernel_available",
           "native_kernel_status"]
