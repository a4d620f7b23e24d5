"""Metadata wrapper around a rank-local shard tensor (never a DTensor on the hot path).

Parity: ``matrix_fsdp/core/state.py:16-145`` and ``core/torch_dtensor.py:17-97``.
"""
from __future__ import annotations

from typing import Any

import torch

from .mesh import mesh_dim_names
from .placement import MatrixShard


class MatrixShardedState:
    """A local tensor plus the facts needed to place it in the logical tensor."""

    def __init__(self, local_tensor: torch.Tensor, *, logical_shape: tuple[int, ...], placement: MatrixShard | None,
                 rank: int, world_size: int, mesh=None, shard_mesh_dim: int | None = None,
                 name: str | None = None) -> None:
        self._local = local_tensor
        self.logical_shape = tuple(int(s) for s in logical_shape)
        self.placement = placement
        self.rank = int(rank)
        self.world_size = int(world_size)
        self.mesh = mesh
        self.shard_mesh_dim = shard_mesh_dim
        self.name = name

    @property
    def dtensor(self):
        return None

    @property
    def local_tensor(self) -> torch.Tensor:
        return self._local

    @property
    def uses_dtensor(self) -> bool:
        return False

    @property
    def fallback_tensor(self) -> torch.Tensor | None:
        return self._local

    def refresh(self, local_tensor: torch.Tensor) -> "MatrixShardedState":
        self._local = local_tensor
        return self

    def shares_storage_with(self, tensor: torch.Tensor) -> bool:
        return self._local.untyped_storage().data_ptr() == tensor.untyped_storage().data_ptr()

    def has_same_data_ptr(self, tensor: torch.Tensor) -> bool:
        return self._local.data_ptr() == tensor.data_ptr()

    def as_metadata(self) -> dict[str, Any]:
        return matrix_sharded_state_metadata(self)


def matrix_shard_metadata(placement: MatrixShard | None) -> dict[str, Any] | None:
    if placement is None:
        return None
    return {"type": "MatrixShard", "dims": tuple(placement.dims), "local_units": tuple(placement.local_units)}


def matrix_sharded_state_metadata(state: MatrixShardedState) -> dict[str, Any]:
    local = state.local_tensor
    return {
        "name": state.name,
        "logical_shape": tuple(state.logical_shape),
        "local_shape": tuple(local.shape),
        "local_numel": int(local.numel()),
        "dtype": str(local.dtype),
        "device": str(local.device),
        "rank": state.rank,
        "world_size": state.world_size,
        "uses_dtensor": False,
        "matrix_shard": matrix_shard_metadata(state.placement),
        "mesh_dim_names": mesh_dim_names(state.mesh) if state.mesh is not None else None,
        "shard_mesh_dim": state.shard_mesh_dim,
    }
