"""Optional DTensor views for interop (checkpoint tooling); never used on the step path.

Parity: ``matrix_fsdp/core/torch_dtensor.py:17-97``.
"""
from __future__ import annotations

import torch

from .placement import MatrixShard


def make_matrix_placements(mesh, shard_mesh_dim: int, placement: MatrixShard) -> tuple:
    """``Replicate`` on every mesh dim except ``shard_mesh_dim``, which gets ``placement``."""
    from torch.distributed.tensor.placement_types import Replicate

    ndim = len(tuple(mesh.mesh.shape))
    return tuple(placement if d == shard_mesh_dim else Replicate() for d in range(ndim))


def _contiguous_stride(shape) -> tuple[int, ...]:
    stride, acc = [], 1
    for s in reversed(tuple(shape)):
        stride.append(acc)
        acc *= int(s)
    return tuple(reversed(stride))


def make_matrix_dtensor_spec(mesh, shard_mesh_dim: int, placement: MatrixShard, logical_shape, dtype: torch.dtype):
    from torch.distributed.tensor._dtensor_spec import DTensorSpec, TensorMeta

    meta = TensorMeta(torch.Size(logical_shape), _contiguous_stride(logical_shape), dtype)
    return DTensorSpec(mesh, make_matrix_placements(mesh, shard_mesh_dim, placement), tensor_meta=meta)


def make_matrix_dtensor(local_tensor: torch.Tensor, mesh, shard_mesh_dim: int, placement: MatrixShard, logical_shape):
    """Wrap ``local_tensor`` as a DTensor carrying a MatrixShard placement (metadata only)."""
    from torch.distributed.tensor import DTensor

    spec = make_matrix_dtensor_spec(mesh, shard_mesh_dim, placement, logical_shape, local_tensor.dtype)
    return DTensor(local_tensor, spec, requires_grad=local_tensor.requires_grad)
