"""Device-mesh helpers: which mesh dimension shards and which replicates.

Parity: ``matrix_fsdp/core/mesh.py:11-178``.  One deliberate difference: with ``mesh=None``
inside an initialised process group the runtime uses the whole world as the shard group
(the reference silently degrades to world size 1, ``runtime/fsdp_unit.py:1754-1765``);
that resolution lives in :func:`resolve_groups`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Union

import torch.distributed as dist

MeshDim = Union[int, str]


@dataclass(frozen=True)
class DataParallelMeshDims:
    shard: MeshDim | tuple[MeshDim, ...] | None = None
    replicate: MeshDim | tuple[MeshDim, ...] | None = None


@dataclass(frozen=True)
class DeviceMeshMetadata:
    device_type: str | None
    ndim: int
    shape: tuple[int, ...]
    mesh_dim_names: tuple[str, ...] | None
    coordinate: tuple[int, ...] | None
    shard_mesh_dim: int
    shard_mesh_dim_name: str | None
    shard_mesh_size: int
    replicate_mesh_dim: int | None
    replicate_mesh_dim_name: str | None
    replicate_mesh_size: int

    def as_dict(self) -> dict[str, Any]:
        return {k: (list(v) if isinstance(v, tuple) else v) for k, v in self.__dict__.items()}


def mesh_shape(mesh) -> tuple[int, ...]:
    return tuple(int(s) for s in mesh.mesh.shape)


def mesh_dim_names(mesh) -> tuple[str, ...] | None:
    names = getattr(mesh, "mesh_dim_names", None)
    return tuple(names) if names else None


def mesh_dim_name(mesh, mesh_dim: int | None) -> str | None:
    names = mesh_dim_names(mesh)
    if names is None or mesh_dim is None:
        return None
    return names[mesh_dim]


def mesh_coordinate(mesh) -> tuple[int, ...] | None:
    coord = mesh.get_coordinate()
    return tuple(int(c) for c in coord) if coord is not None else None


def normalize_mesh_dim(mesh, mesh_dim: MeshDim, *, arg_name: str = "mesh_dim") -> int:
    ndim = len(mesh_shape(mesh))
    if isinstance(mesh_dim, str):
        names = mesh_dim_names(mesh)
        if names is None or mesh_dim not in names:
            raise ValueError(f"{arg_name}={mesh_dim!r} is not a mesh dim name of {names}.")
        return names.index(mesh_dim)
    if isinstance(mesh_dim, bool) or not isinstance(mesh_dim, int):
        raise TypeError(f"{arg_name} must be an int or a mesh dim name, got {type(mesh_dim).__name__}.")
    if not -ndim <= mesh_dim < ndim:
        raise ValueError(f"{arg_name}={mesh_dim} is out of range for a {ndim}-D mesh.")
    return mesh_dim % ndim


def infer_shard_mesh_dim(mesh, shard_mesh_dim: MeshDim | None = None) -> int:
    if mesh is None:
        return 0
    if shard_mesh_dim is not None:
        return normalize_mesh_dim(mesh, shard_mesh_dim, arg_name="dp_shard_mesh_dim")
    names = mesh_dim_names(mesh)
    if names and "dp_shard" in names:
        return names.index("dp_shard")
    ndim = len(mesh_shape(mesh))
    if ndim == 1:
        return 0
    if ndim == 2:
        return 1
    raise ValueError("Cannot infer the shard mesh dim of a >2-D mesh; name it 'dp_shard' or pass dp_mesh_dims.")


def infer_replicate_mesh_dim(mesh, shard_mesh_dim: int, replicate_mesh_dim: MeshDim | None = None) -> int | None:
    if mesh is None:
        return None
    if replicate_mesh_dim is not None:
        dim = normalize_mesh_dim(mesh, replicate_mesh_dim, arg_name="dp_replicate_mesh_dim")
        if dim == shard_mesh_dim:
            raise ValueError("dp_replicate mesh dim must differ from the dp_shard mesh dim.")
        return dim
    names = mesh_dim_names(mesh)
    if names and "dp_replicate" in names:
        dim = names.index("dp_replicate")
        return dim if dim != shard_mesh_dim else None
    ndim = len(mesh_shape(mesh))
    if ndim == 2 and not (names and "dp_shard" in names and len(names) == 2 and set(names) - {"dp_shard", "dp_replicate"}):
        return 1 - shard_mesh_dim
    if ndim == 2:
        return None
    return None


def mesh_metadata(mesh, shard_mesh_dim: MeshDim | None = None, replicate_mesh_dim: MeshDim | None = None) -> DeviceMeshMetadata | None:
    if mesh is None:
        return None
    sdim = infer_shard_mesh_dim(mesh, shard_mesh_dim)
    rdim = infer_replicate_mesh_dim(mesh, sdim, replicate_mesh_dim)
    shape = mesh_shape(mesh)
    return DeviceMeshMetadata(
        device_type=getattr(mesh, "device_type", None),
        ndim=len(shape),
        shape=shape,
        mesh_dim_names=mesh_dim_names(mesh),
        coordinate=mesh_coordinate(mesh),
        shard_mesh_dim=sdim,
        shard_mesh_dim_name=mesh_dim_name(mesh, sdim),
        shard_mesh_size=shape[sdim],
        replicate_mesh_dim=rdim,
        replicate_mesh_dim_name=mesh_dim_name(mesh, rdim),
        replicate_mesh_size=shape[rdim] if rdim is not None else 1,
    )


@dataclass
class ResolvedGroups:
    shard_group: Any
    shard_rank: int
    shard_world: int
    replicate_group: Any
    replicate_rank: int
    replicate_world: int
    metadata: DeviceMeshMetadata | None


def resolve_groups(mesh, shard_dim: MeshDim | None, replicate_dim: MeshDim | None, *, use_world_without_mesh: bool) -> ResolvedGroups:
    """Process groups and ranks of the shard and replicate dimensions."""
    if mesh is None:
        if use_world_without_mesh and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            return ResolvedGroups(dist.group.WORLD, dist.get_rank(), dist.get_world_size(), None, 0, 1, None)
        return ResolvedGroups(None, 0, 1, None, 0, 1, None)
    meta = mesh_metadata(mesh, shard_dim, replicate_dim)
    sgroup = mesh.get_group(meta.shard_mesh_dim)
    srank, sworld = dist.get_rank(sgroup), dist.get_world_size(sgroup)
    rgroup, rrank, rworld = None, 0, 1
    if meta.replicate_mesh_dim is not None and meta.replicate_mesh_size > 1:
        rgroup = mesh.get_group(meta.replicate_mesh_dim)
        rrank, rworld = dist.get_rank(rgroup), dist.get_world_size(rgroup)
    return ResolvedGroups(sgroup, srank, sworld, rgroup, rrank, rworld, meta)
