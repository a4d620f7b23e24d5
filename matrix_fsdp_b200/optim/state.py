"""Checkpoint-facing view of optimizer state: which tensors belong to which sharded parameter.

Every param-shaped state tensor (``exp_avg``, ``momentum_buffer`` …) of an owned parameter piece
is described by the same ``MatrixShard`` metadata as the parameter shard itself; 0-d entries
(``step``) are carried inline.

Parity: ``matrix_fsdp/optim/state.py:1-188`` and ``optim/adamw_state.py:1-218`` (the flat moment
buffers live in :mod:`matrix_fsdp_b200.optim.flat`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch

from ..core.state import MatrixShardedState


@dataclass(frozen=True)
class LocalOptimizerParamInfo:
    component: str
    unit: str
    fqn: str
    param_numel: int
    local_numel: int
    local_start: int
    param_start: int


@dataclass(frozen=True)
class LocalOptimizerStateTensor:
    info: LocalOptimizerParamInfo
    state_name: str
    tensor: torch.Tensor
    sharded: MatrixShardedState | None


@dataclass(frozen=True)
class OptimizerStateSummary:
    num_params: int
    num_state_tensors: int
    local_state_numel: int
    local_state_bytes: int
    by_component: dict[str, int]


class MatrixFSDPOptimizerStateManager:
    def __init__(self, units, optimizers: dict[str, Any]) -> None:
        self.units = list(units)
        self.optimizers = dict(optimizers)

    def _param_index(self) -> dict[int, tuple]:
        out = {}
        for u in self.units:
            for mp in u.registry:
                out[id(mp.param)] = (u, mp)
        return out

    def iter_param_infos(self):
        idx = self._param_index()
        for comp, opt in self.optimizers.items():
            for g in opt.param_groups:
                for p in g["params"]:
                    hit = idx.get(id(p))
                    if hit is None:
                        continue
                    u, mp = hit
                    piece = u.flat_buffer.pieces.get(mp.fqn)
                    if piece is None:
                        continue
                    yield p, LocalOptimizerParamInfo(comp, u.name, mp.fqn, mp.numel, piece.numel, piece.local_start,
                                                     piece.param_start)

    def iter_state_tensors(self):
        by_name = {u.name: u for u in self.units}
        for p, info in self.iter_param_infos():
            state = self.optimizers[info.component].state.get(p, {})
            unit = by_name[info.unit]
            for name, value in state.items():
                if not isinstance(value, torch.Tensor):
                    continue
                sharded = None
                if value.dim() > 0 and value.numel() == info.local_numel:
                    sharded = MatrixShardedState(value, logical_shape=tuple(unit.registry.param(info.fqn).shape),
                                                 placement=unit.flat_buffer.matrix_shard, rank=unit.rank,
                                                 world_size=unit.world_size, name=f"{info.fqn}.{name}")
                yield LocalOptimizerStateTensor(info, name, value, sharded)

    def summary(self) -> OptimizerStateSummary:
        params = {(i.component, i.unit, i.fqn) for _, i in self.iter_param_infos()}
        tensors = list(self.iter_state_tensors())
        by: dict[str, int] = {}
        for t in tensors:
            by[t.info.component] = by.get(t.info.component, 0) + t.tensor.numel()
        return OptimizerStateSummary(len(params), len(tensors), sum(t.tensor.numel() for t in tensors),
                                     sum(t.tensor.numel() * t.tensor.element_size() for t in tensors), by)
