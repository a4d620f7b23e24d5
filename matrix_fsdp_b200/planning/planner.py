"""Concrete group planners: how one unit's flat parameter space is cut across ranks.

Two families cover everything:

* *boundary planners* build an ordered list of indivisible blocks (whole parameters, fixed
  1-D blocks, matrix row blocks) and cut it into rank-contiguous intervals with a
  nearest-to-target greedy (:func:`split_blocks_across_ranks`);
* *owner planners* treat every 2-D matrix (or every expert's parameter set) as a role and
  hand roles, heaviest first, to the currently lightest rank
  (:func:`assign_roles_to_lightest`).

Behavioural parity (golden vectors in ``tests/test_planner.py``):
``matrix_fsdp/planning/planner.py:46-998``.  Additions for B200: role weights can be a
callable (e.g. Newton-Schulz FLOPs instead of element counts) and the even split can be
aligned to 16-byte vectors so every peer shard is addressable by TMA / 128-bit loads.
"""
from __future__ import annotations

from collections.abc import Callable, Sequence
from dataclasses import dataclass
from typing import Protocol

from ..core.layout import LayoutSegment, MatrixGroupLayout, ShardPlan, coalesce_segments, contiguous_shard_plan
from ..core.managed_param import ParamRuntimeKind, ParamShardHint


class PlannerParam(Protocol):
    fqn: str
    numel: int
    offset: int
    end: int
    shape: Sequence[int]
    shard_hint: ParamShardHint


BlockSizeFn = Callable[[PlannerParam], int]
RowBlockFn = Callable[[PlannerParam], int]
RoleWeightFn = Callable[[Sequence[PlannerParam]], int]
ShardGranularity = str


@dataclass(frozen=True)
class ParamBlock:
    fqn: str
    global_start: int
    global_end: int
    block_index: int
    kind: str = "parameter"

    @property
    def numel(self) -> int:
        return self.global_end - self.global_start


BlockBuilder = Callable[[PlannerParam], Sequence[ParamBlock]]


def _check_world(world_size: int) -> None:
    if world_size <= 0:
        raise ValueError(f"world_size must be positive, got {world_size}.")


def _hint(param) -> ParamShardHint:
    return getattr(param, "shard_hint", None) or ParamShardHint()


def _total(params: Sequence[PlannerParam]) -> int:
    return sum(p.numel for p in params)


# --------------------------------------------------------------------------- even split
def contiguous_even_plan(total_numel: int, world_size: int, *, align: int = 1) -> ShardPlan:
    """Flat even split that ignores parameter boundaries.

    ``align > 1`` rounds every boundary to a multiple of ``align`` elements (the last rank
    absorbs the remainder) so shards start on vector / TMA boundaries.
    """
    _check_world(world_size)
    if align <= 1:
        base, rem = divmod(total_numel, world_size)
        sizes = tuple(base + (1 if r < rem else 0) for r in range(world_size))
    else:
        units, tail = divmod(total_numel, align)
        base, rem = divmod(units, world_size)
        sizes_l = [(base + (1 if r < rem else 0)) * align for r in range(world_size)]
        sizes_l[-1] += tail
        sizes = tuple(sizes_l)
    return contiguous_shard_plan(total_numel, sizes)


def _ordered_params(params: Sequence[PlannerParam], order_policy: str = "default") -> list[PlannerParam]:
    if order_policy == "default":
        return list(params)
    if order_policy == "largest_first":
        return sorted(params, key=lambda p: (-p.numel, p.offset))
    if order_policy == "offset":
        return sorted(params, key=lambda p: p.offset)
    raise ValueError(f"Unknown order_policy={order_policy!r}.")


# --------------------------------------------------------------------------- owner layouts
def _layout_from_assignments(params: Sequence[PlannerParam], world_size: int,
                             assignments: Sequence[tuple[PlannerParam, int]], *,
                             merge_adjacent_rank_segments: bool = False) -> MatrixGroupLayout:
    """Whole-parameter layout: each (param, rank) pair appends the param to that rank's shard."""
    per_rank: list[list[LayoutSegment]] = [[] for _ in range(world_size)]
    cursor = [0] * world_size
    for p, rank in assignments:
        if not 0 <= rank < world_size:
            raise ValueError(f"Owner rank for parameter {p.fqn!r} must be in [0, {world_size}), got {rank}.")
        per_rank[rank].append(LayoutSegment(p.offset, p.end, cursor[rank]))
        cursor[rank] += p.numel
    if merge_adjacent_rank_segments:
        per_rank = [list(coalesce_segments(s)) for s in per_rank]
    return MatrixGroupLayout.from_rank_segments(_total(params), per_rank, params)


def _fixed_owner_rank(params: Sequence[PlannerParam], world_size: int) -> int | None:
    pinned = {_hint(p).owner_rank for p in params if _hint(p).owner_rank is not None}
    if not pinned:
        return None
    if len(pinned) != 1:
        raise ValueError(f"Conflicting owner_rank hints for params: {', '.join(p.fqn for p in params)}.")
    rank = next(iter(pinned))
    if rank >= world_size:
        raise ValueError(f"owner_rank={rank} must be in [0, {world_size}).")
    return rank


def _initial_units(initial_rank_units: Sequence[int] | None, world_size: int) -> list[int]:
    if initial_rank_units is None:
        return [0] * world_size
    if len(initial_rank_units) != world_size:
        raise ValueError(
            f"initial_rank_units length must match world_size={world_size}, got {len(initial_rank_units)}.")
    return list(initial_rank_units)


def assign_roles_to_lightest(roles: Sequence[tuple[int, tuple, tuple[PlannerParam, ...]]], rank_units: list[int],
                             world_size: int) -> list[tuple[tuple, tuple[PlannerParam, ...], int]]:
    """Heaviest role first → currently lightest rank (ties: lowest rank).  Mutates ``rank_units``.

    ``roles`` entries are ``(weight, tie_break_key, params)``.
    """
    out = []
    for weight, key, role_params in sorted(roles, key=lambda r: (-r[0], r[1])):
        fixed = _fixed_owner_rank(role_params, world_size)
        rank = fixed if fixed is not None else min(range(world_size), key=lambda r: (rank_units[r], r))
        rank_units[rank] += weight
        out.append((key, role_params, rank))
    return out


def _matrix_and_tail(params: Sequence[PlannerParam]):
    mats = [p for p in params if len(p.shape) == 2]
    tail = [p for p in params if len(p.shape) != 2]
    return mats, tail


def parameter_boundary_plan(params: Sequence[PlannerParam], world_size: int, *,
                            order_policy: str = "default") -> MatrixGroupLayout:
    """Whole parameters, in the chosen order, each to the currently lightest rank."""
    _check_world(world_size)
    units = [0] * world_size
    assignments = []
    for p in _ordered_params(params, order_policy):
        rank = min(range(world_size), key=lambda r: (units[r], r))
        units[rank] += p.numel
        assignments.append((p, rank))
    return _layout_from_assignments(params, world_size, assignments)


def ordered_matrix_owner_tail_plan(params: Sequence[PlannerParam], world_size: int) -> MatrixGroupLayout:
    """Matrix ``i`` → rank ``i % W`` in module order; all non-2-D params packed after them."""
    _check_world(world_size)
    mats, tail = _matrix_and_tail(params)
    tail_rank = min(len(mats), world_size - 1)
    assignments = [(p, i % world_size) for i, p in enumerate(mats)] + [(p, tail_rank) for p in tail]
    return _layout_from_assignments(params, world_size, assignments)


def load_balanced_matrix_owner_tail_plan(params: Sequence[PlannerParam], world_size: int, *,
                                         initial_rank_units: Sequence[int] | None = None,
                                         merge_adjacent_rank_segments: bool = False,
                                         role_weight_fn: RoleWeightFn | None = None) -> MatrixGroupLayout:
    """Role-greedy owner plan: each matrix is a role, all non-2-D params form one tail role."""
    _check_world(world_size)
    units = _initial_units(initial_rank_units, world_size)
    weight = role_weight_fn or _total
    mats, tail = _matrix_and_tail(params)
    roles = [(weight((p,)), (i,), (p,)) for i, p in enumerate(mats)]
    if tail:
        roles.append((weight(tuple(tail)), (len(mats),), tuple(tail)))
    assignments = [(p, rank) for _, ps, rank in assign_roles_to_lightest(roles, units, world_size) for p in ps]
    return _layout_from_assignments(params, world_size, assignments,
                                    merge_adjacent_rank_segments=merge_adjacent_rank_segments)


def load_balanced_matrix_owner_tail_group_plans(param_groups: Sequence[Sequence[PlannerParam]], world_size: int, *,
                                                initial_rank_units: Sequence[int] | None = None,
                                                merge_adjacent_rank_segments: bool = True,
                                                role_weight_fn: RoleWeightFn | None = None,
                                                ) -> tuple[MatrixGroupLayout, ...]:
    """Scope-greedy: one owner decision over the roles of *all* groups, one layout per group."""
    _check_world(world_size)
    units = _initial_units(initial_rank_units, world_size)
    weight = role_weight_fn or _total
    roles = []
    for g, params in enumerate(param_groups):
        mats, tail = _matrix_and_tail(params)
        roles += [(weight((p,)), (g, i), (p,)) for i, p in enumerate(mats)]
        if tail:
            roles.append((weight(tuple(tail)), (g, len(mats)), tuple(tail)))
    per_group: list[list[tuple[PlannerParam, int]]] = [[] for _ in param_groups]
    for key, ps, rank in assign_roles_to_lightest(roles, units, world_size):
        per_group[key[0]] += [(p, rank) for p in ps]
    return tuple(
        _layout_from_assignments(params, world_size, per_group[g],
                                 merge_adjacent_rank_segments=merge_adjacent_rank_segments)
        for g, params in enumerate(param_groups))


def expert_owner_tail_plan(params: Sequence[PlannerParam], world_size: int, *,
                           initial_rank_units: Sequence[int] | None = None,
                           dense_order_policy: str = "largest_first",
                           merge_adjacent_rank_segments: bool = True) -> MatrixGroupLayout:
    """All parameters of one routed expert stay on one rank; dense params fill the lightest ranks."""
    _check_world(world_size)
    units = _initial_units(initial_rank_units, world_size)
    experts: dict[str, list[PlannerParam]] = {}
    dense: list[PlannerParam] = []
    for p in params:
        h = _hint(p)
        if h.runtime_kind == ParamRuntimeKind.EXPERT_OWNER or h.expert_group_id:
            experts.setdefault(h.expert_group_id or p.fqn, []).append(p)
        else:
            dense.append(p)
    roles = [(_total(ps), (min(q.offset for q in ps),), tuple(ps)) for ps in experts.values()]
    assignments = [(p, rank) for _, ps, rank in assign_roles_to_lightest(roles, units, world_size) for p in ps]
    for p in _ordered_params(dense, dense_order_policy):
        fixed = _fixed_owner_rank((p,), world_size)
        rank = fixed if fixed is not None else min(range(world_size), key=lambda r: (units[r], r))
        units[rank] += p.numel
        assignments.append((p, rank))
    return _layout_from_assignments(params, world_size, assignments,
                                    merge_adjacent_rank_segments=merge_adjacent_rank_segments)


def fsdp2_chunk_plan(params: Sequence[PlannerParam], world_size: int, *,
                     order_policy: str = "default") -> MatrixGroupLayout:
    """FSDP2-style: every parameter is cut into ``W`` equal chunks, rank r keeps chunk r of each."""
    _check_world(world_size)
    per_rank: list[list[LayoutSegment]] = [[] for _ in range(world_size)]
    cursor = [0] * world_size
    for p in _ordered_params(params, order_policy):
        if p.numel % world_size != 0:
            raise ValueError(
                f"fsdp2_chunk_plan requires parameter {p.fqn!r} numel={p.numel} "
                f"to be divisible by world_size={world_size}.")
        chunk = p.numel // world_size
        for r in range(world_size):
            per_rank[r].append(LayoutSegment(p.offset + r * chunk, p.offset + (r + 1) * chunk, cursor[r]))
            cursor[r] += chunk
    return MatrixGroupLayout.from_rank_segments(_total(params), per_rank, params)


# --------------------------------------------------------------------------- block builders
def whole_param_blocks(param: PlannerParam) -> tuple[ParamBlock, ...]:
    return (ParamBlock(param.fqn, param.offset, param.end, 0, "parameter"),)


def _requires_whole_parameter(hint: ParamShardHint) -> bool:
    return hint.split_granularity in ("parameter", "matrix_owner")


def _block_size_from_hint(hint: ParamShardHint) -> int | None:
    if hint.block_shape is None or hint.split_granularity != "block":
        return None
    if len(hint.block_shape) != 1:
        raise ValueError(f"block split_granularity expects a 1D block_shape, got {hint.block_shape}.")
    return hint.block_shape[0]


def _row_block_from_hint(hint: ParamShardHint) -> int | None:
    if hint.block_shape is None or hint.split_granularity != "row_block":
        return None
    if len(hint.block_shape) in (1, 2):
        return hint.block_shape[0]
    raise ValueError(f"row_block split_granularity expects a 1D or 2D block_shape, got {hint.block_shape}.")


def _cut(param: PlannerParam, step: int, kind: str, *, strict: bool) -> tuple[ParamBlock, ...]:
    if step <= 0:
        raise ValueError(f"block_size_fn returned {step} for {param.fqn}.")
    if strict and param.numel % step != 0:
        raise ValueError(f"Parameter {param.fqn} numel={param.numel} is not divisible by block_size={step}.")
    return tuple(ParamBlock(param.fqn, s, min(s + step, param.end), i, kind)
                 for i, s in enumerate(range(param.offset, param.end, step)))


def uniform_block_builder(block_size_fn: BlockSizeFn, *, kind: str = "uniform") -> BlockBuilder:
    """Strict equal 1-D blocks (a size that does not divide the parameter raises)."""
    def build(param: PlannerParam) -> tuple[ParamBlock, ...]:
        h = _hint(param)
        if _requires_whole_parameter(h):
            return whole_param_blocks(param)
        return _cut(param, _block_size_from_hint(h) or block_size_fn(param), kind, strict=True)
    return build


def bounded_block_builder(block_size_fn: BlockSizeFn, *, kind: str = "block") -> BlockBuilder:
    """Best-effort 1-D blocks: a smaller tail block is allowed unless the hint is explicit."""
    def build(param: PlannerParam) -> tuple[ParamBlock, ...]:
        h = _hint(param)
        if _requires_whole_parameter(h):
            return whole_param_blocks(param)
        if h.split_granularity == "block":
            return uniform_block_builder(block_size_fn, kind=kind)(param)
        return _cut(param, block_size_fn(param), kind, strict=False)
    return build


def _rows_cols(param: PlannerParam) -> tuple[int, int]:
    if len(param.shape) != 2:
        raise ValueError(f"Parameter {param.fqn} must be 2D for matrix row blocks, got shape={tuple(param.shape)}.")
    return int(param.shape[0]), int(param.shape[1])


def matrix_row_block_builder(row_block_fn: RowBlockFn, *, kind: str = "matrix_row_block") -> BlockBuilder:
    """Strict row blocks of a 2-D matrix."""
    def build(param: PlannerParam) -> tuple[ParamBlock, ...]:
        h = _hint(param)
        if _requires_whole_parameter(h):
            return whole_param_blocks(param)
        rows, cols = _rows_cols(param)
        rb = _row_block_from_hint(h) or row_block_fn(param)
        if rb <= 0:
            raise ValueError(f"row_block_fn returned {rb} for {param.fqn}.")
        if rows % rb != 0:
            raise ValueError(f"Parameter {param.fqn} rows={rows} is not divisible by row_block={rb}.")
        return _cut(param, rb * cols, kind, strict=True)
    return build


def bounded_matrix_row_block_builder(row_block_fn: RowBlockFn, *, kind: str = "matrix_row_block") -> BlockBuilder:
    """Best-effort row blocks (final block may hold fewer rows)."""
    def build(param: PlannerParam) -> tuple[ParamBlock, ...]:
        h = _hint(param)
        if _requires_whole_parameter(h):
            return whole_param_blocks(param)
        if h.split_granularity == "row_block":
            return matrix_row_block_builder(row_block_fn, kind=kind)(param)
        _, cols = _rows_cols(param)
        rb = row_block_fn(param)
        if rb <= 0:
            raise ValueError(f"row_block_fn returned {rb} for {param.fqn}.")
        return _cut(param, rb * cols, kind, strict=False)
    return build


def _default_row_block_units(param: PlannerParam, explicit: int | RowBlockFn | None) -> int:
    if callable(explicit):
        return explicit(param)
    if explicit is not None:
        return explicit
    return max(1, int(param.shape[0])) if len(param.shape) == 2 else 1


def hint_aware_block_builder(*, default_granularity: ShardGranularity = "parameter",
                             target_block_units: int | None = None,
                             row_block_units: int | RowBlockFn | None = None,
                             block_kind: str = "block") -> BlockBuilder:
    """Each parameter's legal cut points follow its ``ParamShardHint`` (explicit hints are strict)."""
    valid = {"parameter", "matrix_owner", "block", "row_block"}
    if default_granularity not in valid:
        raise ValueError(
            f"Unknown default_granularity={default_granularity!r}. Valid granularities: {', '.join(sorted(valid))}.")
    if target_block_units is not None and target_block_units <= 0:
        raise ValueError(f"target_block_units must be positive, got {target_block_units}.")
    if isinstance(row_block_units, int) and row_block_units <= 0:
        raise ValueError(f"row_block_units must be positive, got {row_block_units}.")

    def block_units(p: PlannerParam) -> int:
        return target_block_units or max(1, p.numel)

    def row_units(p: PlannerParam) -> int:
        return _default_row_block_units(p, row_block_units)

    def build(param: PlannerParam) -> tuple[ParamBlock, ...]:
        h = _hint(param)
        g = h.split_granularity or default_granularity
        if g in ("parameter", "matrix_owner"):
            return whole_param_blocks(param)
        if g == "block":
            maker = uniform_block_builder if h.split_granularity == "block" else bounded_block_builder
            return maker(block_units, kind=block_kind)(param)
        if g == "row_block":
            explicit = h.split_granularity == "row_block"
            if len(param.shape) != 2 and not explicit:
                return whole_param_blocks(param)
            maker = matrix_row_block_builder if explicit else bounded_matrix_row_block_builder
            return maker(row_units)(param)
        raise ValueError(f"Unknown split_granularity={g!r} for parameter {param.fqn}.")
    return build


def validate_param_blocks(param: PlannerParam, blocks: Sequence[ParamBlock]) -> None:
    cursor, seen = param.offset, set()
    for b in sorted(blocks, key=lambda c: (c.global_start, c.global_end)):
        if b.fqn != param.fqn:
            raise ValueError(f"Block for {b.fqn} cannot be used for parameter {param.fqn}.")
        if b.block_index in seen:
            raise ValueError(f"Parameter {param.fqn} has duplicate block_index={b.block_index}.")
        seen.add(b.block_index)
        if b.global_start < param.offset or b.global_end > param.end:
            raise ValueError(f"Block {b} crosses parameter {param.fqn} boundary.")
        if b.global_start < cursor:
            raise ValueError(f"Parameter {param.fqn} blocks overlap at {b}.")
        if b.global_start > cursor:
            raise ValueError(f"Parameter {param.fqn} blocks have gap before {b}.")
        if b.global_start >= b.global_end:
            raise ValueError(f"Parameter {param.fqn} has empty block {b}.")
        cursor = b.global_end
    if cursor != param.end:
        raise ValueError(f"Parameter {param.fqn} block coverage ends at {cursor}, expected {param.end}.")


def split_blocks_across_ranks(blocks: Sequence[ParamBlock], total_numel: int, world_size: int) -> list[list[ParamBlock]]:
    """Greedy cut: rank r takes blocks while that moves its end closer to ``total*(r+1)/W``."""
    groups: list[list[ParamBlock]] = []
    idx = assigned = 0
    for rank in range(world_size):
        if rank == world_size - 1:
            groups.append(list(blocks[idx:]))
            break
        target = round(total_numel * (rank + 1) / world_size)
        mine: list[ParamBlock] = []
        while idx < len(blocks):
            n = blocks[idx].numel
            if mine and abs(assigned + n - target) > abs(assigned - target):
                break
            mine.append(blocks[idx])
            assigned += n
            idx += 1
            if assigned >= target:
                break
        groups.append(mine)
    return groups


def ordered_group_plan(params: Sequence[PlannerParam], world_size: int, *, block_builder: BlockBuilder | None = None,
                       block_size_fn: BlockSizeFn | None = None, order_policy: str = "default") -> MatrixGroupLayout:
    """Keep tensor order, cut the group buffer into rank-contiguous intervals at block boundaries."""
    _check_world(world_size)
    if block_builder is not None and block_size_fn is not None:
        raise ValueError("Pass only one of block_builder or block_size_fn.")
    total = _total(params)
    if total == 0:
        return MatrixGroupLayout.from_rank_segments(0, [() for _ in range(world_size)])
    builder = block_builder or (uniform_block_builder(block_size_fn) if block_size_fn else whole_param_blocks)
    blocks: list[ParamBlock] = []
    for p in _ordered_params(params, order_policy):
        pb = tuple(builder(p))
        validate_param_blocks(p, pb)
        blocks.extend(pb)
    per_rank = []
    for group in split_blocks_across_ranks(blocks, total, world_size):
        segs, local = [], 0
        for b in group:
            segs.append(LayoutSegment(b.global_start, b.global_end, local))
            local += b.numel
        per_rank.append(coalesce_segments(segs))
    return MatrixGroupLayout.from_rank_segments(total, per_rank, params)


def hinted_ordered_group_plan(params: Sequence[PlannerParam], world_size: int, *,
                              default_granularity: ShardGranularity = "parameter",
                              target_block_units: int | None = None,
                              row_block_units: int | RowBlockFn | None = None, block_kind: str = "block",
                              order_policy: str = "default") -> MatrixGroupLayout:
    """Rank-contiguous layout whose cut points obey every parameter's shard hint."""
    builder = hint_aware_block_builder(default_granularity=default_granularity,
                                       target_block_units=target_block_units,
                                       row_block_units=row_block_units, block_kind=block_kind)
    return ordered_group_plan(params, world_size, block_builder=builder, order_policy=order_policy)


def rotate_layout_ranks(layout: MatrixGroupLayout, rank_offset: int) -> MatrixGroupLayout:
    """Shift ownership by ``rank_offset`` ranks, keeping each rank's internal order."""
    world = layout.world_size
    if world <= 0 or rank_offset % world == 0:
        return layout
    rank_offset %= world
    per_rank: list[list[LayoutSegment]] = [[] for _ in range(world)]
    for old_rank, segs in enumerate(layout.rank_segments):
        new_rank = (old_rank + rank_offset) % world
        local = 0
        for s in segs:
            per_rank[new_rank].append(LayoutSegment(s.global_start, s.global_end, local))
            local += s.numel

    class _P:  # ParamLayout → LayoutParam adapter
        def __init__(self, pl):
            self.fqn, self.offset, self.end = pl.fqn, pl.global_start, pl.global_end

    return MatrixGroupLayout.from_rank_segments(layout.total_numel, per_rank, [_P(p) for p in layout.params])
