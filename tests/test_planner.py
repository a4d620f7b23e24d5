"""Planner golden vectors (even split, whole-param, owner plans, block plans, stateful planners)."""
from dataclasses import dataclass, field

import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry, ParamShardHint
from matrix_fsdp_b200.planning import planner as P
from matrix_fsdp_b200.planning.auto_planner import (auto_group_plan, build_auto_planner_report,
                                                    format_auto_planner_report,
                                                    make_cost_aware_muon_shard_aware_group_planner,
                                                    make_model_wide_muon_planner, make_muon_shard_aware_group_planner,
                                                    make_scoped_muon_shard_aware_group_planner)
from matrix_fsdp_b200.planning.layout_validator import explain_runtime_layout_compatibility, validate_group_layout
from matrix_fsdp_b200.planning.planner_eval import call_group_planner
from matrix_fsdp_b200.planning.shard_hint import build_shard_hints


@dataclass
class FP:
    fqn: str
    shape: tuple
    offset: int
    shard_hint: ParamShardHint = field(default_factory=ParamShardHint)
    dtype: torch.dtype = torch.float32

    @property
    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    @property
    def end(self):
        return self.offset + self.numel


def mk(shapes, hints=None):
    out, off = [], 0
    for i, sh in enumerate(shapes):
        sh = sh if isinstance(sh, tuple) else (sh,)
        p = FP(f"p{i}", sh, off, (hints or {}).get(i, ParamShardHint()))
        out.append(p)
        off = p.end
    return out


def test_contiguous_even_plan():
    plan = P.contiguous_even_plan(10, 4)
    assert plan.shard_sizes == (3, 3, 2, 2) and plan.shard_offsets == (0, 3, 6, 8)
    aligned = P.contiguous_even_plan(100, 3, align=8)
    assert aligned.shard_sizes == (32, 32, 36) and sum(aligned.shard_sizes) == 100
    with pytest.raises(ValueError):
        P.contiguous_even_plan(4, 0)


def test_parameter_boundary_plan():
    lay = P.parameter_boundary_plan(mk([5, 4, 3, 2]), 2)
    assert lay.shard_sizes == (7, 7)
    assert lay.rank_segments[0] == (S(0, 5, 0), S(12, 14, 5))
    assert lay.rank_segments[1] == (S(5, 9, 0), S(9, 12, 4))
    lay2 = P.parameter_boundary_plan(mk([2, 5, 4]), 2, order_policy="largest_first")
    assert lay2.owner_ranks("p1") == (0,) and lay2.owner_ranks("p2") == (1,) and lay2.owner_ranks("p0") == (1,)


def test_rotate_layout_ranks():
    lay = P.parameter_boundary_plan(mk([5, 4, 3]), 3)
    assert lay.shard_sizes == (5, 4, 3)
    rot = P.rotate_layout_ranks(lay, 1)
    assert rot.shard_sizes == (3, 5, 4)
    assert rot.owner_ranks("p0") == (1,)


def test_fsdp2_chunk_plan():
    lay = P.fsdp2_chunk_plan(mk([6, 4]), 2)
    assert lay.rank_segments[0] == (S(0, 3, 0), S(6, 8, 3))
    assert lay.rank_segments[1] == (S(3, 6, 0), S(8, 10, 3))
    with pytest.raises(ValueError, match="divisible"):
        P.fsdp2_chunk_plan(mk([5]), 2)


def test_ordered_group_plan():
    lay = P.ordered_group_plan(mk([5, 4, 3, 2]), 2)
    assert lay.shard_sizes == (9, 5)
    assert all(len(s) == 1 for s in lay.rank_segments)
    lay = P.ordered_group_plan(mk([6, 6]), 3, block_size_fn=lambda p: 3)
    assert lay.shard_sizes == (3, 6, 3)
    assert lay.owner_ranks("p0") == (0, 1)


def test_row_blocks_and_hints():
    params = mk([(6, 4)])
    b = P.matrix_row_block_builder(lambda p: 2)(params[0])
    assert [x.numel for x in b] == [8, 8, 8]
    owner = mk([(6, 4)], {0: ParamShardHint(split_granularity="matrix_owner")})
    assert len(P.matrix_row_block_builder(lambda p: 2)(owner[0])) == 1
    bounded = P.bounded_matrix_row_block_builder(lambda p: 4)(params[0])
    assert [x.numel for x in bounded] == [16, 8]
    with pytest.raises(ValueError, match="not divisible"):
        P.matrix_row_block_builder(lambda p: 4)(params[0])


def test_hinted_ordered_group_plan_respects_hints():
    hints = {
        0: ParamShardHint(split_granularity="row_block", block_shape=(2, 4)),   # 6x4 = 24
        1: ParamShardHint(split_granularity="parameter"),                        # 11
        2: ParamShardHint(split_granularity="block", block_shape=(4,)),           # 24
    }
    params = mk([(6, 4), 11, 24], hints)
    lay = P.hinted_ordered_group_plan(params, 3)
    assert sum(lay.shard_sizes) == 59
    assert len(lay.param("p1").segments) == 1
    for seg in lay.param("p0").segments:
        assert (seg.global_start - 0) % 8 == 0 and (seg.global_end - 0) % 8 == 0
    for seg in lay.param("p2").segments:
        assert (seg.global_start - 35) % 4 == 0


def test_expert_owner_tail_plan():
    def eh(e):
        return ParamShardHint(runtime_kind="expert_owner", expert_group_id=f"experts.{e}", expert_id=e)
    params = mk([8, 8, 4, 4, 10, 2], {0: eh(0), 1: eh(0), 2: eh(1), 3: eh(1),
                                      5: ParamShardHint(parallel_role="router")})
    lay = P.expert_owner_tail_plan(params, 2)
    assert lay.owner_ranks("p0") == lay.owner_ranks("p1") == (0,)
    assert lay.owner_ranks("p2") == lay.owner_ranks("p3") == (1,)
    assert lay.owner_ranks("p4") == (1,)            # dense(10) goes to the lighter rank (8 vs 16)
    assert sum(lay.shard_sizes) == 36


def split_qkv_block(prefix="", hidden=16, inter=64):
    shapes = [(hidden, hidden)] * 4 + [(inter // 2, hidden)] * 2 + [(hidden, inter // 2)] + [hidden] * 4
    names = ["q", "k", "v", "proj", "up0", "up1", "down", "norm1.w", "norm1.b", "norm2.w", "norm2.b"]
    out, off = [], 0
    for n, sh in zip(names, shapes):
        sh = sh if isinstance(sh, tuple) else (sh,)
        p = FP(prefix + n, sh, off)
        out.append(p)
        off = p.end
    return out


def test_matrix_owner_plans_on_split_qkv_block():
    blk = split_qkv_block()
    lay = P.ordered_matrix_owner_tail_plan(blk, 8)
    for i, n in enumerate(["q", "k", "v", "proj", "up0", "up1", "down"]):
        assert lay.owner_ranks(n) == (i,)
    assert all(lay.owner_ranks(n) == (7,) for n in ["norm1.w", "norm1.b", "norm2.w", "norm2.b"])
    lay = P.load_balanced_matrix_owner_tail_plan(blk, 8, initial_rank_units=(0, 0, 0, 1024, 1024, 0, 0, 0))
    assert lay.shard_sizes == (512, 512, 512, 0, 0, 512, 320, 256)
    assert tuple(s.numel for s in lay.rank_segments[6]) == (256, 16, 16, 16, 16)
    lay = P.load_balanced_matrix_owner_tail_plan(blk, 4, merge_adjacent_rank_segments=True)
    assert lay.owner_ranks("q") == lay.owner_ranks("k") == (3,)
    assert lay.rank_segments[3] == (S(0, 512, 0),)
    assert len(lay.rank_segments[2]) == 1 and lay.rank_segments[2][0].numel == 576


def test_stateful_muon_planners():
    blk = split_qkv_block()
    pl = make_muon_shard_aware_group_planner(matrix_owner_tail=True)
    a = pl(blk, 8)
    lay_a = a if not hasattr(a, "layout") else a.layout
    assert lay_a.owner_ranks("q") == (0,) and lay_a.owner_ranks("down") == (6,)
    b = pl(blk, 8)
    lay_b = b if not hasattr(b, "layout") else b.layout
    assert lay_b.owner_ranks("q") == (3,) and lay_b.owner_ranks("down") == (1,) and lay_b.owner_ranks("norm1.w") == (2,)
    rr = make_muon_shard_aware_group_planner(matrix_owner_tail=True, rotation_strategy="round_robin")
    rr(blk, 8)
    second = rr(blk, 8)
    lay = second if not hasattr(second, "layout") else second.layout
    assert lay.owner_ranks("q") == (1,) and lay.owner_ranks("down") == (7,)
    rg = make_muon_shard_aware_group_planner(owner_assignment="role_greedy")
    totals = [0] * 8
    results = [rg(blk, 8) for _ in range(4)]
    for r in results:
        for i, u in enumerate(r.layout.shard_sizes):
            totals[i] += u
    assert tuple(totals) == (1536, 1280, 1152, 1280, 1344, 1280, 1280, 1344)
    assert results[0].layout.owner_ranks("up0") == (0,) and results[0].layout.owner_ranks("q") == (3,)
    assert results[0].layout.owner_ranks("norm1.w") == (7,)
    assert results[1].layout.owner_ranks("up0") == (7,) and results[1].layout.owner_ranks("q") == (5,)
    assert results[0].name == "matrix_owner_tail_role_greedy" and results[0].policy == "muon_shard_aware"


def test_scope_and_cost_aware_planners():
    groups = [split_qkv_block(f"b{i}.") for i in range(4)]
    lays = P.load_balanced_matrix_owner_tail_group_plans(groups, 8)
    totals = [sum(l.shard_sizes[r] for l in lays) for r in range(8)]
    assert tuple(totals) == (1344, 1344, 1344, 1344, 1280, 1280, 1280, 1280)
    assert [l.owner_ranks(f"b{i}.up0")[0] for i, l in enumerate(lays)] == [0, 3, 6, 1]
    scoped = make_scoped_muon_shard_aware_group_planner(groups)
    assert scoped(groups[0], 8).name == "matrix_owner_tail_scope_greedy"
    with pytest.raises(RuntimeError, match="call order"):
        scoped(groups[0], 8)
    loose = make_cost_aware_muon_shard_aware_group_planner(groups, max_workspace_ratio=2.0,
                                                           max_workspace_padding_ratio=4.0)
    r = loose(groups[0], 8)
    assert "cost_aware_owner_assignment=scope_greedy" in r.warnings
    tight = make_cost_aware_muon_shard_aware_group_planner(groups, max_workspace_ratio=1.01,
                                                           max_workspace_padding_ratio=1.0)
    r = tight(groups[0], 8)
    assert "cost_aware_owner_assignment=role_greedy" in r.warnings
    wide = make_model_wide_muon_planner(groups)
    flops = [0] * 8
    for g in groups:
        res = wide(g, 8)
        validate_group_layout(res.layout, g, 8)


def test_auto_planner_policies_and_report():
    model = nn.Sequential(nn.Linear(8, 16), nn.LayerNorm(16), nn.Linear(16, 4))
    reg = ManagedParamRegistry.from_module(model, shard_hints=build_shard_hints(model))
    for policy in ("balanced", "min_comm", "max_balance", "muon_full_matrix", "zero_copy_friendly",
                   "muon_zero_copy", "muon_shard_aware", "debug"):
        res = auto_group_plan(reg.params, 2, policy=policy)
        assert res.runtime_compatible and res.policy == policy
        res.validate()
    rows = build_auto_planner_report(reg.params, 2, policy="muon_shard_aware")
    assert rows[0].selected and any(r.candidate == "matrix_owner_tail_role_greedy" for r in rows)
    text = format_auto_planner_report(rows)
    assert "candidate" in text and "selected=" in text
    with pytest.raises(ValueError, match="Unknown auto planner policy"):
        auto_group_plan(reg.params, 2, policy="nope")


def test_shard_hint_rules_and_runtime_mode():
    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(4, 2)
            self.emb = nn.Embedding(10, 4)
            self.lm_head = nn.Linear(4, 10, bias=False)
            self.gate = nn.Linear(4, 3, bias=False)
            self.experts = nn.ModuleList([nn.Linear(4, 4) for _ in range(2)])
    m = Blk()
    h = build_shard_hints(m)
    assert (h["fc.weight"].optimizer_type, h["fc.weight"].split_granularity) == ("muon", "matrix_owner")
    assert (h["fc.bias"].optimizer_type, h["fc.bias"].split_granularity) == ("adamw", "parameter")
    assert h["emb.weight"].optimizer_type == "adamw"
    assert h["lm_head.weight"].optimizer_type == "adamw"
    assert h["gate.weight"].parallel_role == "router"
    assert h["experts.1.weight"].expert_group_id == "experts.1" and h["experts.1.weight"].expert_id == 1
    reg = ManagedParamRegistry.from_module(nn.Linear(4, 2))
    res = call_group_planner(lambda ps, w: P.contiguous_even_plan(sum(p.numel for p in ps), w), reg.params, 2)
    assert res.runtime_mode == "matrix_shard" and res.matrix_shard_compatible
    lay = P.fsdp2_chunk_plan(reg.params, 2)
    assert explain_runtime_layout_compatibility(lay, reg.params, 2).mode == "segment_runtime"
