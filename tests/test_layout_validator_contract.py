"""The layout validator, one rule per test: each hand-built broken layout trips exactly the check it was built
for, and the runtime-mode classification follows the shape of a valid layout.  The reference's counterpart is
test/fsdp/test_layout_validator.py (18 tests)."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.core.layout import MatrixGroupLayout, ParamLayout, ParamSegment, RankLayout
from matrix_fsdp_b200.core.managed_param import ManagedParamRegistry, ParamShardHint
from matrix_fsdp_b200.planning.layout_validator import (explain_runtime_layout_compatibility, flat_reorder_order,
                                                        validate_group_layout, validate_runtime_layout)


def _params(hints=None):
    """Two parameters: ``w`` [4, 3] at [0, 12) and ``b`` [4] at [12, 16)."""
    torch.manual_seed(0)
    m = nn.Module()
    m.w = nn.Parameter(torch.randn(4, 3))
    m.b = nn.Parameter(torch.randn(4))
    return ManagedParamRegistry.from_module(m, shard_hints=hints).params


def _layout(rank_segments, params):
    return MatrixGroupLayout.from_rank_segments(16, rank_segments, params)


def _even(params):
    return _layout([[S(0, 8, 0)], [S(8, 16, 0)]], params)


# ------------------------------------------------------------------------------------------ accepted layouts
def test_an_even_split_is_valid_and_runs_as_matrix_shard():
    params = _params()
    validate_group_layout(_even(params), params, 2)
    compat = explain_runtime_layout_compatibility(_even(params), params, 2)
    assert compat.compatible and compat.mode == "matrix_shard" and compat.matrix_shard_compatible


def test_whole_parameter_owners_run_as_segment_runtime_and_say_why():
    params = _params()
    layout = _layout([[S(12, 16, 0)], [S(0, 12, 0)]], params)              # b on rank 0, w on rank 1: not rank ordered
    compat = explain_runtime_layout_compatibility(layout, params, 2)
    assert compat.compatible and compat.mode == "segment_runtime" and compat.reason and not compat.matrix_shard_compatible


def test_without_segment_runtime_a_whole_parameter_layout_is_reordered():
    params = _params()
    layout = _layout([[S(12, 16, 0)], [S(0, 12, 0)]], params)
    compat = explain_runtime_layout_compatibility(layout, params, 2, allow_segment_runtime=False)
    assert compat.mode == "flat_reorder" and compat.requires_flat_reorder
    assert flat_reorder_order(layout) == ["b", "w"]                        # rank-major order of the owners


def test_a_split_multi_segment_layout_has_no_fallback_when_segment_runtime_is_off():
    params = _params()
    layout = _layout([[S(0, 4, 0), S(10, 16, 4)], [S(4, 10, 0)]], params)
    compat = explain_runtime_layout_compatibility(layout, params, 2, allow_segment_runtime=False)
    assert not compat.compatible and compat.mode == "unsupported"
    with pytest.raises(ValueError, match="cannot execute planner layout"):
        validate_runtime_layout(layout, params, 2, allow_segment_runtime=False)
    assert validate_runtime_layout(layout, params, 2).mode == "segment_runtime"


def test_an_empty_rank_is_allowed():
    params = _params()
    layout = _layout([[S(0, 16, 0)], []], params)
    validate_group_layout(layout, params, 2)
    assert layout.shard_sizes == (16, 0)


# ------------------------------------------------------------------------------------------ structure checks
def test_world_size_has_to_match():
    params = _params()
    with pytest.raises(ValueError, match="world_size"):
        validate_group_layout(_even(params), params, 4)


def test_total_has_to_match_the_parameters():
    params = _params()
    layout = MatrixGroupLayout.from_rank_segments(20, [[S(0, 8, 0)], [S(8, 20, 0)]], params)
    with pytest.raises(ValueError, match="total_numel"):
        validate_group_layout(layout, params, 2)


def test_parameter_set_has_to_match():
    params = _params()
    layout = _layout([[S(0, 8, 0)], [S(8, 16, 0)]], params[:1])            # the layout does not know ``b``
    with pytest.raises(ValueError, match="parameter set"):
        validate_group_layout(layout, params, 2)


def test_a_gap_between_rank_segments_is_found():
    params = _params()
    layout = _layout([[S(0, 7, 0)], [S(8, 16, 0)]], params)
    with pytest.raises(ValueError, match="gap"):
        validate_group_layout(layout, params, 2)


def test_an_overlap_between_rank_segments_is_found():
    params = _params()
    layout = _layout([[S(0, 9, 0)], [S(8, 16, 0)]], params)
    with pytest.raises(ValueError, match="overlap"):
        validate_group_layout(layout, params, 2)


def test_a_segment_outside_the_flat_space_is_found():
    params = _params()
    layout = _layout([[S(0, 8, 0)], [S(8, 17, 0)]], params)
    with pytest.raises(ValueError, match="outside"):
        validate_group_layout(layout, params, 2)


def test_local_offsets_have_to_pack_the_shard_without_holes():
    params = _params()
    layout = _layout([[S(0, 4, 0), S(4, 8, 5)], [S(8, 16, 0)]], params)    # second piece should start at 4
    with pytest.raises(ValueError, match="local packing"):
        validate_group_layout(layout, params, 2)


def test_local_units_have_to_equal_what_the_segments_pack():
    params = _params()
    good = _even(params)
    broken = MatrixGroupLayout(16, (RankLayout(0, 9, good.ranks[0].segments), good.ranks[1]), good.params)
    with pytest.raises(ValueError, match="local_units"):
        validate_group_layout(broken, params, 2)


def test_a_parameter_range_that_disagrees_with_the_registry_is_found():
    params = _params()
    good = _even(params)
    w, b = good.params
    moved = ParamLayout("w", 1, 13, w.segments)
    with pytest.raises(ValueError, match="offset range"):
        validate_group_layout(MatrixGroupLayout(16, good.ranks, (moved, b)), params, 2)


def test_a_parameter_segment_has_to_lie_inside_a_segment_of_its_rank():
    params = _params()
    good = _even(params)
    w, b = good.params
    stray = ParamLayout("w", 0, 12, (ParamSegment("w", 0, 0, 8, 0), ParamSegment("w", 0, 8, 12, 8)))   # rank 0 ends at 8
    with pytest.raises(ValueError, match="not contained"):
        validate_group_layout(MatrixGroupLayout(16, good.ranks, (stray, b)), params, 2)


def test_parameter_segments_have_to_cover_the_parameter_exactly():
    params = _params()
    good = _even(params)
    w, b = good.params
    short = ParamLayout("w", 0, 12, (w.segments[0],))                       # the part on rank 1 is missing
    with pytest.raises(ValueError, match="cover"):
        validate_group_layout(MatrixGroupLayout(16, good.ranks, (short, b)), params, 2)


# ------------------------------------------------------------------------------------------ hint checks
def test_a_whole_parameter_hint_forbids_a_split():
    params = _params({"w": ParamShardHint(split_granularity="parameter")})
    with pytest.raises(ValueError, match="whole-parameter owner"):
        validate_group_layout(_even(params), params, 2)
    validate_group_layout(_layout([[S(0, 12, 0)], [S(12, 16, 0)]], params), params, 2)


def test_a_matrix_owner_hint_forbids_a_split():
    params = _params({"w": ParamShardHint(split_granularity="matrix_owner", optimizer_type="muon")})
    with pytest.raises(ValueError, match="matrix_owner"):
        validate_group_layout(_even(params), params, 2)


def test_row_block_hints_want_cuts_on_row_boundaries():
    params = _params({"w": ParamShardHint(split_granularity="row_block", block_shape=(1, 3))})
    with pytest.raises(ValueError, match="not aligned"):
        validate_group_layout(_even(params), params, 2)                     # cut at 8: inside row 2
    validate_group_layout(_layout([[S(0, 6, 0)], [S(6, 16, 0)]], params), params, 2)


def test_block_hints_want_cuts_on_block_boundaries():
    params = _params({"b": ParamShardHint(split_granularity="block", block_shape=(2,))})
    with pytest.raises(ValueError, match="not aligned"):
        validate_group_layout(_layout([[S(0, 13, 0)], [S(13, 16, 0)]], params), params, 2)
    validate_group_layout(_layout([[S(0, 14, 0)], [S(14, 16, 0)]], params), params, 2)
