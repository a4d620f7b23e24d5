"""Parameter-buffer descriptors (what the transports read their copy tables and staging sizes from), one property
per test.  The reference's counterparts are test/fsdp/test_static_param_buffer.py (4 tests) and
test/fsdp/test_elastic_param_buffer.py (13 tests)."""
import pytest
import torch
from torch import nn

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.parallel.collectives import SegmentTables
from matrix_fsdp_b200.parallel.param_buffers import (ElasticParamBuffer, ElasticParamBufferLayout, StaticParamBuffer,
                                                     StaticParamBufferLayout, describe_unit_param_buffer)
from matrix_fsdp_b200.parallel.workspace_cache import CommWorkspaceCache

CPU = torch.device("cpu")


# ------------------------------------------------------------------------------------------ static
def test_static_layout_reports_the_cost_of_padding_to_the_largest_shard():
    lay = StaticParamBufferLayout((4, 6, 2))
    assert lay.world_size == 3 and lay.total_shard_numel == 12 and lay.max_shard_size == 6 and lay.min_shard_size == 2
    assert lay.padded_numel == 18 and lay.padding_waste_numel == 6 and lay.padding_waste_ratio == pytest.approx(0.5)
    assert lay.owner_imbalance_ratio == pytest.approx(1.5)


def test_static_layout_derives_rank_ordered_chunks_from_the_sizes():
    lay = StaticParamBufferLayout((3, 0, 5))
    assert lay.rank_segments == ((S(0, 3, 0),), (), (S(3, 8, 0),))
    assert lay.rank_chunk_fast_path and lay.packed_rank_shards_are_full_tensor_order and lay.segment_count == 2


def test_static_equal_shards_need_no_workspace():
    buf = StaticParamBuffer(StaticParamBufferLayout((5, 5)), total_numel=10)
    plan = buf.workspace_plan(can_direct_all_gather=True)
    assert not plan.needs_workspace and plan.kind == "none" and plan.preferred_workspace_numel == 0
    assert plan.padding_waste_ratio == 0.0


def test_static_uneven_shards_stage_through_padded_rank_chunks():
    buf = StaticParamBuffer(StaticParamBufferLayout((4, 6)), total_numel=10)
    plan = buf.workspace_plan(can_direct_all_gather=False)
    assert plan.needs_workspace and plan.preferred_workspace_kind == "padded_rank_chunks"
    assert plan.preferred_workspace_numel == 12 and plan.padding_waste_ratio == pytest.approx(0.2)


def test_static_summary_names_the_library_collectives_it_resolves_to():
    buf = StaticParamBuffer(StaticParamBufferLayout((5, 5)), total_numel=10)
    s = buf.communication_summary(param_gather_strategy="auto", matrix_collective_backend="owner_broadcast",
                                  can_direct_all_gather=True)
    assert s["param_buffer_type"] == "static" and s["effective_param_gather_backend"] == "all_gather_into_tensor"
    assert s["effective_grad_reduce_backend"] == "reduce_scatter_tensor" and s["owner_segment_collectives"] is False
    assert s["workspace_needed"] is False and s["world_size"] == 2


def test_summary_follows_the_transport_kind():
    buf = StaticParamBuffer(StaticParamBufferLayout((5, 5)), total_numel=10)
    common = dict(param_gather_strategy="auto", matrix_collective_backend="custom", can_direct_all_gather=True)
    assert buf.communication_summary(transport_kind="peer", **common)["effective_param_gather_backend"] == "peer_pull"
    assert buf.communication_summary(transport_kind="peer", **common)["effective_grad_reduce_backend"] == "peer_pull_reduce"
    assert buf.communication_summary(transport_kind="local", **common)["effective_param_gather_backend"] == "local_copy"


def test_an_explicit_gather_strategy_is_reported_as_given():
    buf = StaticParamBuffer(StaticParamBufferLayout((4, 6)), total_numel=10)
    for strategy in ("owner_broadcast", "uneven_all_gather", "all_reduce", "matrix_all_gather"):
        assert buf.effective_param_gather_backend(param_gather_strategy=strategy, can_direct_all_gather=False) == strategy
    assert buf.effective_param_gather_backend(param_gather_strategy="auto", can_direct_all_gather=False) == "padded_all_gather"


# ------------------------------------------------------------------------------------------ elastic
def _elastic(sizes, segs, total):
    return ElasticParamBuffer(ElasticParamBufferLayout(tuple(sizes), segs), total_numel=total)


def test_elastic_layout_counts_segments_and_reports_imbalance():
    segs = ((S(0, 3, 0), S(8, 10, 3)), (S(3, 8, 0),))
    lay = ElasticParamBufferLayout((5, 5), segs)
    assert lay.segment_count == 3 and lay.max_segments_per_rank == 2 and not lay.rank_chunk_fast_path
    assert not lay.packed_rank_shards_are_full_tensor_order and lay.padding_waste_numel == 0
    assert lay.owner_imbalance_ratio == pytest.approx(1.0)


def test_communication_plan_merges_pieces_adjacent_in_both_spaces():
    buf = _elastic((6, 4), ((S(0, 3, 0), S(3, 6, 3)), (S(6, 10, 0),)), 10)
    plan = buf.communication_plan
    assert plan.segment_count == 3 and plan.coalesced_segment_count == 2 and plan.rank_chunk_count == 2
    assert plan.rank_chunk_shard_sizes == (6, 4)                     # one chunk per rank after merging: fast path
    assert plan.peer_pull_table() == ((0, 0, 0, 6), (1, 0, 6, 4))


def test_pieces_adjacent_in_one_space_only_do_not_merge():
    # globally adjacent but packed in reverse locally
    buf = _elastic((6, 4), ((S(0, 3, 3), S(3, 6, 0)), (S(6, 10, 0),)), 10)
    plan = buf.communication_plan
    assert plan.coalesced_segment_count == 3 and plan.rank_chunk_shard_sizes is None
    assert plan.max_coalesced_segments_per_rank == 2
    assert plan.peer_pull_table() == ((0, 3, 0, 3), (0, 0, 3, 3), (1, 0, 6, 4))


def test_empty_ranks_contribute_no_pull_rows():
    buf = _elastic((7, 0, 3), ((S(0, 7, 0),), (), (S(7, 10, 0),)), 10)
    assert [row[0] for row in buf.communication_plan.peer_pull_table()] == [0, 2]
    assert buf.communication_plan.nonempty_rank_chunk_count == 2


def test_elastic_workspace_is_needed_only_by_the_library_transport():
    buf = _elastic((6, 4), ((S(0, 6, 0),), (S(6, 10, 0),)), 10)
    lib = buf.workspace_plan(can_direct_all_gather=False, transport_kind="torch_dist")
    assert lib.needs_workspace and lib.kind == "padded_rank_chunks" and lib.preferred_workspace_numel == 12
    compact = buf.workspace_plan(can_direct_all_gather=False, transport_kind="torch_dist", compact=True)
    assert compact.kind == "compact_rank_chunks" and compact.preferred_workspace_numel == 10
    assert not buf.workspace_plan(can_direct_all_gather=False, transport_kind="peer").needs_workspace
    assert not buf.workspace_plan(can_direct_all_gather=True).needs_workspace


def test_elastic_summary_reports_reduce_backend_per_transport_and_request():
    buf = _elastic((6, 4), ((S(0, 6, 0),), (S(6, 10, 0),)), 10)
    common = dict(param_gather_strategy="auto", matrix_collective_backend="custom", can_direct_all_gather=False)
    assert buf.communication_summary(**common)["effective_grad_reduce_backend"] == "padded_reduce_scatter"
    assert buf.communication_summary(reduce_impl="owner_reduce", **common)["effective_grad_reduce_backend"] == "owner_reduce"
    peer = buf.communication_summary(transport_kind="peer", **common)
    assert peer["effective_grad_reduce_backend"] == "peer_pull_reduce" and peer["owner_segment_collectives"] is True
    assert peer["communication_rank_chunk_fast_path"] is True and peer["param_buffer_type"] == "elastic"


def test_workspace_cache_reuses_a_released_tensor_of_the_same_shape_dtype_and_device():
    cache = CommWorkspaceCache(max_cached_per_key=1)
    a = cache.lease(16, torch.float32, CPU)
    ptr = a.tensor.data_ptr()
    assert not a.reused
    a.release()
    b = cache.lease(16, torch.float32, CPU)
    assert b.reused and b.tensor.data_ptr() == ptr
    c = cache.lease(16, torch.bfloat16, CPU)                          # another dtype: another tensor
    assert not c.reused and c.tensor.data_ptr() != ptr


def test_workspace_cache_never_hands_out_a_tensor_that_is_in_use():
    cache = CommWorkspaceCache(max_cached_per_key=2)
    a = cache.lease(8, torch.float32, CPU)
    b = cache.lease(8, torch.float32, CPU)
    assert a.tensor.data_ptr() != b.tensor.data_ptr() and not b.reused
    a.release()
    b.release()
    assert cache.stats()["cached"] == 2 and cache.stats()["allocations"] == 2


def test_workspace_cache_can_be_switched_off():
    cache = CommWorkspaceCache(max_cached_per_key=0)
    a = cache.lease(8, torch.float32, CPU)
    a.release()
    b = cache.lease(8, torch.float32, CPU)
    assert not b.reused and cache.stats()["cached"] == 0 and cache.stats()["reuses"] == 0


def test_rank_chunk_workspace_of_a_descriptor_is_leased_from_its_own_cache():
    buf = _elastic((6, 4), ((S(0, 6, 0),), (S(6, 10, 0),)), 10)
    lease = buf.acquire_rank_chunk_workspace(dtype=torch.float32, device=CPU)
    assert lease.tensor.numel() == 12 and not lease.reused
    lease.release()
    again = buf.acquire_rank_chunk_workspace(dtype=torch.float32, device=CPU)
    assert again.reused
    compact = buf.acquire_rank_chunk_workspace(dtype=torch.float32, device=CPU, compact=True)
    assert compact.tensor.numel() == 10


# ------------------------------------------------------------------------------------------ wiring
def test_segment_tables_pick_the_descriptor_that_fits_the_layout():
    equal = SegmentTables.build(10, ((S(0, 5, 0),), (S(5, 10, 0),)), 0)
    assert isinstance(equal.param_buffer, StaticParamBuffer) and equal.staging_numel() == 0
    uneven = SegmentTables.build(10, ((S(0, 6, 0),), (S(6, 10, 0),)), 0)
    assert isinstance(uneven.param_buffer, ElasticParamBuffer) and uneven.staging_numel("torch_dist") == 12
    assert uneven.staging_numel("peer") == 0
    assert uneven.pull_rows() == ((0, 0, 0, 6), (1, 0, 6, 4))


def test_a_unit_describes_its_own_buffer():
    from matrix_fsdp_b200 import fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    m = nn.Linear(4, 4)
    fully_shard(m)
    desc = describe_unit_param_buffer(m._matrix_fsdp_param_group)
    assert isinstance(desc, StaticParamBuffer) and desc.total_numel == 20 and desc.layout.shard_sizes == (20,)
