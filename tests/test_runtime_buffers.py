"""Unit tests of the runtime's storage helpers: gradient-bucket packing (golden vectors), full-parameter
buffer pool, communication workspace cache, static / elastic buffer descriptors and the world-size-1
branches of the collectives and transports."""
import torch

from matrix_fsdp_b200.core.layout import LayoutSegment as S
from matrix_fsdp_b200.parallel.collectives import (MatrixCollectiveHandle, SegmentTables, gather_local_segments,
                                                   pack_rank_major_padded, scatter_local_segments)
from matrix_fsdp_b200.parallel.grad_bucket import BucketParam, MatrixGradBucket, classify_bucket_layout

CPU = torch.device("cpu")


# ------------------------------------------------------------------------------------ grad bucket
def test_padded_rank_major_packing_of_uneven_shards():
    # weight (2x3) = 10..15, bias (4) = 20..23, shards of 4 and 6 elements
    tables = SegmentTables.build(10, [(S(0, 4, 0),), (S(4, 10, 0),)], rank=0)
    params = [BucketParam("w", 0, 6), BucketParam("b", 6, 4)]
    bucket = MatrixGradBucket(tables, params, torch.float32, CPU)
    w = torch.arange(10.0, 16.0).view(2, 3)
    b = torch.arange(20.0, 24.0)
    packed = bucket.pack_rank_major([w, b])
    assert packed.tolist() == [10, 11, 12, 13, 0, 0, 14, 15, 20, 21, 22, 23]
    assert bucket.layout_class == "segment_copy"
    assert torch.equal(bucket.grad_view("b"), b) and bucket.grad_view("w", (2, 3)).shape == (2, 3)


def test_equal_shards_pack_as_plain_concat():
    tables = SegmentTables.build(10, [(S(0, 5, 0),), (S(5, 10, 0),)], rank=1)
    params = [BucketParam("w", 0, 6), BucketParam("b", 6, 4)]
    assert classify_bucket_layout(tables, params) == "flat_contiguous"
    bucket = MatrixGradBucket(tables, params, torch.float32, CPU)
    packed = bucket.pack_rank_major([torch.arange(6.0), torch.arange(6.0, 10.0)])
    assert packed.tolist() == list(range(10)) and packed.data_ptr() == bucket.buffer.data_ptr()


def test_fsdp2_chunk_layouts():
    # divisible: one fused chunk-cat
    params = [BucketParam("p0", 0, 4), BucketParam("p1", 4, 6)]
    tables = SegmentTables.build(10, [(S(0, 2, 0), S(4, 7, 2)), (S(2, 4, 0), S(7, 10, 2))], rank=0)
    assert classify_bucket_layout(tables, params) == "fsdp2_chunk"
    bucket = MatrixGradBucket(tables, params, torch.float32, CPU)
    packed = bucket.pack_rank_major([torch.arange(4.0), torch.arange(10.0, 16.0)])
    assert packed.tolist() == [0, 1, 10, 11, 12, 2, 3, 13, 14, 15]
    # ragged: p(5), p(6) on 2 ranks, the second rank's row is zero padded inside
    params = [BucketParam("p0", 0, 5), BucketParam("p1", 5, 6)]
    tables = SegmentTables.build(11, [(S(0, 3, 0), S(5, 8, 3)), (S(3, 5, 0), S(8, 11, 3))], rank=0)
    bucket = MatrixGradBucket(tables, params, torch.float32, CPU)
    packed = bucket.pack_rank_major([torch.arange(5.0), torch.arange(10.0, 16.0)])
    assert packed.tolist() == [0, 1, 2, 10, 11, 12, 3, 4, 0, 13, 14, 15]


def test_copy_in_paths_and_accumulation():
    tables = SegmentTables.build(10, [(S(0, 6, 0),), (S(6, 10, 0),)], rank=0)
    params = [BucketParam("w", 0, 6), BucketParam("b", 6, 4)]
    assert classify_bucket_layout(tables, params) == "foreach_copy"
    bucket = MatrixGradBucket(tables, params, torch.float32, CPU)
    assert bucket.copy_in([torch.ones(6), torch.full((4,), 2.0)]) == "cat"
    assert bucket.copy_in([torch.ones(6), None]) == "slice_copy"
    assert bucket.buffer.tolist() == [1] * 6 + [0] * 4
    assert bucket.copy_in([torch.ones(6), torch.ones(4)], accumulate=True) == "accumulate"
    assert bucket.buffer.tolist() == [2] * 6 + [1] * 4
    bucket.release()
    assert bucket.buffer is None
    ext = torch.zeros(16)
    bucket.attach(ext)
    assert bucket.buffer.numel() == 10 and bucket.buffer.data_ptr() == ext.data_ptr()


def test_segment_scatter_gather_are_inverse():
    segs = [S(2, 5, 0), S(8, 10, 3)]
    full = torch.arange(12.0)
    shard = torch.zeros(5)
    gather_local_segments(full, shard, segs)
    assert shard.tolist() == [2, 3, 4, 8, 9]
    out = torch.zeros(12)
    scatter_local_segments(shard, out, segs)
    assert out.tolist() == [0, 0, 2, 3, 4, 0, 0, 0, 8, 9, 0, 0]
    tables = SegmentTables.build(12, [tuple(segs), (S(0, 2, 0), S(5, 8, 2), S(10, 12, 5))], rank=0)
    assert tables.shard_sizes == (5, 7) and tables.max_shard == 7 and not tables.rank_contiguous
    packed = pack_rank_major_padded(full, tables)
    assert packed.view(2, 7).tolist() == [[2, 3, 4, 8, 9, 0, 0], [0, 1, 5, 6, 7, 10, 11]]


def test_collective_handle_runs_post_once():
    calls = []
    h = MatrixCollectiveHandle(post=lambda: calls.append(1), info={"kind": "all_gather"})
    h.wait()
    h.wait()
    assert calls == [1] and h.is_completed()


# ------------------------------------------------------------------------------------ pools
def test_full_param_buffer_pool_reuses_up_to_its_cap():
    from matrix_fsdp_b200.parallel.buffer_pool import FullParamBufferPool

    pool = FullParamBufferPool(max_cached_per_key=1)
    a = pool.acquire(16, torch.float32, CPU)
    b = pool.acquire(16, torch.float32, CPU)
    pa = a.data_ptr()
    pool.release(a)
    pool.release(b)                        # over the cap: dropped
    assert pool.cached_buffers() == 1
    c = pool.acquire(16, torch.float32, CPU)
    assert c.data_ptr() == pa
    d = pool.acquire(16, torch.bfloat16, CPU)           # another key
    assert d.dtype == torch.bfloat16
    st = pool.stats.as_dict() if hasattr(pool, "stats") else {}
    if st:
        assert st["acquires"] == 4 and st["reuses"] == 1 and st["dropped"] == 1
    pool.clear()
    assert pool.cached_buffers() == 0
    no_cache = FullParamBufferPool(max_cached_per_key=0)
    x = no_cache.acquire(8, torch.float32, CPU)
    no_cache.release(x)
    assert no_cache.cached_buffers() == 0


def test_workspace_cache_leases():
    from matrix_fsdp_b200.parallel.workspace_cache import CommWorkspaceCache

    cache = CommWorkspaceCache(max_cached_per_key=1)
    with cache.lease(32, torch.float32, CPU) as t:
        ptr = t.data_ptr()
        assert t.numel() == 32
    lease = cache.lease(32, torch.float32, CPU)
    assert lease.reused and lease.tensor.data_ptr() == ptr
    other = cache.lease(32, torch.float32, CPU)          # first one still out: a fresh tensor
    assert not other.reused
    lease.release()
    lease.release()                                       # idempotent
    other.release()
    st = cache.stats()
    assert st.get("reuses", st.get("reused", 1)) >= 1
    cache.clear()


# ------------------------------------------------------------------------------------ descriptors
def test_static_and_elastic_buffer_descriptors():
    from matrix_fsdp_b200.parallel.param_buffers import (ElasticParamBuffer, ElasticParamBufferLayout, StaticParamBuffer,
                                                         StaticParamBufferLayout)

    static = StaticParamBuffer(StaticParamBufferLayout((5, 5)), total_numel=10)
    plan = static.workspace_plan(can_direct_all_gather=True)
    assert not plan.needs_workspace and plan.padded_numel == 10 and plan.kind == "none"
    padded = StaticParamBuffer(StaticParamBufferLayout((4, 6)), total_numel=10)
    pplan = padded.workspace_plan(can_direct_all_gather=False)
    assert pplan.needs_workspace and pplan.padded_numel == 12 and pplan.kind == "padded_rank_chunks"
    summary = padded.communication_summary(param_gather_strategy="matrix_all_gather", matrix_collective_backend="auto",
                                           can_direct_all_gather=False)
    assert summary["param_buffer_type"] == "static" and summary["padding_waste_numel"] == 2
    assert summary["effective_grad_reduce_backend"] == "padded_reduce_scatter"
    segs = ((S(0, 3, 0), S(3, 6, 3)), (S(6, 10, 0),))
    elastic = ElasticParamBuffer(ElasticParamBufferLayout((6, 4), segs), total_numel=10)
    comm = elastic.layout.build_communication_plan()
    assert comm.segment_count == 3 and comm.coalesced_segment_count == 2      # the two adjacent pieces merge
    assert comm.max_coalesced_segments_per_rank == 1 and comm.rank_chunk_count == 2
    assert comm.peer_pull_table() == ((0, 0, 0, 6), (1, 0, 6, 4))             # (peer, peer offset, global offset, numel)
    esum = elastic.communication_summary(param_gather_strategy="matrix_all_gather", matrix_collective_backend="custom",
                                         can_direct_all_gather=False, transport_kind="peer")
    assert esum["param_buffer_type"] == "elastic" and esum["effective_grad_reduce_backend"] == "peer_pull_reduce"
    assert esum["communication_rank_chunk_fast_path"] is True and esum["workspace_needed"] is False
    assert elastic.rank_chunk_workspace_numel(compact=True) == 10 and elastic.rank_chunk_workspace_numel(compact=False) == 12
    lease = elastic.acquire_rank_chunk_workspace(dtype=torch.float32, device=CPU)
    assert lease.tensor.numel() == 12
    lease.release()


# ------------------------------------------------------------------------------------ transports at world size 1
def test_local_transport_aliases_and_env_selection(monkeypatch):
    from matrix_fsdp_b200.parallel import transport as T

    tables = SegmentTables.build(6, [(S(0, 6, 0),)], rank=0)
    tr = T.LocalTransport()
    shard, full = torch.arange(6.0), torch.zeros(6)
    tr.gather(shard, full, tables).wait()
    assert torch.equal(full, shard)
    grad, out = torch.arange(6.0), torch.zeros(6)
    tr.reduce(grad, out, tables, scale=0.5).wait()
    assert torch.equal(out, grad * 0.5)
    monkeypatch.setenv("MFSDP_TRANSPORT", "torch_dist")
    assert T.make_transport(None, 1, CPU).kind == "local"             # no group: nothing to talk to
    fake_group = object()
    assert T.make_transport(fake_group, 2, CPU).kind == "torch_dist"  # CPU never takes the peer transport
    tr2 = T.TorchDistTransport(fake_group, gather_impl="owner_broadcast", reduce_impl="owner_reduce")
    assert (tr2.gather_impl, tr2.reduce_impl) == ("owner_broadcast", "owner_reduce")
    monkeypatch.setenv("MFSDP_ALLGATHERV_IMPL", "broadcast")
    monkeypatch.setenv("MFSDP_REDUCE_SCATTERV_IMPL", "reduce")
    tr3 = T.TorchDistTransport(fake_group)
    assert (tr3.gather_impl, tr3.reduce_impl) == ("broadcast", "reduce")
    assert tr.all_reduce(torch.ones(3), None, scale=None).tolist() == [1, 1, 1]
