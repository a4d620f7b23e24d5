"""The library transport on three gloo ranks (an odd world size), one (layout, implementation, dtype) per case:
every gather implementation rebuilds the flat vector from the ranks' shards, every reduce implementation leaves
the scaled sum of the ranks' full gradients on the owner of each segment, and the per-parameter reduce does the
same parameter by parameter.  Layouts: equal chunks, uneven chunks, interleaved multi-segment shards, a rank that
owns nothing, a single owner, shards packed in a different order than the flat space.  All cases share one spawn.
The reference's counterpart is test/fsdp/test_collectives.py (17 tests)."""
import itertools
import json
import os
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks

WORLD = 3
LAYOUTS = ("equal", "uneven_chunks", "interleaved", "empty_rank", "single_owner", "reordered_local")
GATHERS = ("auto", "padded", "owner_broadcast", "uneven_all_gather", "all_reduce")
REDUCES = ("auto", "owner_reduce", "uneven_reduce_scatter", "per_param")
DTYPES = ("float32", "bfloat16")
GATHER_CASES = [f"gather-{l}-{g}-{d}" for l, g, d in itertools.product(LAYOUTS, GATHERS, DTYPES)]
REDUCE_CASES = [f"reduce-{l}-{r}-{d}" for l, r, d in itertools.product(LAYOUTS, REDUCES, DTYPES)]
CASES = GATHER_CASES + REDUCE_CASES + ["gather-equal-equal_all_gather-float32", "gather-uneven_chunks-equal_all_gather-float32"]


def _layout(name):
    """(total, per-rank [(global_start, global_end, local_start)]) for three ranks."""
    from matrix_fsdp_b200.core.layout import LayoutSegment as S

    spec = {
        "equal": (30, [[(0, 10, 0)], [(10, 20, 0)], [(20, 30, 0)]]),
        "uneven_chunks": (31, [[(0, 17, 0)], [(17, 20, 0)], [(20, 31, 0)]]),
        "interleaved": (37, [[(0, 5, 0), (20, 29, 5)], [(5, 12, 0), (29, 30, 7)], [(12, 20, 0), (30, 37, 8)]]),
        "empty_rank": (24, [[(0, 15, 0)], [], [(15, 24, 0)]]),
        "single_owner": (19, [[], [(0, 19, 0)], []]),
        "reordered_local": (26, [[(13, 20, 0), (0, 6, 7)], [(6, 13, 0)], [(23, 26, 0), (20, 23, 3)]]),
    }[name]
    return spec[0], [[S(*t) for t in segs] for segs in spec[1]]


def _param_ranges(total):
    cuts = sorted({0, total // 4, total // 2 + 1, total})
    return list(zip(cuts[:-1], cuts[1:]))


def _run_case(rank, world, name):
    from matrix_fsdp_b200.parallel import collectives as C
    from matrix_fsdp_b200.parallel.transport import TorchDistTransport

    kind, layout, impl, dtype_name = name.split("-")
    dtype = getattr(torch, dtype_name)
    total, segs = _layout(layout)
    tables = C.SegmentTables.build(total, segs, rank)
    assert tables.world_size == world and sum(tables.shard_sizes) == total
    group = dist.group.WORLD
    transport = TorchDistTransport(group)
    # small integers: exact in bf16, so every implementation has to agree bit for bit
    flat = (torch.arange(total) % 13 - 6).to(dtype)
    if kind == "gather":
        shard = torch.zeros(tables.shard_sizes[rank], dtype=dtype)
        C.gather_local_segments(flat, shard, tables.my_segments)
        full = torch.full((total,), 99, dtype=dtype)
        if impl == "equal_all_gather" and not tables.equal_contiguous:
            with pytest.raises(RuntimeError, match="equal"):
                transport.gather(shard, full, tables, impl=impl)
            return
        h = transport.gather(shard, full, tables, impl=impl)
        h.wait()
        assert torch.equal(full, flat), (full, flat)
        assert h.info["kind"] == "all_gather" and h.info["backend"] == "torch_dist"
        return
    full_grad = (flat.float() * (rank + 1)).to(dtype)                       # rank r contributes (r + 1) * flat
    expect_full = flat.float() * sum(range(1, world + 1)) * 0.5             # scale 0.5
    out = torch.full((tables.shard_sizes[rank],), 77, dtype=dtype)
    if impl == "per_param":
        h = C.reduce_scatter_per_param_async(full_grad, out, tables, _param_ranges(total), group, scale=0.5)
    else:
        h = transport.reduce(full_grad, out, tables, scale=0.5, impl=impl)
    h.wait()
    expect = torch.zeros(tables.shard_sizes[rank])
    C.gather_local_segments(expect_full, expect, tables.my_segments)
    assert torch.equal(out.float(), expect), (out, expect)
    assert h.info["kind"] == "reduce_scatter"


def _worker(rank, world, out_path):
    results = {}
    for name in CASES:
        try:
            _run_case(rank, world, name)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        gathered = [None] * world
        dist.all_gather_object(gathered, mine)
        results[name] = "\n".join(f"--- rank {r} ---\n{t}" for r, t in enumerate(gathered) if t)
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(results, f)


@pytest.fixture(scope="module")
def outcomes():
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, WORLD, path, timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.mark.parametrize("case", CASES)
def test_three_rank_library_collectives(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]
