"""Failure detection without touching a GPU: a rank that leaves or goes silent is noticed on the host
between steps; a collective whose peer never joins ends with an error after a short timeout; broken
checkpoint metadata and mismatched layouts are reported, not loaded."""
import datetime
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from matrix_fsdp_b200.utils.health import RankFailure, RankHealth


def _hb_worker(rank, world, path, result_dir):
    store = dist.FileStore(path, world)
    health = RankHealth(store, rank, world, timeout_s=1.0)
    outcome = "finished"
    deadline = time.time() + 60.0                      # start together: a rank that is still importing is not a failure
    while time.time() < deadline and any(rec is None for rec in health.peers().values()):
        time.sleep(0.05)
    try:
        for step in range(6):
            health.beat(step)
            if rank == 2 and step == 1:
                raise ValueError("injected host-side failure")     # dies without saying goodbye
            if rank == 1 and step == 3:
                health.leave("preempted")                           # orderly exit between steps
                outcome = "left"
                break
            time.sleep(0.4)
            if rank != 2:                                           # the rank that will crash only beats
                health.assert_alive()
    except RankFailure as exc:
        outcome = f"detected:{sorted(exc.missing)}:{exc.reason}"
        health.leave("stopped after a peer failure")
    except ValueError:
        outcome = "crashed"
    with open(os.path.join(result_dir, f"{rank}.txt"), "w") as f:
        f.write(outcome)


def test_heartbeat_detects_crashed_and_departed_ranks():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_hb_worker, args=(3, os.path.join(d, "store"), d), nprocs=3, join=True)
        out = {r: open(os.path.join(d, f"{r}.txt")).read() for r in range(3)}
    assert out[2] == "crashed"
    assert out[0].startswith("detected:")
    missing = out[0].split(":")[1]                      # "[2]", "[1]" or, on a loaded machine, "[1, 2]"
    assert "1" in missing or "2" in missing, out
    assert out[1] == "left" or out[1].startswith("detected:")


def _timeout_worker(rank, world, init_file, result_dir):
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world,
                            timeout=datetime.timedelta(seconds=3))
    outcome = "ok"
    if rank == 1:
        time.sleep(8)            # never joins the collective in time
        outcome = "late"
    else:
        try:
            dist.all_reduce(torch.ones(4))
        except Exception as exc:  # noqa: BLE001
            outcome = f"error:{type(exc).__name__}"
    with open(os.path.join(result_dir, f"{rank}.txt"), "w") as f:
        f.write(outcome)
    os._exit(0)                  # skip the (now broken) process-group teardown


def test_collective_with_absent_peer_times_out_with_an_error():
    with tempfile.TemporaryDirectory() as d:
        mp.spawn(_timeout_worker, args=(2, os.path.join(d, "rdzv"), d), nprocs=2, join=True)
        assert open(os.path.join(d, "0.txt")).read().startswith("error:")


def test_corrupt_or_missing_checkpoint_metadata_is_reported():
    from matrix_fsdp_b200 import fully_shard, load_matrix_dcp, save_matrix_dcp

    m = nn.Linear(4, 4)
    fully_shard(m)
    with tempfile.TemporaryDirectory() as d:
        with pytest.raises(FileNotFoundError):
            load_matrix_dcp(m, d, no_dist=True)
        save_matrix_dcp(m, d, no_dist=True)
        with open(os.path.join(d, "matrix_metadata.pt"), "wb") as f:
            f.write(b"not a checkpoint")
        with pytest.raises(Exception):
            load_matrix_dcp(m, d, no_dist=True)
        torch.save({"metadata": {"format": "something_else"}, "ranks": {}}, os.path.join(d, "matrix_metadata.pt"))
        with pytest.raises(ValueError, match="not a matrix_dcp metadata file"):
            load_matrix_dcp(m, d, no_dist=True)


def test_layout_signature_mismatch_is_detected(monkeypatch):
    from matrix_fsdp_b200.core.layout import LayoutSegment as S
    from matrix_fsdp_b200.parallel import collectives as Cc

    a = Cc.SegmentTables.build(10, [(S(0, 5, 0),), (S(5, 10, 0),)], 0)
    b = Cc.SegmentTables.build(10, [(S(0, 6, 0),), (S(6, 10, 0),)], 0)
    assert a.signature != b.signature
    monkeypatch.setenv(Cc.VALIDATE_SIGNATURE_ENV, "1")
    monkeypatch.setattr(Cc, "_world", lambda g: 2)
    sigs = iter([hash(a.signature), hash(b.signature)])

    def fake_all_gather_object(out, obj, group=None):
        out[0], out[1] = next(sigs), next(sigs)

    monkeypatch.setattr(Cc.dist, "all_gather_object", fake_all_gather_object)
    with pytest.raises(RuntimeError, match="signature differs"):
        Cc.validate_layout_signature(a, group=object())
