"""Host-side failure detection and recovery, no GPU involved.  Heartbeat rules one per test on an in-process
store; then the whole recovery path on gloo ranks: three ranks train and checkpoint, one leaves between steps,
the survivors notice it on the host before their next launch and stop, and a two-rank job resumes from the
three-rank checkpoint (re-sharded) and trains on."""
import os
import tempfile
import time

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks
from matrix_fsdp_b200.utils.health import RankFailure, RankHealth


def _store():
    return dist.HashStore()


# ------------------------------------------------------------------------------------------ heartbeat rules
def test_a_rank_announces_itself_when_its_health_object_is_made():
    store = _store()
    a = RankHealth(store, 0, 2)
    assert a.peers()[0][2] == "alive" and a.peers()[0][0] == -1 and a.peers()[1] is None


def test_all_ranks_beating_means_alive():
    store = _store()
    a, b = RankHealth(store, 0, 2, timeout_s=5.0), RankHealth(store, 1, 2, timeout_s=5.0)
    a.beat(3)
    b.beat(3)
    a.assert_alive()
    b.assert_alive(min_step=3)
    assert a.peers()[1][0] == 3


def test_a_rank_that_never_showed_up_is_reported_as_silent():
    a = RankHealth(_store(), 0, 3, timeout_s=0.5)
    with pytest.raises(RankFailure) as exc:
        a.assert_alive()
    assert exc.value.missing == [1, 2] and "no heartbeat" in exc.value.reason


def test_an_orderly_exit_is_reported_as_left_with_its_rank():
    store = _store()
    a, b = RankHealth(store, 0, 2), RankHealth(store, 1, 2)
    b.leave("preempted")
    with pytest.raises(RankFailure) as exc:
        a.assert_alive()
    assert exc.value.missing == [1] and exc.value.reason == "left the job"
    assert a.peers()[1][2] == "preempted"


def test_a_stale_heartbeat_counts_as_silence():
    store = _store()
    a, b = RankHealth(store, 0, 2, timeout_s=0.2), RankHealth(store, 1, 2, timeout_s=0.2)
    b.beat(0)
    a.assert_alive()
    time.sleep(0.3)
    with pytest.raises(RankFailure) as exc:
        a.assert_alive()
    assert exc.value.missing == [1]
    b.beat(1)                                             # it was only slow: the next beat clears it
    a.assert_alive()


def test_departures_are_reported_before_silences():
    store = _store()
    a, b = RankHealth(store, 0, 3, timeout_s=0.5), RankHealth(store, 1, 3, timeout_s=0.5)
    b.leave()
    with pytest.raises(RankFailure) as exc:             # rank 2 never showed up, rank 1 left: the departure is named
        a.assert_alive()
    assert exc.value.missing == [1] and exc.value.reason == "left the job"


def test_a_rank_does_not_judge_itself():
    a = RankHealth(_store(), 0, 1, timeout_s=0.01)
    time.sleep(0.05)
    a.assert_alive()


def test_jobs_with_different_prefixes_do_not_see_each_other():
    store = _store()
    a = RankHealth(store, 0, 2, prefix="job_a")
    RankHealth(store, 1, 2, prefix="job_b")
    assert a.peers()[1] is None


def test_rank_failure_is_a_runtime_error_that_names_the_ranks():
    err = RankFailure([2, 5], "left the job")
    assert isinstance(err, RuntimeError) and "[2, 5]" in str(err) and err.missing == [2, 5]


# ------------------------------------------------------------------------------------------ recovery path
def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(6, 12), nn.Tanh()), nn.Linear(12, 6))


def _build(seed=0):
    from matrix_fsdp_b200 import configure_optimizer, fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    model = _model(seed)
    fully_shard(model[0])
    fully_shard(model)
    return model, configure_optimizer(model, "adamw", lr=1e-2)


def _step(model, opt, index):
    x = torch.randn(4, 6, generator=torch.Generator().manual_seed(900 + index))      # same batch on every rank
    model(x).pow(2).mean().backward()
    opt.step()
    opt.zero_grad()


def _full(model):
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions, get_model_state_dict

    return get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))


def _first_job(rank, world, directory):
    """Three ranks; rank 2 is preempted after step 1 (between steps, nothing in flight)."""
    from matrix_fsdp_b200 import save_matrix_dcp

    health = RankHealth(dist.FileStore(os.path.join(directory, "hb"), world), rank, world, timeout_s=20.0)
    model, opt = _build()
    outcome = "finished"
    try:
        for step in range(4):
            health.assert_alive()                          # before every launch
            _step(model, opt, step)
            if step == 1:
                save_matrix_dcp(model, os.path.join(directory, "ckpt"), optimizer=opt)
                full = _full(model)
                if rank == 0:
                    torch.save(full, os.path.join(directory, "saved_full.pt"))
                dist.barrier()
                if rank == 2:
                    health.leave("preempted")
                    outcome = "left"
                    break
                # give the notice time to land: the survivors must not enter step 2's collectives
                deadline = time.time() + 10.0
                while time.time() < deadline and health.peers()[2][2] == "alive":
                    time.sleep(0.05)
            health.beat(step)
    except RankFailure as exc:
        outcome = f"stopped:{exc.missing}:{exc.reason}"
        health.leave("stopped after a peer failure")
    with open(os.path.join(directory, f"first_{rank}.txt"), "w") as f:
        f.write(outcome)


def _second_job(rank, world, directory):
    """Two ranks resume from the three-rank checkpoint."""
    from matrix_fsdp_b200 import load_matrix_dcp

    model, opt = _build(seed=9)
    with pytest.raises(ValueError):
        load_matrix_dcp(model, os.path.join(directory, "ckpt"), optimizer=opt)          # another world size: ask for it
    load_matrix_dcp(model, os.path.join(directory, "ckpt"), optimizer=opt, allow_reshard=True)
    saved = torch.load(os.path.join(directory, "saved_full.pt"))
    got = _full(model)
    for k, v in saved.items():
        assert torch.equal(got[k], v), k
    _step(model, opt, 2)
    after = _full(model)
    assert any(not torch.equal(after[k], saved[k]) for k in saved)
    if rank == 0:
        torch.save(after, os.path.join(directory, "resumed_after.pt"))


def _uninterrupted(rank, world, directory):
    """What three ranks would have reached at step 2 had nobody left (same batches on every rank)."""
    model, opt = _build()
    for step in range(3):
        _step(model, opt, step)
    full = _full(model)
    if rank == 0:
        torch.save(full, os.path.join(directory, "uninterrupted_after.pt"))


def test_survivors_stop_between_steps_and_a_smaller_job_resumes_from_the_checkpoint():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_first_job, 3, d)
        out = {r: open(os.path.join(d, f"first_{r}.txt")).read() for r in range(3)}
        assert out[2] == "left"
        for r in (0, 1):         # a survivor may also see the other survivor's "stopped" notice; rank 2 is always named
            assert out[r].startswith("stopped:[") and out[r].endswith(":left the job") and "2]" in out[r], out
        run_ranks(_second_job, 2, d)
        run_ranks(_uninterrupted, 3, d)
        resumed = torch.load(os.path.join(d, "resumed_after.pt"))
        straight = torch.load(os.path.join(d, "uninterrupted_after.pt"))
        for k, v in straight.items():                      # same batches, so losing a rank changed nothing in the maths
            assert torch.allclose(resumed[k], v, atol=2e-6), k
