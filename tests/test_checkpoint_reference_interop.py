"""Checkpoints are interchangeable with the reference package: it loads what this package saves and this
package loads what it saves (same layout), and this package reshards what the reference saved.

The reference (installed under ``baseline/_ref``) patches ``torch.optim.Optimizer`` process-wide, so every
use of it runs in spawned ranks, never in the pytest process."""
import os
import sys
import tempfile

import pytest
import torch
from torch import nn


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "matrix_fsdp")),
                                reason="reference package is not installed under baseline/_ref")


def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(8, 12), nn.Tanh()), nn.Sequential(nn.Linear(12, 8, bias=False)))


def _batches(rank, n):
    g = torch.Generator().manual_seed(70 + rank)
    return [torch.randn(4, 8, generator=g) for _ in range(n)]


def _package(which):
    if which == "ref":
        if REF not in sys.path:
            sys.path.insert(0, REF)
        import matrix_fsdp as P
    else:
        import matrix_fsdp_b200 as P
    return P


def _build(which, world, kind):
    from torch.distributed.device_mesh import init_device_mesh

    P = _package(which)
    if which == "ours":
        from matrix_fsdp_b200.api import reset_shared_owner_planners

        reset_shared_owner_planners()
    mesh = init_device_mesh("cpu", (world,))
    policy = "mixed_muon_adamw" if kind == "mixed_muon_adamw" else None
    model = _model()
    for blk in model:
        P.fully_shard(blk, mesh=mesh, optimizer_policy=policy)
    opt = P.configure_optimizer(model, kind, lr=1e-2)
    return P, model, opt


def _dump(P, model, opt):
    """Everything a load has to restore, keyed without reference to either package's classes."""
    out = {"shards": [u.flat_buffer.local_shard.detach().clone() for u in P.collect_param_groups(model)], "opt": {}}
    names = {id(p): n for n, p in model.named_parameters()}
    comps = list(opt.iter_named_optimizers()) if hasattr(opt, "iter_named_optimizers") else \
        [("optimizer", getattr(opt, "optimizer", opt))]
    for comp, o in comps:
        for p, st in o.state.items():
            if p.numel() == 0 and not any(torch.is_tensor(v) and v.numel() > 1 for v in st.values()):
                continue
            for k, v in st.items():
                if torch.is_tensor(v):
                    out["opt"][f"{comp}/{names[id(p)]}/{k}"] = v.detach().clone().float().reshape(-1)
    return out


def _writer(rank, world, which, kind, d):
    P, model, opt = _build(which, world, kind)
    for x in _batches(rank, 2):
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    P.save_matrix_dcp(model, d, optimizer=opt)
    torch.save(_dump(P, model, opt), os.path.join(d, f"expect_rank{rank}.pt"))


def _reader(rank, world, which, kind, d, reshard_from):
    P, model, opt = _build(which, world, kind)
    P.load_matrix_dcp(model, d, optimizer=opt, allow_reshard=reshard_from is not None)
    got = _dump(P, model, opt)
    if reshard_from is None:
        want = torch.load(os.path.join(d, f"expect_rank{rank}.pt"))
        for a, b in zip(got["shards"], want["shards"]):
            assert torch.equal(a, b)
        tens = {k: v for k, v in want["opt"].items() if v.numel() > 1}
        assert tens, "the writer saved no optimizer tensors"
        for k, v in tens.items():
            assert k in got["opt"], (k, sorted(got["opt"]))
            assert torch.equal(got["opt"][k], v), k
        steps = {k: float(v) for k, v in want["opt"].items() if k.endswith("/step")}
        for k, v in steps.items():
            assert float(got["opt"][k]) == v, k
    else:
        # world 1 target: the single shard of every unit is the concatenation of the source shards
        pieces = [torch.load(os.path.join(d, f"expect_rank{r}.pt")) for r in range(reshard_from)]
        for i, a in enumerate(got["shards"]):
            assert torch.equal(a, torch.cat([p["shards"][i] for p in pieces]))
        for k, v in got["opt"].items():
            if v.numel() > 1:
                assert torch.equal(v, torch.cat([p["opt"][k] for p in pieces if k in p["opt"]])), k
    # and the loaded state trains on
    model(_batches(rank, 1)[0]).pow(2).mean().backward()
    opt.step()


def _write_then_read(rank, world, writer, reader, kind, base):
    d = os.path.join(base, f"{writer}-{reader}-{kind}-w{world}")
    if rank == 0:
        os.makedirs(d, exist_ok=True)
    if world > 1:
        torch.distributed.barrier()
    _writer(rank, world, writer, kind, d)
    if world > 1:
        torch.distributed.barrier()
    _reader(rank, world, reader, kind, d, None)


def _write_for_reshard(rank, world, base):
    d = os.path.join(base, "reshard-2-to-1")
    if rank == 0:
        os.makedirs(d, exist_ok=True)
    torch.distributed.barrier()
    _writer(rank, world, "ref", "adamw", d)


def _read_resharded(rank, world, base):
    _reader(rank, world, "ours", "adamw", os.path.join(base, "reshard-2-to-1"), 2)


_PAIRS = [("ref", "ours"), ("ours", "ref")]


@pytest.fixture(scope="module")
def outcomes():
    """Two spawns for the whole file: the two-rank cases first (one of them leaves the checkpoint that the
    one-rank job re-shards), then the one-rank cases.  Both packages are loaded into the same ranks."""
    from dist_utils import run_cases

    with tempfile.TemporaryDirectory() as base:
        two = [(f"adamw:{w}->{r}:2", _write_then_read, (w, r, "adamw", base)) for w, r in _PAIRS]
        two.append(("reshard:write", _write_for_reshard, (base,)))
        one = [(f"adamw:{w}->{r}:1", _write_then_read, (w, r, "adamw", base)) for w, r in _PAIRS]
        one += [(f"mixed:{w}->{r}", _write_then_read, (w, r, "mixed_muon_adamw", base)) for w, r in _PAIRS]
        one.append(("reshard:read", _read_resharded, (base,)))
        out = run_cases(2, two)
        out.update(run_cases(1, one))
        return out


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("writer,reader", _PAIRS)
def test_adamw_checkpoints_load_across_packages(outcomes, writer, reader, world):
    from dist_utils import check_case

    check_case(outcomes, f"adamw:{writer}->{reader}:{world}")


@pytest.mark.parametrize("writer,reader", _PAIRS)
def test_mixed_muon_checkpoints_load_across_packages(outcomes, writer, reader):
    from dist_utils import check_case

    check_case(outcomes, f"mixed:{writer}->{reader}")


def test_reference_checkpoint_reshards_from_two_ranks_to_one(outcomes):
    from dist_utils import check_case

    check_case(outcomes, "reshard:write")
    check_case(outcomes, "reshard:read")
