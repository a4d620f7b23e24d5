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

from dist_utils import run_ranks

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


@pytest.mark.parametrize("world", [1, 2])
@pytest.mark.parametrize("writer,reader", [("ref", "ours"), ("ours", "ref")])
def test_adamw_checkpoints_load_across_packages(writer, reader, world):
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_writer, world, writer, "adamw", d)
        run_ranks(_reader, world, reader, "adamw", d, None)


@pytest.mark.parametrize("writer,reader", [("ref", "ours"), ("ours", "ref")])
def test_mixed_muon_checkpoints_load_across_packages(writer, reader):
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_writer, 1, writer, "mixed_muon_adamw", d)
        run_ranks(_reader, 1, reader, "mixed_muon_adamw", d, None)


def test_reference_checkpoint_reshards_from_two_ranks_to_one():
    with tempfile.TemporaryDirectory() as d:
        run_ranks(_writer, 2, "ref", "adamw", d)
        run_ranks(_reader, 1, "ours", "adamw", d, 2)
