"""More multi-rank CPU (gloo) cases: a 3-D mesh whose tensor-parallel dim is left alone, mixed precision across
ranks, activation checkpointing across ranks, and the owner-broadcast / padded variants of the library transport."""
import copy
import os

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import check_case, run_cases


def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Sequential(nn.Linear(8, 12), nn.Tanh()), nn.Sequential(nn.Linear(12, 8), nn.Tanh()),
                         nn.Linear(8, 3))


def _allreduce_grads(model, group=None):
    world = dist.get_world_size(group)
    for p in model.parameters():
        dist.all_reduce(p.grad, group=group)
        p.grad.div_(world)


def _full_params(model):
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    units = collect_param_groups(model)
    for u in units:
        u.unshard("test")
    out = {n: p.detach().clone().float() for n, p in model.named_parameters()}
    for u in units:
        u.reshard("test")
    return out


def _mesh3d_worker(rank, world):
    """(dp_replicate=1, dp_shard=2, tp=2): shard over dp_shard only; ranks that differ in tp never talk."""
    from torch.distributed.device_mesh import init_device_mesh

    from matrix_fsdp_b200 import DataParallelMeshDims, configure_optimizer, fully_shard

    mesh = init_device_mesh("cpu", (1, 2, 2), mesh_dim_names=("dp_replicate", "dp_shard", "tp"))
    tp = rank % 2
    model = _model(seed=tp)                      # different weights per tp coordinate, like TP-local slices
    ref = copy.deepcopy(model)
    dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    for blk in list(model.children())[:-1]:
        fully_shard(blk, mesh=mesh, dp_mesh_dims=dims)
    fully_shard(model, mesh=mesh, dp_mesh_dims=dims)
    unit = model[0]._matrix_fsdp_param_group
    assert unit.world_size == 2 and unit.rank == rank // 2 and unit.replicate_world_size == 1
    opt = configure_optimizer(model, "adamw", lr=1e-2, weight_decay=0.0)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    shard_group = mesh.get_group("dp_shard")
    g = torch.Generator().manual_seed(10 + rank)
    for _ in range(2):
        x = torch.randn(4, 8, generator=g)
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        _allreduce_grads(ref, shard_group)
        ropt.step()
        ropt.zero_grad()
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=2e-5), n


def test_three_d_mesh_leaves_the_tp_dim_alone(four_rank_outcomes):
    check_case(four_rank_outcomes, "mesh3d")


def _mixed_precision_worker(rank, world):
    from torch.distributed.fsdp import MixedPrecisionPolicy

    from matrix_fsdp_b200 import configure_optimizer, fully_shard
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    model = _model()
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    root_mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, output_dtype=torch.float32)
    for blk in list(model.children())[:-1]:
        fully_shard(blk, mp_policy=mp)
    fully_shard(model, mp_policy=root_mp)                       # only the root casts the model output back
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(rank))
    out = model(x)
    assert out.dtype == torch.float32
    out.pow(2).mean().backward()
    for u in collect_param_groups(model):
        fb = u.flat_buffer
        assert fb.local_shard.dtype == torch.float32 and fb.param_dtype == torch.bfloat16
        assert fb.local_grad_shard is None or fb.local_grad_shard.dtype == torch.float32
    opt.step()
    opt.zero_grad()
    for st in opt.state.values():
        assert st["exp_avg"].dtype == torch.float32
    # both ranks hold shards of one consistent model
    full = _full_params(model)
    for n, t in full.items():
        ref = t.clone()
        dist.broadcast(ref, src=0)
        assert torch.equal(ref, t), n


def test_two_rank_mixed_precision_keeps_fp32_master(two_rank_outcomes):
    check_case(two_rank_outcomes, "mixed_precision")


def _checkpointing_worker(rank, world):
    from torch.utils.checkpoint import checkpoint

    from matrix_fsdp_b200 import configure_optimizer, fully_shard

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(0)
            self.blocks = nn.ModuleList([nn.Sequential(nn.Linear(8, 8), nn.Tanh()) for _ in range(3)])

        def forward(self, x, ckpt):
            for b in self.blocks:
                x = checkpoint(b, x, use_reentrant=False) if ckpt else b(x)
            return x

    model, ref = Net(), Net()
    for b in model.blocks:
        fully_shard(b)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
    g = torch.Generator().manual_seed(3 + rank)
    for _ in range(2):
        x = torch.randn(4, 8, generator=g)
        loss = model(x, True).pow(2).mean()
        loss.backward()
        opt.step()
        opt.zero_grad()
        rl = ref(x, False).pow(2).mean()
        rl.backward()
        _allreduce_grads(ref)
        ropt.step()
        ropt.zero_grad()
        assert torch.allclose(loss, rl, atol=1e-6)
    events = [e.name for e in model.blocks[0]._matrix_fsdp_param_group.runtime_events]
    assert "pre_forward_recompute_skip" in events or events.count("pre_forward") >= 2


def test_two_rank_activation_checkpointing(two_rank_outcomes):
    check_case(two_rank_outcomes, "checkpointing")


def _library_variants_worker(rank, world, gather_impl, reduce_impl):
    from matrix_fsdp_b200 import configure_optimizer, fully_shard
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    os.environ["MFSDP_ALLGATHERV_IMPL"] = gather_impl
    os.environ["MFSDP_REDUCE_SCATTERV_IMPL"] = reduce_impl
    reset_shared_owner_planners()
    model = _model()
    ref = copy.deepcopy(model)
    for blk in list(model.children())[:-1]:
        fully_shard(blk, optimizer_policy="mixed_muon_adamw")          # whole-matrix owners: uneven shards
    fully_shard(model, optimizer_policy="mixed_muon_adamw")
    unit = model[0]._matrix_fsdp_param_group
    assert unit.flat_buffer.transport.kind == "torch_dist"
    assert unit.flat_buffer.transport.gather_impl == gather_impl
    opt = configure_optimizer(model, "adamw", lr=1e-2, weight_decay=0.0)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.0)
    g = torch.Generator().manual_seed(20 + rank)
    for _ in range(2):
        x = torch.randn(4, 8, generator=g)
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        _allreduce_grads(ref)
        ropt.step()
        ropt.zero_grad()
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=2e-5), (gather_impl, reduce_impl, n)


_LIBRARY_VARIANTS = (("owner_broadcast", "owner_reduce"), ("padded_all_gather", "padded_reduce_scatter"), ("auto", "auto"))


@pytest.mark.parametrize("gather_impl,reduce_impl", _LIBRARY_VARIANTS)
def test_owner_layout_over_every_library_collective_variant(two_rank_outcomes, gather_impl, reduce_impl):
    check_case(two_rank_outcomes, f"library:{gather_impl}:{reduce_impl}")


def _clip_worker(rank, world):
    from matrix_fsdp_b200 import configure_optimizer, fully_shard
    from matrix_fsdp_b200.utils import clip_grad_norm_

    model = _model()
    ref = copy.deepcopy(model)
    for blk in list(model.children())[:-1]:
        fully_shard(blk)
    fully_shard(model)
    opt = configure_optimizer(model, "sgd", lr=0.5)
    ropt = torch.optim.SGD(ref.parameters(), lr=0.5)
    g = torch.Generator().manual_seed(40 + rank)
    for max_norm in (0.05, 1e6):                      # one step that clips, one that does not
        x = torch.randn(4, 8, generator=g) * 3
        model(x).pow(2).mean().backward()
        total = clip_grad_norm_(model, max_norm)
        opt.step()
        opt.zero_grad()
        ref(x).pow(2).mean().backward()
        _allreduce_grads(ref)
        rtotal = torch.nn.utils.clip_grad_norm_(ref.parameters(), max_norm)
        ropt.step()
        ropt.zero_grad()
        assert torch.allclose(total, rtotal, rtol=1e-5), (total, rtotal)
    full = _full_params(model)
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=1e-5), n


def test_two_rank_global_gradient_clipping(two_rank_outcomes):
    check_case(two_rank_outcomes, "clip")


# ----------------------------------------------------------------------------- unused unit keeps its shard
class _TwoBranch(nn.Module):
    def __init__(self, d=8):
        super().__init__()
        self.a = nn.Linear(d, d)
        self.b = nn.Linear(d, d)

    def forward(self, x, use_b=True):
        y = self.a(x)
        return self.b(y) if use_b else y


def _unused_unit_body(rank, world, opt_kind):
    from matrix_fsdp_b200.api import fully_shard
    from matrix_fsdp_b200.optim import configure_optimizer

    torch.manual_seed(0)
    model = _TwoBranch()
    fully_shard(model.a)
    fully_shard(model.b)
    kw = dict(lr=0.01) if opt_kind == "adamw" else dict(lr=0.01, momentum=0.9)
    opt = configure_optimizer(model, opt_kind, **kw)
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(rank))
    model(x).sum().backward()
    opt.step()
    opt.zero_grad()
    fb = model.b._matrix_fsdp_param_group.flat_buffer
    before = fb.local_shard.clone()
    a_before = model.a._matrix_fsdp_param_group.flat_buffer.local_shard.clone()
    # second step never runs b: it has no gradient, so its shard (and its moments) must not move
    model(x, use_b=False).sum().backward()
    opt.step()
    opt.zero_grad()
    assert torch.equal(fb.local_shard, before), "a unit without a gradient was updated with a stale one"
    assert not torch.equal(model.a._matrix_fsdp_param_group.flat_buffer.local_shard, a_before)


@pytest.mark.parametrize("opt_kind", ["adamw", "sgd"])
def test_unit_without_backward_is_skipped_by_the_flat_optimizer(two_rank_outcomes, opt_kind):
    check_case(two_rank_outcomes, f"unused_unit:{opt_kind}")


# ----------------------------------------------------------------------------- full optimizer state round trip
def _full_opt_roundtrip_body(rank, world, kind):
    from matrix_fsdp_b200 import get_optimizer_state_dict, set_optimizer_state_dict
    from matrix_fsdp_b200.api import fully_shard, reset_shared_owner_planners
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions
    from matrix_fsdp_b200.optim import configure_optimizer

    def build(seed):
        reset_shared_owner_planners()
        torch.manual_seed(seed)
        m = nn.Sequential(nn.Linear(8, 12), nn.Tanh(), nn.Linear(12, 8, bias=False))
        fully_shard(m, optimizer_policy="mixed_muon_adamw" if kind == "mixed_muon_adamw" else None)
        return m, configure_optimizer(m, kind, lr=1e-2)

    model, opt = build(0)
    g = torch.Generator().manual_seed(9 + rank)
    for _ in range(2):
        model(torch.randn(4, 8, generator=g)).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
    full_opts = MatrixStateDictOptions(full_state_dict=True)
    full = get_optimizer_state_dict(model, opt, options=full_opts)
    other, opt2 = build(0)
    set_optimizer_state_dict(other, opt2, full, options=full_opts)          # used to raise KeyError('params')
    again = get_optimizer_state_dict(other, opt2, options=full_opts)
    assert set(again) == set(full)
    for comp in full:
        assert set(again[comp]["state"]) == set(full[comp]["state"]), comp
        for name, entry in full[comp]["state"].items():
            for k, v in entry.items():
                w = again[comp]["state"][name][k]
                assert (torch.equal(v, w) if torch.is_tensor(v) else float(v) == float(w)), (comp, name, k)
    # the name-keyed form is recognised without the option, too
    other3, opt3 = build(0)
    set_optimizer_state_dict(other3, opt3, full)
    # several optimizers are keyed "0", "1", ...
    multi = get_optimizer_state_dict(model, [opt, opt], options=full_opts)
    assert set(multi) == {"0", "1"}


@pytest.mark.parametrize("kind", ["adamw", "mixed_muon_adamw"])
def test_full_optimizer_state_dict_loads_back(two_rank_outcomes, kind):
    check_case(two_rank_outcomes, f"full_opt:{kind}")


@pytest.fixture(scope="module")
def two_rank_outcomes():
    """Every two-rank case of this file in one spawn (see ``dist_utils.run_cases``)."""
    cases = [("mixed_precision", _mixed_precision_worker, ()), ("checkpointing", _checkpointing_worker, ()),
             ("clip", _clip_worker, ())]
    cases += [(f"library:{g}:{r}", _library_variants_worker, (g, r)) for g, r in _LIBRARY_VARIANTS]
    cases += [(f"unused_unit:{k}", _unused_unit_body, (k,)) for k in ("adamw", "sgd")]
    cases += [(f"full_opt:{k}", _full_opt_roundtrip_body, (k,)) for k in ("adamw", "mixed_muon_adamw")]
    return run_cases(2, cases)


@pytest.fixture(scope="module")
def four_rank_outcomes():
    return run_cases(4, [("mesh3d", _mesh3d_worker, ())])


def test_patched_load_state_dict_forwards_strict():
    from matrix_fsdp_b200 import fully_shard, patch_model_state_dict
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.checkpoint import MatrixStateDictOptions

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(4, 4), nn.Linear(4, 2))
    fully_shard(model)
    patch_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))
    sd = model.state_dict()
    partial = {k: v for k, v in sd.items() if not k.startswith("1.")}
    with pytest.raises(KeyError):
        model.load_state_dict(partial)
    model.load_state_dict(partial, strict=False)
