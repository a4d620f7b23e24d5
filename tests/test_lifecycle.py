"""Single-process (world=1) lifecycle contract: states, event order, prefetch, no_sync, rejections."""
import copy
import inspect

import pytest
import torch
from torch import nn
from torch.distributed.fsdp import MixedPrecisionPolicy
from torch.distributed.tensor.placement_types import Shard

from matrix_fsdp_b200 import (DataParallelMeshDims, FSDPLifecycleState, configure_optimizer, fully_shard,
                              matrix_fully_shard, module_type_policy, summarize_param_groups)
from matrix_fsdp_b200.api import reset_shared_owner_planners


class Blk(nn.Module):
    def __init__(self, d=8):
        super().__init__()
        self.a = nn.Linear(d, 2 * d)
        self.b = nn.Linear(2 * d, d)

    def forward(self, x):
        return x + self.b(torch.relu(self.a(x)))


def _stack(n=3, d=8):
    torch.manual_seed(0)
    return nn.Sequential(*[Blk(d) for _ in range(n)])


def _names(unit):
    return [e.name for e in unit.runtime_events]


def test_fully_shard_signature_is_fsdp2_shaped():
    sig = inspect.signature(fully_shard)
    assert list(sig.parameters) == ["module", "mesh", "reshard_after_forward", "shard_placement_fn", "mp_policy",
                                    "offload_policy", "ignored_params", "dp_mesh_dims", "optimizer_policy"]
    assert all(p.kind is inspect.Parameter.KEYWORD_ONLY for n, p in sig.parameters.items() if n != "module")


def test_states_event_order_and_prefetch():
    model = _stack()
    for b in model:
        fully_shard(b)
    opt = configure_optimizer(model, "sgd", lr=0.1)
    units = [b._matrix_fsdp_param_group for b in model]
    out = model(torch.randn(2, 8))
    for u in units:
        assert u.state == FSDPLifecycleState.FORWARD_RESHARDED and u.full_param_storage_nbytes() == 0
    out.sum().backward()
    for u in units:
        assert u.state == FSDPLifecycleState.SHARDED and u.finalized_after_backward
    opt.step()
    assert all(u.flat_buffer.pending_reduce is None for u in units)
    ev = _names(units[1])
    order = [ev.index(n) for n in ("pre_forward", "unshard", "reshard_after_forward", "pre_backward_unshard",
                                   "finalize_backward")]
    assert order == sorted(order)
    # unit 1 was prefetched during unit 0's forward, and unit 0 during unit 1's backward
    assert ev.index("forward_prefetch") < ev.index("start_unshard:forward_prefetch") < ev.index("pre_forward")
    assert "backward_prefetch" in _names(units[0])
    assert any(e.name == "unshard" and e.prefetched for e in units[1].runtime_events)


def test_matches_eager_with_activation_checkpointing_and_unused_unit():
    from torch.utils.checkpoint import checkpoint

    model = _stack(3)
    ref = copy.deepcopy(model)
    for b in model:
        fully_shard(b)
    opt = configure_optimizer(model, "adamw", lr=1e-2)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2)
    for _ in range(2):
        x = torch.randn(4, 8)
        h = checkpoint(model[0], x, use_reentrant=False)
        h = checkpoint(model[1], h, use_reentrant=True)      # model[2] is never used
        h.pow(2).mean().backward()
        opt.step(); opt.zero_grad()
        ref[1](ref[0](x)).pow(2).mean().backward()
        ropt.step(); ropt.zero_grad()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n
    unused = model[2]._matrix_fsdp_param_group
    assert unused.state == FSDPLifecycleState.SHARDED and "pre_forward" not in _names(unused)
    assert any(e.recompute for e in model[0]._matrix_fsdp_param_group.runtime_events)


def test_multiple_forwards_need_no_reshard():
    m = Blk()
    fully_shard(m)
    m(torch.randn(2, 8))
    with pytest.raises(RuntimeError, match="another forward before"):
        m(torch.randn(2, 8))
    m2 = Blk()
    ref = copy.deepcopy(m2)
    fully_shard(m2, reshard_after_forward=False)
    x1, x2 = torch.randn(2, 8), torch.randn(2, 8)
    (m2(x1).sum() + m2(x2).sum()).backward()
    (ref(x1).sum() + ref(x2).sum()).backward()
    u = m2._matrix_fsdp_param_group
    u.prepare_for_optimizer_step()
    assert u.state == FSDPLifecycleState.SHARDED
    assert torch.allclose(m2.a.weight.grad, ref.a.weight.grad, atol=1e-6)


def test_nested_outputs_and_parallel_branches():
    class Multi(nn.Module):
        def __init__(self):
            super().__init__()
            self.l = nn.Linear(4, 4)

        def forward(self, x):
            y = self.l(x)
            return {"a": y, "b": (y * 2, [y + 1])}

    m = Multi()
    fully_shard(m)
    out = m(torch.randn(2, 4))
    out["b"][1][0].sum().backward()
    assert m._matrix_fsdp_param_group.state == FSDPLifecycleState.SHARDED
    branches = nn.ModuleList([nn.Linear(4, 4) for _ in range(3)])
    for b in branches:
        fully_shard(b)
    x = torch.randn(2, 4)
    sum(b(x).sum() for b in branches).backward()
    assert all(b._matrix_fsdp_param_group.state == FSDPLifecycleState.SHARDED for b in branches)


def test_no_sync_accumulates_then_reduces():
    m = Blk()
    ref = copy.deepcopy(m)
    fully_shard(m)
    opt = configure_optimizer(m, "sgd", lr=0.1)
    u = m._matrix_fsdp_param_group
    xs = [torch.randn(2, 8) for _ in range(2)]
    with m.no_sync():
        m(xs[0]).sum().backward()
        assert u.state == FSDPLifecycleState.SHARDED and u.has_accumulated_grads and u.defer_backward_reduce
        with pytest.raises(RuntimeError, match="no_sync"):
            opt.step()
        with pytest.raises(RuntimeError, match="no_sync"):
            opt.zero_grad()
    m(xs[1]).sum().backward()
    opt.step()
    assert not u.has_accumulated_grads
    for x in xs:
        ref(x).sum().backward()
    torch.optim.SGD(ref.parameters(), lr=0.1).step()
    assert torch.allclose(m.a.weight, ref.a.weight, atol=1e-6)


def test_mixed_precision_keeps_fp32_master_and_state():
    m = Blk()
    fully_shard(m, mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16, output_dtype=torch.float32))
    opt = configure_optimizer(m, "adamw", lr=1e-3)
    u = m._matrix_fsdp_param_group
    out = m(torch.randn(2, 8).bfloat16())
    assert out.dtype == torch.float32 and u.flat_buffer.full_buffer.dtype == torch.bfloat16
    out.sum().backward()
    opt.step()
    assert u.flat_buffer.local_shard.dtype == torch.float32 and m.a.weight.dtype == torch.float32
    assert all(st["exp_avg"].dtype == torch.float32 for st in opt.state.values() if "exp_avg" in st)


def test_rejections_and_policies():
    m = Blk()
    m.a.weight.requires_grad_(False)
    with pytest.raises(ValueError, match="require grad"):
        fully_shard(Blk().requires_grad_(False))
    fully_shard(m, ignored_params={m.a.weight})            # frozen params may be ignored
    tied = nn.Sequential(nn.Linear(4, 4, bias=False), nn.Linear(4, 4, bias=False))
    tied[1].weight = tied[0].weight
    with pytest.raises(NotImplementedError, match="shared parameters"):
        fully_shard(tied)
    with pytest.raises(ValueError, match="non-trivial divisor"):
        fully_shard(Blk(), reshard_after_forward=1)
    with pytest.raises(NotImplementedError):
        fully_shard(Blk(), reshard_after_forward=2)
    with pytest.raises(NotImplementedError):
        fully_shard(Blk(), shard_placement_fn=lambda p: Shard(1))
    with pytest.raises(NotImplementedError):
        fully_shard(Blk(), dp_mesh_dims=DataParallelMeshDims(shard=("a", "b")))
    with pytest.raises(ValueError, match="cannot be combined"):
        fully_shard(Blk(), optimizer_policy="muon", shard_placement_fn=lambda p: Shard(0))
    with pytest.raises(ValueError, match="Unknown fully_shard optimizer_policy"):
        fully_shard(Blk(), optimizer_policy="nope")


def test_planner_selection_from_policy_and_placement():
    reset_shared_owner_planners()
    m = Blk()
    fully_shard(m, optimizer_policy="mixed_muon_adamw")
    res = m._matrix_fsdp_param_group.planner_result
    assert (res.policy, res.name) == ("muon_shard_aware", "matrix_owner_tail_role_greedy")
    hints = {mp.fqn: mp.shard_hint for mp in m._matrix_fsdp_param_group.registry}
    assert (hints["a.weight"].optimizer_type, hints["a.weight"].split_granularity) == ("muon", "matrix_owner")
    assert (hints["a.bias"].optimizer_type, hints["a.bias"].split_granularity) == ("adamw", "parameter")
    lin = nn.Linear(4, 2)
    fully_shard(lin, shard_placement_fn=lambda p: Shard(0))
    u = lin._matrix_fsdp_param_group
    h = {mp.fqn: mp.shard_hint for mp in u.registry}
    assert (h["weight"].split_granularity, h["weight"].block_shape) == ("row_block", (1, 4))
    assert (h["bias"].split_granularity, h["bias"].block_shape) == ("block", (1,))
    assert u.runtime_mode == "matrix_shard"


def test_wrap_policy_and_plain_torch_optimizer_auto_prepare():
    from matrix_fsdp_b200 import install_matrix_optimizer_auto_prepare

    install_matrix_optimizer_auto_prepare()
    model = _stack(3)
    ref = copy.deepcopy(model)
    matrix_fully_shard(model, wrap_policy=module_type_policy(Blk), auto_shard_hints=True,
                       auto_planner_policy="muon_shard_aware", owner_assignment="scope_greedy")
    assert len(summarize_param_groups(model)) == 3
    opt = torch.optim.SGD(model.parameters(), lr=0.1)       # built after sharding: sees shard views
    x = torch.randn(2, 8)
    model(x).sum().backward()
    opt.step(); opt.zero_grad()
    ref(x).sum().backward()
    torch.optim.SGD(ref.parameters(), lr=0.1).step()
    for (n, p), (_, q) in zip(model.named_parameters(), ref.named_parameters()):
        assert torch.allclose(p, q, atol=1e-6), n
