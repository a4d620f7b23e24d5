"""Two gloo ranks, one option per case: two training steps of the sharded model equal the eager model whose
gradients are averaged over the ranks, and every unit ends sharded with no full-parameter storage.

All cases of one world size run inside ONE spawn (the rendezvous and the imports are the expensive part); each
case records its own outcome and is reported as its own test.  The reference keeps one test per option in
test/fsdp/test_matrix_fsdp_distributed.py:2624-3121."""
import copy
import json
import os
import tempfile
import traceback
from collections import OrderedDict

import pytest
import torch
import torch.distributed as dist
from torch import nn

from dist_utils import run_ranks


class Blk(nn.Module):
    def __init__(self, d):
        super().__init__()
        self.a = nn.Linear(d, 2 * d)
        self.n = nn.LayerNorm(2 * d)
        self.b = nn.Linear(2 * d, d, bias=False)

    def forward(self, x):
        return x + self.b(torch.relu(self.n(self.a(x))))


class CkptBlk(Blk):
    def forward(self, x):
        from torch.utils.checkpoint import checkpoint

        return checkpoint(super().forward, x, use_reentrant=False)


def _model(block=Blk, d=8, n=3):
    torch.manual_seed(0)
    m = nn.Sequential(*[block(d) for _ in range(n)])
    m.add_module("head", nn.Linear(d, d))
    return m


def _bf16():
    from torch.distributed.fsdp import MixedPrecisionPolicy

    return MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)


def _rows(param):
    from torch.distributed.tensor.placement_types import Shard

    return Shard(0)


def _bf16_everywhere():
    from torch.distributed.fsdp import MixedPrecisionPolicy

    return MixedPrecisionPolicy(param_dtype=torch.bfloat16)           # gradients are reduced in bf16 as well


def _bf16_out_fp32():
    from torch.distributed.fsdp import MixedPrecisionPolicy

    return MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, output_dtype=torch.float32)


def _planner(name):
    from matrix_fsdp_b200.planning import planner as P

    return getattr(P, name)


# name -> (wrap, shard kwargs factory, optimizer, options)
#   wrap: "root" one unit | "units" one unit per block + root | "policy" wrap_policy over blocks + root
CASES = {
    "root_default": ("root", lambda: {}, "adamw", {}),
    "units_default": ("units", lambda: {}, "adamw", {}),
    "policy_default": ("policy", lambda: {}, "adamw", {}),
    "root_keep_after_forward": ("root", lambda: dict(reshard_after_forward=False), "adamw", {}),
    "units_keep_after_forward": ("units", lambda: dict(reshard_after_forward=False), "adamw", {}),
    "policy_keep_after_forward": ("policy", lambda: dict(reshard_after_forward=False), "adamw", {}),
    "root_finalize_at_end_of_backward": ("root", lambda: dict(finalize_after_backward=False), "adamw", {}),
    "units_finalize_at_end_of_backward": ("units", lambda: dict(finalize_after_backward=False), "adamw", {}),
    "policy_finalize_at_end_of_backward": ("policy", lambda: dict(finalize_after_backward=False), "adamw", {}),
    "units_no_forward_prefetch": ("units", lambda: dict(forward_prefetch=False), "adamw", {}),
    "units_no_backward_prefetch": ("units", lambda: dict(backward_prefetch=False), "adamw", {}),
    "policy_no_prefetch_at_all": ("policy", lambda: dict(forward_prefetch=False, backward_prefetch=False), "sgd", {}),
    "units_reduce_flat": ("units", lambda: dict(backward_reduce_strategy="flat"), "adamw", {}),
    "units_reduce_per_param": ("units", lambda: dict(backward_reduce_strategy="per_param"), "adamw", {}),
    "units_reduce_per_param_allreduce": ("units", lambda: dict(backward_reduce_strategy="per_param_allreduce"), "adamw", {}),
    "units_grad_reduce_alias": ("units", lambda: dict(grad_reduce_strategy="bucket_reduce_scatter"), "sgd", {}),
    "units_fsdp2_chunks": ("units", lambda: dict(group_planner=_planner("fsdp2_chunk_plan")), "adamw", {}),
    "units_parameter_boundaries": ("units", lambda: dict(group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_ordered_groups": ("units", lambda: dict(group_planner=_planner("ordered_group_plan")), "adamw", {}),
    "units_owner_tail": ("units", lambda: dict(group_planner=_planner("ordered_matrix_owner_tail_plan"),
                                               auto_shard_hints=True), "adamw", {}),
    "units_plain_planner": ("units", lambda: dict(planner=_planner("contiguous_even_plan")), "adamw", {}),
    "units_layout_planner": ("units", lambda: dict(layout_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_auto_hints_only": ("units", lambda: dict(auto_shard_hints=True), "adamw", {}),
    "units_auto_max_balance": ("units", lambda: dict(auto_planner_policy="max_balance"), "adamw", {}),
    "units_auto_debug": ("units", lambda: dict(auto_planner_policy="debug"), "sgd", {}),
    "units_auto_block_units": ("units", lambda: dict(auto_planner_policy="balanced", target_block_units=16), "adamw", {}),
    "units_auto_muon_zero_copy": ("units", lambda: dict(auto_planner_policy="muon_zero_copy", auto_shard_hints=True),
                                  "adamw", {}),
    "units_auto_muon_shard_aware_round_robin": ("units", lambda: dict(auto_planner_policy="muon_shard_aware",
                                                                      auto_shard_hints=True,
                                                                      rotation_strategy="round_robin"), "sgd", {}),
    "units_auto_muon_full_matrix": ("units", lambda: dict(auto_planner_policy="muon_full_matrix", auto_shard_hints=True),
                                    "sgd", {}),
    "units_auto_balanced": ("units", lambda: dict(auto_planner_policy="balanced"), "adamw", {}),
    "units_auto_zero_copy_friendly": ("units", lambda: dict(auto_planner_policy="zero_copy_friendly"), "adamw", {}),
    "units_auto_min_comm": ("units", lambda: dict(auto_planner_policy="min_comm"), "sgd", {}),
    "units_gather_equal": ("units", lambda: dict(param_gather_strategy="equal_all_gather"), "adamw", {}),
    "units_gather_uneven": ("units", lambda: dict(param_gather_strategy="uneven_all_gather",
                                                  group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_gather_padded": ("units", lambda: dict(param_gather_strategy="matrix_all_gather",
                                                  group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_gather_owner_broadcast": ("units", lambda: dict(param_gather_strategy="owner_broadcast",
                                                           group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_gather_all_reduce": ("units", lambda: dict(param_gather_strategy="all_reduce",
                                                      group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_backend_torch": ("units", lambda: dict(matrix_collective_backend="torch",
                                                  group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_layout_segment_runtime": ("units", lambda: dict(runtime_layout_policy="segment_runtime",
                                                           group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_layout_flat_reorder": ("units", lambda: dict(runtime_layout_policy="flat_reorder",
                                                        group_planner=_planner("parameter_boundary_plan")), "adamw", {}),
    "units_layout_matrix_shard": ("units", lambda: dict(runtime_layout_policy="matrix_shard"), "adamw", {}),
    "root_layout_flat_reorder_sgd": ("root", lambda: dict(runtime_layout_policy="flat_reorder",
                                                           group_planner=_planner("parameter_boundary_plan")), "sgd", {}),
    "units_rows": ("units", lambda: dict(shard_placement_fn=_rows), "adamw", {}),
    "root_rows": ("root", lambda: dict(shard_placement_fn=_rows), "sgd", {}),
    "units_zero_copy_bucket": ("units", lambda: dict(use_zero_copy_grad_bucket=True), "adamw", {}),
    "units_saved_tensor_hooks": ("units", lambda: dict(use_saved_tensor_hooks=True), "adamw", {}),
    "units_keep_storage_after_backward": ("units", lambda: dict(shrink_full_param_storage_after_backward=False),
                                          "adamw", {"storage_may_stay": True}),
    "units_sum_not_mean": ("units", lambda: dict(divide_grads_by_world=False), "sgd", {"sum": True}),
    "root_bf16": ("root", lambda: dict(mp_policy=_bf16()), "adamw", {"bf16": True}),
    "units_bf16": ("units", lambda: dict(mp_policy=_bf16()), "adamw", {"bf16": True}),
    "units_bf16_flat_reduce": ("units", lambda: dict(mp_policy=_bf16(), backward_reduce_strategy="flat"), "adamw",
                               {"bf16": True}),
    "units_bf16_reduce_in_bf16": ("units", lambda: dict(mp_policy=_bf16_everywhere()), "adamw", {"bf16": True}),
    "units_bf16_reduce_in_bf16_owner_layout": ("units", lambda: dict(mp_policy=_bf16_everywhere(),
                                                                     group_planner=_planner("parameter_boundary_plan")),
                                               "sgd", {"bf16": True}),
    # (one unit: inside a stack every unit would hand fp32 to a sibling whose inputs nobody casts)
    "root_bf16_fp32_outputs": ("root", lambda: dict(mp_policy=_bf16_out_fp32()), "adamw", {"bf16": True}),
    "units_bf16_zero_copy_bucket": ("units", lambda: dict(mp_policy=_bf16_everywhere(), use_zero_copy_grad_bucket=True),
                                    "adamw", {"bf16": True}),
    "units_bf16_wrapped_torch_adam": ("units", lambda: dict(mp_policy=_bf16()), "torch:Adam",
                                      {"torch_kw": dict(lr=1e-2), "bf16": True}),
    "units_replicate_only_mesh": ("units", lambda: {}, "adamw", {"mesh": "replicate_only"}),
    "units_replicate_only_mesh_no_sync": ("units", lambda: {}, "sgd", {"mesh": "replicate_only", "no_sync": True}),
    "units_replicate_only_mesh_bf16": ("units", lambda: dict(mp_policy=_bf16()), "adamw", {"mesh": "replicate_only", "bf16": True}),
    "units_one_d_named_mesh": ("units", lambda: {}, "adamw", {"mesh": "one_d_named"}),
    "root_no_sync": ("root", lambda: {}, "sgd", {"no_sync": True}),
    "units_no_sync": ("units", lambda: {}, "sgd", {"no_sync": True}),
    "units_no_sync_keep_after_forward": ("units", lambda: dict(reshard_after_forward=False), "sgd", {"no_sync": True}),
    "units_no_sync_flat_reduce": ("units", lambda: dict(backward_reduce_strategy="flat"), "sgd", {"no_sync": True}),
    "units_bf16_no_sync": ("units", lambda: dict(mp_policy=_bf16()), "sgd", {"no_sync": True, "bf16": True}),
    "root_activation_checkpoint": ("root", lambda: {}, "adamw", {"ckpt": True}),
    "units_activation_checkpoint": ("units", lambda: {}, "adamw", {"ckpt": True}),
    "units_sched_two_ahead": ("units", lambda: {}, "adamw", {"opt_kw": dict(max_unsharded_prefetch_units=2)}),
    "units_sched_post_reshard_prefetch": ("units", lambda: {}, "adamw",
                                          {"opt_kw": dict(backward_prefetch_timing="post_reshard")}),
    "units_sched_one_active_buffer": ("units", lambda: {}, "adamw", {"opt_kw": dict(max_active_full_param_buffers=1)}),
    "units_sched_two_pending_reduces": ("units", lambda: {}, "adamw", {"opt_kw": dict(max_pending_backward_reduces=2)}),
    # two backward passes over one kept graph (two losses on one forward)
    "root_two_losses": ("root", lambda: {}, "adamw", {"two_losses": True}),
    "units_two_losses": ("units", lambda: {}, "adamw", {"two_losses": True}),
    "policy_two_losses_keep_after_forward": ("policy", lambda: dict(reshard_after_forward=False), "sgd", {"two_losses": True}),
    "units_two_losses_zero_copy_bucket": ("units", lambda: dict(use_zero_copy_grad_bucket=True), "adamw", {"two_losses": True}),
    "units_two_losses_flat_reduce": ("units", lambda: dict(backward_reduce_strategy="flat"), "sgd", {"two_losses": True}),
    "units_two_losses_owner_layout": ("units", lambda: dict(group_planner=_planner("parameter_boundary_plan")), "adamw",
                                      {"two_losses": True}),
    "units_two_losses_bf16": ("units", lambda: dict(mp_policy=_bf16()), "adamw", {"two_losses": True, "bf16": True}),
    "units_two_losses_no_sync": ("units", lambda: {}, "sgd", {"two_losses": True, "no_sync": True}),
    "units_two_losses_activation_checkpoint": ("units", lambda: {}, "adamw", {"two_losses": True, "ckpt": True}),
    # any element-wise torch optimizer, built by the user over model.parameters() and wrapped
    "wrapped_torch_adamw_amsgrad": ("units", lambda: {}, "torch:AdamW", {"torch_kw": dict(lr=1e-2, amsgrad=True)}),
    "wrapped_torch_adam": ("units", lambda: {}, "torch:Adam", {"torch_kw": dict(lr=1e-2)}),
    "wrapped_torch_sgd_nesterov": ("units", lambda: {}, "torch:SGD", {"torch_kw": dict(lr=0.05, momentum=0.9, nesterov=True)}),
    "wrapped_torch_rmsprop": ("root", lambda: {}, "torch:RMSprop", {"torch_kw": dict(lr=1e-3)}),
    "wrapped_torch_adagrad_owner_layout": ("units", lambda: dict(group_planner=_planner("parameter_boundary_plan")),
                                           "torch:Adagrad", {"torch_kw": dict(lr=1e-2)}),
    # the same without the wrapper: the optimizer hooks installed by the package run the lifecycle
    "bare_torch_adamw": ("units", lambda: {}, "bare:AdamW", {"torch_kw": dict(lr=1e-2, weight_decay=0.0)}),
    "bare_torch_sgd_bf16": ("units", lambda: dict(mp_policy=_bf16()), "bare:SGD", {"torch_kw": dict(lr=0.05), "bf16": True}),
}


# how the units are called: name -> (forward function over the block stack, shard keywords)
def _chain(m, x):
    for blk in m.children():
        x = blk(x)
    return x


def _twice(m, x):
    return _chain(m, x) + _chain(m, x * 0.5)                    # every unit runs twice before one backward


def _branches(m, x):
    return m[0](x) + m[1](x) + m[2](x) + m.head(x)              # units side by side, not in a chain


def _shared_block(m, x):
    return m.head(m[1](m[0](m[1](x))))                          # one unit used at two depths, one unit never used


def _partial_output(m, x):
    y = _chain(m, x)
    return y[:, :4]                                             # only a slice of the output reaches the loss


def _checkpointed_chain(m, x):
    from torch.utils.checkpoint import checkpoint

    x = x.clone().requires_grad_(True)
    for blk in list(m.children()):
        x = checkpoint(blk, x, use_reentrant=False)
    return x


def _reentrant_checkpointed_chain(m, x):
    from torch.utils.checkpoint import checkpoint

    x = x.clone().requires_grad_(True)
    for blk in list(m.children()):
        x = checkpoint(blk, x, use_reentrant=True)
    return x


def _detached_prefix(m, x):
    with torch.no_grad():
        h = m[0](x)                                             # this unit gets no gradient in this step
    return m.head(m[2](m[1](h)))


_ORDERS = ([0, 1, 2], [2, 1, 0], [0, 2], [1], [2, 0], [0, 1, 2])


def _changing_order(m, x):
    """Another order (and another subset) of the blocks at every call: what the scheduler learnt from the last
    iteration is wrong for this one, prefetched units may go unused."""
    calls = getattr(m, "_calls", 0)
    m._calls = calls + 1
    for j in _ORDERS[calls % len(_ORDERS)]:
        x = m[j](x)
    return m.head(x)


TOPOLOGIES = {
    "topo_twice_keep": (_twice, dict(reshard_after_forward=False)),
    "topo_branches": (_branches, {}),
    "topo_branches_no_prefetch": (_branches, dict(forward_prefetch=False, backward_prefetch=False)),
    "topo_shared_block_keep": (_shared_block, dict(reshard_after_forward=False)),
    "topo_partial_output": (_partial_output, {}),
    "topo_checkpointed_chain": (_checkpointed_chain, {}),
    "topo_reentrant_checkpointed_chain": (_reentrant_checkpointed_chain, {}),
    "topo_detached_prefix": (_detached_prefix, {}),
    "topo_detached_prefix_keep": (_detached_prefix, dict(reshard_after_forward=False)),
    "topo_changing_order": (_changing_order, {}),
    "topo_changing_order_keep": (_changing_order, dict(reshard_after_forward=False)),
    "topo_changing_order_no_prefetch": (_changing_order, dict(forward_prefetch=False, backward_prefetch=False)),
}
CASES.update({name: ("units", (lambda kw=kw: dict(kw)), "adamw", {"fn": fn}) for name, (fn, kw) in TOPOLOGIES.items()})
for _name, _opt_kw in {"three_ahead": dict(max_unsharded_prefetch_units=3), "one_buffer": dict(max_active_full_param_buffers=1),
                       "post_reshard": dict(backward_prefetch_timing="post_reshard", max_unsharded_prefetch_units=2),
                       "adaptive": dict(prefetch_policy="adaptive", adaptive_wait_threshold_ms=0.0),
                       "next_step_prefetch": dict(prefetch_first_unit_after_step=True, next_step_prefetch_units=2)}.items():
    CASES[f"topo_changing_order_{_name}"] = ("units", lambda: {}, "adamw", {"fn": _changing_order, "opt_kw": _opt_kw})


class TopoNet(nn.Sequential):
    """The block stack with a forward of its own choosing: the root has to stay the entry point (its hooks gather
    the parameters the root unit owns, here the head), so the call pattern lives inside its forward."""
    pattern = None

    def forward(self, x):
        return self.pattern(self, x) if self.pattern is not None else super().forward(x)


# four ranks as a 2 x 2 mesh: shards inside a replica, replicas average the reduced shards
HSDP_CASES = {
    "hsdp_units_default": ("units", lambda: {}, "adamw", {}),
    "hsdp_root_default": ("root", lambda: {}, "adamw", {}),
    "hsdp_policy_default": ("policy", lambda: {}, "sgd", {}),
    "hsdp_units_keep_after_forward": ("units", lambda: dict(reshard_after_forward=False), "adamw", {}),
    "hsdp_units_reduce_flat": ("units", lambda: dict(backward_reduce_strategy="flat"), "adamw", {}),
    "hsdp_units_reduce_per_param": ("units", lambda: dict(backward_reduce_strategy="per_param"), "adamw", {}),
    "hsdp_units_parameter_boundaries": ("units", lambda: dict(group_planner=_planner("parameter_boundary_plan")),
                                        "adamw", {}),
    "hsdp_units_bf16": ("units", lambda: dict(mp_policy=_bf16()), "adamw", {"bf16": True}),
    "hsdp_units_no_sync": ("units", lambda: {}, "sgd", {"no_sync": True}),
    "hsdp_units_activation_checkpoint": ("units", lambda: {}, "adamw", {"ckpt": True}),
    "hsdp_units_zero_copy_bucket": ("units", lambda: dict(use_zero_copy_grad_bucket=True), "adamw", {}),
    "hsdp_units_two_losses": ("units", lambda: {}, "adamw", {"two_losses": True}),
}


def _shard(model, wrap, kw):
    from matrix_fsdp_b200 import fully_shard, matrix_fully_shard
    from matrix_fsdp_b200.policy.wrap import module_type_policy

    if "shard_placement_fn" in kw:                              # an option of the FSDP2-shaped entry point only
        for m in ([] if wrap == "root" else list(model.children())[:-1]) + [model]:
            fully_shard(m, **kw)
        return

    if wrap == "units":
        for blk in list(model.children())[:-1]:
            matrix_fully_shard(blk, **kw)
    elif wrap == "policy":
        matrix_fully_shard(model, wrap_policy=module_type_policy(Blk), **kw)
    matrix_fully_shard(model, **kw)          # the root unit: everything no block claimed (all of it for "root")


_MESH = {}


def _hsdp_mesh(world):
    if world not in _MESH:                    # one mesh (one set of process groups) for all cases of the spawn
        from torch.distributed.device_mesh import init_device_mesh

        _MESH[world] = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    return _MESH[world]


def _full_params(model):
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    units = collect_param_groups(model)
    for u in units:
        u.unshard("test")
    out = {n: p.detach().clone().float() for n, p in model.named_parameters()}
    for u in units:
        u.reshard("test")
    return out


def _run_case(rank, world, name):
    from matrix_fsdp_b200 import configure_optimizer
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

    wrap, make_kw, opt_kind, o = (HSDP_CASES if name.startswith("hsdp_") else CASES)[name]
    reset_shared_owner_planners()
    model = _model(CkptBlk if o.get("ckpt") else Blk)
    if o.get("fn"):
        pattern = o["fn"]
        model = TopoNet(OrderedDict(model._modules))
        model.pattern = pattern
    ref = copy.deepcopy(model)
    kw = make_kw()
    if o.get("mesh") == "replicate_only":                     # a 2 x 1 mesh: nothing to shard, gradients averaged over replicas
        from torch.distributed.device_mesh import init_device_mesh

        from matrix_fsdp_b200 import DataParallelMeshDims

        if "replicate_only" not in _MESH:
            _MESH["replicate_only"] = init_device_mesh("cpu", (world, 1), mesh_dim_names=("dp_replicate", "dp_shard"))
        kw.update(mesh=_MESH["replicate_only"], dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    elif o.get("mesh") == "one_d_named":
        from torch.distributed.device_mesh import init_device_mesh

        if "one_d" not in _MESH:
            _MESH["one_d"] = init_device_mesh("cpu", (world,), mesh_dim_names=("dp",))
        kw.update(mesh=_MESH["one_d"])
    if name.startswith("hsdp_"):
        from matrix_fsdp_b200 import DataParallelMeshDims

        kw.update(mesh=_hsdp_mesh(world), dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))
    _shard(model, wrap, kw)
    if ":" in opt_kind:
        from matrix_fsdp_b200.optim.wrapper import MatrixFSDPOptimizer, install_matrix_optimizer_auto_prepare

        how, cls_name = opt_kind.split(":")
        cls = getattr(torch.optim, cls_name)
        opt = cls(model.parameters(), **o["torch_kw"])
        if how == "torch":
            opt = MatrixFSDPOptimizer(opt, model)
        else:
            install_matrix_optimizer_auto_prepare()
        ropt = cls(ref.parameters(), **o["torch_kw"])
    else:
        hyper = dict(lr=1e-2, weight_decay=0.0) if opt_kind == "adamw" else dict(lr=0.05)
        opt = configure_optimizer(model, opt_kind, **hyper, **o.get("opt_kw", {}))
        ropt = (torch.optim.AdamW if opt_kind == "adamw" else torch.optim.SGD)(ref.parameters(), **hyper)
    bf16 = bool(o.get("bf16"))
    g = torch.Generator().manual_seed(100 + rank)

    def loss_of(m, x):
        y = m(x.bfloat16()) if (bf16 and m is model) else m(x)
        return y.float().pow(2).mean()

    def backward_of(m, x):
        if not o.get("two_losses"):
            loss_of(m, x).backward()
            return
        # two losses over one forward: the graph is kept and walked twice, the gradients add up
        y = (m(x.bfloat16()) if (bf16 and m is model) else m(x)).float()
        y.pow(2).mean().backward(retain_graph=True)
        y.abs().mean().backward()

    for _ in range(len(_ORDERS) if o.get("fn") is _changing_order else 2):
        xs = [torch.randn(4, 8, generator=g) for _ in range(2 if o.get("no_sync") else 1)]
        if o.get("no_sync"):
            with model.no_sync():
                backward_of(model, xs[0])
            backward_of(model, xs[1])
        else:
            backward_of(model, xs[0])
        opt.step()
        opt.zero_grad()
        for x in xs:
            backward_of(ref, x)
        for p in ref.parameters():
            if p.grad is None:                                  # a module the step did not use
                continue
            dist.all_reduce(p.grad)
            if not o.get("sum"):
                p.grad /= world
        ropt.step()
        ropt.zero_grad()
    full = _full_params(model)
    tol = 3e-2 if bf16 else 3e-5
    for n, p in ref.named_parameters():
        assert torch.allclose(full[n], p.detach(), atol=tol, rtol=1e-3 if bf16 else 1e-4), \
            (n, float((full[n] - p.detach()).abs().max()))
    units = collect_param_groups(model)
    assert len(units) == {"root": 1}.get(wrap, 4)
    for u in units:
        if name.startswith("hsdp_"):
            assert u.world_size == world // 2 and u.replicate_world_size == 2
        assert u.state.value == "sharded", (u.name, u.state)
        assert u.flat_buffer.pending_reduce is None
        if not o.get("storage_may_stay"):
            assert u.full_param_storage_nbytes() == 0, u.name
        # the optimizer state of a rank is the size of its own shard, never of the whole unit
        assert u.flat_buffer.local_numel <= u.flat_buffer.total_numel
    if o.get("mesh") == "replicate_only":
        assert all(u.world_size == 1 and u.replicate_world_size == world for u in units)
    elif world > 1:
        assert sum(u.flat_buffer.local_numel for u in units) < sum(u.flat_buffer.total_numel for u in units)


# an odd world size: shard sizes with a remainder, rows that do not divide, three owners
THREE_RANK_CASES = ["root_default", "units_default", "policy_default", "units_keep_after_forward", "units_reduce_flat",
                    "units_reduce_per_param", "units_reduce_per_param_allreduce", "units_parameter_boundaries",
                    "units_ordered_groups", "units_owner_tail", "units_auto_balanced", "units_auto_min_comm",
                    "units_gather_padded", "units_gather_owner_broadcast", "units_gather_all_reduce", "units_rows",
                    "root_rows", "units_zero_copy_bucket", "units_saved_tensor_hooks", "units_bf16", "units_no_sync",
                    "units_activation_checkpoint", "units_layout_flat_reorder", "topo_branches", "topo_twice_keep",
                    "wrapped_torch_adam", "bare_torch_adamw", "units_two_losses", "root_two_losses", "topo_changing_order",
                    "topo_changing_order_next_step_prefetch"]


def _worker(rank, world, out_path, which):
    results = {}
    for name in {"hsdp": HSDP_CASES, "three": THREE_RANK_CASES}.get(which, CASES):
        try:
            _run_case(rank, world, name)
            mine = ""
        except Exception:
            mine = traceback.format_exc()
        # a case fails if it failed on any rank (ranks stay in lock-step: every collective of a case either ran
        # on both or raised before being issued)
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
        run_ranks(_worker, 2, path, "flat", timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.fixture(scope="module")
def three_rank_outcomes():
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, 3, path, "three", timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.fixture(scope="module")
def hsdp_outcomes():
    with tempfile.TemporaryDirectory() as tmp:
        path = os.path.join(tmp, "outcomes.json")
        run_ranks(_worker, 4, path, "hsdp", timeout=600.0)
        with open(path) as f:
            return json.load(f)


@pytest.mark.parametrize("case", sorted(CASES))
def test_two_rank_step_matches_eager_model(outcomes, case):
    assert case in outcomes, "the worker did not reach this case"
    assert not outcomes[case], outcomes[case]


@pytest.mark.parametrize("case", sorted(HSDP_CASES))
def test_four_rank_hsdp_step_matches_eager_model(hsdp_outcomes, case):
    assert case in hsdp_outcomes, "the worker did not reach this case"
    assert not hsdp_outcomes[case], hsdp_outcomes[case]


@pytest.mark.parametrize("case", THREE_RANK_CASES)
def test_three_rank_step_matches_eager_model(three_rank_outcomes, case):
    assert case in three_rank_outcomes, "the worker did not reach this case"
    assert not three_rank_outcomes[case], three_rank_outcomes[case]
