"""The flat buffer of one unit, one property per test (single rank, CPU): how parameters, gradients and their
views map onto the flat storage.  The reference keeps the same properties in test/fsdp/test_flat_buffer.py."""
import pytest
import torch
from torch import nn
from torch.distributed.fsdp import MixedPrecisionPolicy

from matrix_fsdp_b200 import configure_optimizer, fully_shard, matrix_fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners


def _unit(module=None, **kw):
    reset_shared_owner_planners()
    torch.manual_seed(0)
    module = module if module is not None else nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2))
    fully_shard(module, **kw)
    return module, module._matrix_fsdp_param_group


def test_pieces_tile_the_flat_space_in_registration_order():
    m, u = _unit()
    fb = u.flat_buffer
    assert fb.total_numel == sum(p.numel() for p in m.parameters()) == fb.local_numel
    ends = 0
    for (fqn, piece), (name, p) in zip(fb.pieces.items(), m.named_parameters()):
        assert fqn == name and piece.local_start == ends and piece.local_end - piece.local_start == p.numel()
        assert tuple(piece.shape) == tuple(p.shape)
        ends = piece.local_end
    assert ends == fb.local_numel and fb.owned_fqns() == tuple(n for n, _ in m.named_parameters())


def test_local_views_keep_the_parameter_shapes_and_alias_the_shard():
    m, u = _unit()
    fb = u.flat_buffer
    views = fb.local_param_views()
    lo, hi = fb.local_shard.data_ptr(), fb.local_shard.data_ptr() + fb.local_shard.numel() * 4
    for name, p in m.named_parameters():
        assert tuple(views[name].shape) == tuple(p.shape) and lo <= views[name].data_ptr() < hi
    views["0.bias"].fill_(7.0)
    piece = fb.pieces["0.bias"]
    assert torch.all(fb.local_shard[piece.local_start:piece.local_end] == 7.0)


def test_module_parameters_are_views_of_the_flat_shard_while_sharded():
    m, u = _unit()
    fb = u.flat_buffer
    lo, hi = fb.local_shard.data_ptr(), fb.local_shard.data_ptr() + fb.local_shard.numel() * 4
    assert all(lo <= p.data_ptr() < hi for p in m.parameters())
    with torch.no_grad():
        fb.local_shard.zero_()
    assert all(float(p.abs().sum()) == 0.0 for p in m.parameters())          # one storage, many views


def test_single_rank_full_buffer_aliases_the_shard():
    m, u = _unit()
    fb = u.flat_buffer
    assert fb.full_aliases_shard and fb.full_storage_nbytes() == 0
    u.unshard()
    assert fb.full_storage_nbytes() == 0 and m[0].weight.data_ptr() >= fb.local_shard.data_ptr()
    u.reshard()


def test_gradients_land_in_the_bucket_and_become_the_local_gradient_shard():
    m, u = _unit()
    opt = configure_optimizer(m, "sgd", lr=0.1)
    fb = u.flat_buffer
    assert not fb.local_grad_valid
    x = torch.randn(3, 4)
    m(x).sum().backward()
    assert fb.local_grad_valid and fb.local_grad_shard.shape == (fb.local_numel,)
    ref = nn.Sequential(nn.Linear(4, 6), nn.Linear(6, 2))
    ref.load_state_dict({k: v.detach().clone() for k, v in m.state_dict().items()})
    ref(x).sum().backward()
    for name, p in ref.named_parameters():
        piece = fb.pieces[name]
        assert torch.allclose(fb.local_grad_shard[piece.local_start:piece.local_end].view(p.shape), p.grad, atol=1e-6), name
    opt.step()
    opt.zero_grad()
    assert not fb.local_grad_valid                                           # consumed and cleared


def test_memory_snapshot_accounts_for_shard_bucket_and_gradient():
    m, u = _unit()
    configure_optimizer(m, "sgd", lr=0.1)
    fb = u.flat_buffer
    before = fb.memory_snapshot()
    assert before["local_shard_bytes"] == fb.local_numel * 4 and before["grad_bucket_bytes"] == 0
    m(torch.randn(3, 4)).sum().backward()
    after = fb.memory_snapshot()
    assert after["local_grad_shard_numel"] == fb.local_numel and after["local_grad_shard_bytes"] > 0


def test_param_dtype_casts_the_compute_copy_only():
    m, u = _unit(nn.Linear(4, 4), mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16))
    fb = u.flat_buffer
    assert fb.local_shard.dtype == torch.float32 and fb.param_dtype == torch.bfloat16
    assert fb.local_shard_lp is not None and fb.local_shard_lp.dtype == torch.bfloat16
    u.unshard()
    assert m.weight.dtype == torch.bfloat16
    u.reshard()
    assert torch.allclose(fb.local_shard_lp.float(), fb.local_shard, atol=1e-2)


def test_reduce_dtype_is_recorded_and_transports_that_sum_in_fp32_keep_the_compute_dtype_on_the_wire():
    m, u = _unit(nn.Linear(4, 4), mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32))
    opt = configure_optimizer(m, "sgd", lr=0.1)
    fb = u.flat_buffer
    assert fb.reduce_dtype == torch.float32
    # one rank only copies (no rounding in the "sum"), so the bucket stays in the dtype the gradients were produced in
    assert fb.transport.accumulates_fp32 and fb._bucket_dtype() == torch.bfloat16
    before = fb.local_shard.clone()
    m(torch.randn(2, 4).bfloat16()).float().sum().backward()
    assert fb.local_grad_valid
    opt.step()
    assert fb.local_shard.dtype == torch.float32 and not torch.equal(fb.local_shard, before)


def test_low_precision_copy_follows_the_master_after_an_update():
    m, u = _unit(nn.Linear(4, 4), mp_policy=MixedPrecisionPolicy(param_dtype=torch.bfloat16))
    opt = configure_optimizer(m, "sgd", lr=0.5)
    fb = u.flat_buffer
    before = fb.local_shard.clone()
    m(torch.randn(2, 4).bfloat16()).float().sum().backward()
    opt.step()
    assert not torch.equal(fb.local_shard, before)
    u.unshard()                                                              # the gather refreshes the bf16 copy
    assert torch.allclose(m.weight.float().reshape(-1), fb.local_shard[:16].bfloat16().float())
    u.reshard()


def test_unknown_collective_backend_and_strategies_are_rejected():
    with pytest.raises(ValueError, match="matrix_collective_backend"):
        matrix_fully_shard(nn.Linear(4, 4), matrix_collective_backend="smoke_signals")
    with pytest.raises(ValueError):
        matrix_fully_shard(nn.Linear(4, 4), param_gather_strategy="teleport")
    with pytest.raises(ValueError):
        matrix_fully_shard(nn.Linear(4, 4), backward_reduce_strategy="telepathy")


def test_zero_copy_bucket_makes_param_grads_views_of_the_bucket():
    reset_shared_owner_planners()
    m = nn.Linear(4, 4)
    matrix_fully_shard(m, use_zero_copy_grad_bucket=True)
    u = m._matrix_fsdp_param_group
    configure_optimizer(m, "sgd", lr=0.1)
    seen = {}
    m.weight.register_hook(lambda g: seen.update(shape=tuple(g.shape)))
    m(torch.randn(2, 4)).sum().backward()
    assert seen["shape"] == (4, 4) and u.flat_buffer.local_grad_valid


def test_accumulated_local_gradients_add_up_under_no_sync():
    m, u = _unit(nn.Linear(4, 4))
    opt = configure_optimizer(m, "sgd", lr=0.1)
    fb = u.flat_buffer
    x = torch.randn(2, 4)
    m(x).sum().backward()
    single = fb.local_grad_shard.clone()
    opt.zero_grad()
    with opt.no_sync():
        m(x).sum().backward()
    m(x).sum().backward()
    assert torch.allclose(fb.local_grad_shard, 2 * single, atol=1e-6)


def test_clear_full_params_keeps_or_drops_storage_on_request():
    m, u = _unit()
    fb = u.flat_buffer
    u.unshard()
    fb.use_local_shards()
    fb.clear_full_params(keep_storage=True)
    fb.clear_full_params()
    assert fb.full_storage_nbytes() == 0
