"""Ordinary PyTorch modules and training-loop habits under ``fully_shard`` (single rank, CPU): every case trains the
sharded module and an untouched copy side by side and expects identical parameters.  Modules: keyword inputs and
dataclass outputs, autocast, in-place edits of outputs, user hooks, integer inputs (embedding), buffers (batch
norm), ``nn.LSTM``, ``nn.MultiheadAttention``.  Habits: stepping twice, ``zero_grad(set_to_none=False)``, an
exception inside a forward, accumulation without ``no_sync``, discarding gradients - each with the flat optimizer
and with a user-built torch optimizer behind the wrapper."""
import copy
import dataclasses

import pytest
import torch
from torch import nn

from matrix_fsdp_b200 import configure_optimizer, fully_shard
from matrix_fsdp_b200.api import reset_shared_owner_planners
from matrix_fsdp_b200.optim.wrapper import MatrixFSDPOptimizer
from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups


def _difference(model, ref) -> float:
    units = collect_param_groups(model)
    for u in units:
        u.unshard("test")
    worst = max(float((p.detach() - q.detach()).abs().max()) for p, q in zip(model.parameters(), ref.parameters()))
    for u in units:
        u.reshard("test")
    return worst


def _train(model, ref, loss_of, steps=2, make_input=None):
    opt, ropt = configure_optimizer(model, "adamw", lr=1e-2), torch.optim.AdamW(ref.parameters(), lr=1e-2)
    for i in range(steps):
        g = torch.Generator().manual_seed(i)
        x = make_input(g) if make_input else torch.randn(3, 4, generator=g)
        loss_of(model, x).backward()
        loss_of(ref, x).backward()
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    return _difference(model, ref)


def _sharded(module, *, inner=None):
    reset_shared_owner_planners()
    ref = copy.deepcopy(module)
    if inner is not None:
        fully_shard(inner(module))
    fully_shard(module)
    return module, ref


def _mlp():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(4, 4), nn.ReLU(), nn.Linear(4, 4))


# ------------------------------------------------------------------------------------------ modules
@dataclasses.dataclass
class _Out:
    y: torch.Tensor
    aux: torch.Tensor


class _Keyworded(nn.Module):
    def __init__(self):
        super().__init__()
        self.a, self.b = nn.Linear(4, 4), nn.Linear(4, 4)

    def forward(self, x, *, scale=None):
        y = self.a(x)
        if scale is not None:
            y = y * scale
        return _Out(self.b(y), y.mean())


def test_keyword_inputs_and_dataclass_outputs():
    torch.manual_seed(0)
    model, ref = _sharded(_Keyworded())

    def loss_of(m, x):
        out = m(x, scale=torch.full((4,), 0.5))
        return out.y.pow(2).mean() + out.aux

    assert _train(model, ref, loss_of) == 0.0


def test_autocast_around_the_forward():
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])

    def loss_of(m, x):
        with torch.autocast("cpu", dtype=torch.bfloat16):
            return m(x).float().pow(2).mean()

    assert _train(model, ref, loss_of) == 0.0


def test_in_place_edits_of_a_units_output():
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])

    def loss_of(m, x):
        y = m(x)
        y += 1.0
        y.mul_(2.0)
        return y.pow(2).mean()

    assert _train(model, ref, loss_of) == 0.0


def test_user_hooks_on_a_unit_keep_firing():
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    calls = []
    model[0].register_forward_hook(lambda mod, i, o: calls.append("forward"))
    model[0].register_full_backward_hook(lambda mod, gi, go: calls.append("backward"))
    assert _train(model, ref, lambda m, x: m(x).pow(2).mean()) == 0.0
    assert calls == ["forward", "backward", "forward", "backward"]


def test_integer_inputs_reach_an_embedding_inside_a_unit():
    class Emb(nn.Module):
        def __init__(self):
            super().__init__()
            self.e, self.l = nn.Embedding(10, 4), nn.Linear(4, 4)

        def forward(self, ids):
            return self.l(self.e(ids))

    torch.manual_seed(0)
    model, ref = _sharded(Emb())
    diff = _train(model, ref, lambda m, ids: m(ids).pow(2).mean(), make_input=lambda g: torch.randint(0, 10, (3, 5), generator=g))
    assert diff == 0.0


def test_buffers_stay_ordinary_tensors():
    torch.manual_seed(0)
    model, ref = _sharded(nn.Sequential(nn.Linear(4, 4), nn.BatchNorm1d(4), nn.Linear(4, 4)))
    assert _train(model, ref, lambda m, x: m(x).pow(2).mean()) == 0.0
    assert torch.equal(model[1].running_mean, ref[1].running_mean) and int(model[1].num_batches_tracked) == 2


def test_lstm_with_its_flattened_weights():
    torch.manual_seed(0)
    model, ref = _sharded(nn.LSTM(4, 4, batch_first=True))
    assert _train(model, ref, lambda m, x: m(x.unsqueeze(0))[0].pow(2).mean()) == 0.0


def test_multihead_attention_with_its_packed_projection():
    torch.manual_seed(0)
    model, ref = _sharded(nn.MultiheadAttention(4, 2, batch_first=True))

    def loss_of(m, x):
        q = x.unsqueeze(0)
        return m(q, q, q)[0].pow(2).mean()

    assert _train(model, ref, loss_of) == 0.0


# ------------------------------------------------------------------------------------------ habits
def _optimizers(kind, model, ref):
    if kind == "flat":
        opt = configure_optimizer(model, "sgd", lr=0.1, momentum=0.9)
    else:
        opt = MatrixFSDPOptimizer(torch.optim.SGD(model.parameters(), lr=0.1, momentum=0.9), model)
    return opt, torch.optim.SGD(ref.parameters(), lr=0.1, momentum=0.9)


def _both_backward(model, ref, seed):
    x = torch.randn(2, 4, generator=torch.Generator().manual_seed(seed))
    model(x).sum().backward()
    ref(x).sum().backward()


@pytest.mark.parametrize("kind", ["flat", "torch"])
def test_stepping_twice_applies_the_kept_gradients_twice(kind):
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    opt, ropt = _optimizers(kind, model, ref)
    _both_backward(model, ref, 0)
    opt.step(), opt.step()
    ropt.step(), ropt.step()
    assert _difference(model, ref) == 0.0


@pytest.mark.parametrize("kind", ["flat", "torch"])
def test_zero_grad_that_keeps_the_tensors(kind):
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    opt, ropt = _optimizers(kind, model, ref)
    for i in range(3):
        _both_backward(model, ref, i)
        opt.step(), ropt.step()
        opt.zero_grad(set_to_none=False), ropt.zero_grad(set_to_none=False)
    assert _difference(model, ref) == 0.0


@pytest.mark.parametrize("kind", ["flat", "torch"])
def test_an_exception_inside_a_forward_leaves_the_units_usable(kind):
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    opt, ropt = _optimizers(kind, model, ref)
    with pytest.raises(RuntimeError):
        model(torch.randn(2, 5))                            # wrong width: the first unit raises mid-forward
    for i in range(2):
        _both_backward(model, ref, i)
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    assert _difference(model, ref) == 0.0


@pytest.mark.parametrize("kind", ["flat", "torch"])
def test_accumulation_without_no_sync_reduces_every_time_and_adds_up(kind):
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    opt, ropt = _optimizers(kind, model, ref)
    for i in range(2):
        _both_backward(model, ref, 2 * i)
        _both_backward(model, ref, 2 * i + 1)
        opt.step(), ropt.step()
        opt.zero_grad(), ropt.zero_grad()
    assert _difference(model, ref) == 0.0


@pytest.mark.parametrize("kind", ["flat", "torch"])
def test_zero_grad_discards_reduced_gradients(kind):
    model, ref = _sharded(_mlp(), inner=lambda m: m[0])
    opt, ropt = _optimizers(kind, model, ref)
    _both_backward(model, ref, 0)
    opt.zero_grad(), ropt.zero_grad()
    _both_backward(model, ref, 1)
    opt.step(), ropt.step()
    assert _difference(model, ref) == 0.0
