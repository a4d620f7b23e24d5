"""Sharded flat optimizers: one launch per FSDP unit over its contiguous local shard.

``FlatShardedAdamW`` and ``FlatShardedSGD`` are ``torch.optim.Optimizer`` subclasses, so
``param_groups`` / ``state`` / ``state_dict()`` behave as usual (per-parameter ``exp_avg`` /
``exp_avg_sq`` / ``step`` entries), but those state tensors are *views* of one flat fp32 buffer
per unit and ``step()`` runs a single fused kernel per unit: read the reduced gradient (bf16 or
fp32), apply the ``1/world`` / clipping scale, update fp32 master weights and moments, and emit
the bf16 copy that the next all-gather ships.  On CPU the same math runs as torch ops on the
flat buffers.  Parameters outside any unit are handled by a plain per-parameter loop.

What the reference does instead: hands shard views to ``torch.optim.AdamW`` (many small
tensors, ``matrix_fsdp/optim/wrapper.py:803-812``) and optionally pre-allocates the moments as
views of one flat buffer (``optim/adamw_state.py:44-87``); the dtype cast for the next gather
is a separate kernel (``runtime/flat_buffer.py:1186-1206``).
"""
from __future__ import annotations

import math
from collections.abc import Iterable

import torch
from torch.optim import Optimizer

from ..parallel.unit_collection import collect_param_groups


def _native(device: torch.device) -> bool:
    if device.type != "cuda":
        return False
    from ..ops import lib

    if lib.disabled_by_env():
        return False
    lib.load(required=True)   # on a GPU box a missing kernel library is an error, not a fallback
    return True


def _adamw_reference_(p, m, v, g, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale, p_lp=None) -> None:
    """torch-op AdamW on flat tensors (same update rule as ``torch.optim.AdamW``)."""
    g = g.to(torch.float32)
    if grad_scale != 1.0:
        g = g * grad_scale
    p.mul_(1.0 - lr * weight_decay)
    m.lerp_(g, 1.0 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
    bias1 = 1.0 - beta1 ** step
    bias2_sqrt = math.sqrt(1.0 - beta2 ** step)
    denom = (v.sqrt() / bias2_sqrt).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bias1)
    if p_lp is not None:
        p_lp.copy_(p)


# torch.optim keyword arguments that only select an implementation: accepted and irrelevant here
_IMPLEMENTATION_OPTIONS = ("foreach", "fused", "capturable", "differentiable")


def _check_torch_options(name: str, options: dict, **must_equal) -> None:
    """Reject keyword arguments this optimizer would otherwise silently drop."""
    for key, value in options.items():
        if key in _IMPLEMENTATION_OPTIONS:
            continue
        if key in must_equal:
            if value != must_equal[key]:
                raise NotImplementedError(f"{name}: {key}={value!r} is not supported by the flat sharded optimizer.")
            continue
        raise TypeError(f"{name}: unexpected keyword argument {key!r}.")


class _UnitState:
    """Flat optimizer state of one FSDP unit."""

    def __init__(self, unit, names: tuple[str, ...]) -> None:
        self.unit = unit
        fb = unit.flat_buffer
        self.buffers = {n: torch.zeros(fb.local_numel, dtype=torch.float32, device=fb.device) for n in names}
        self.step = 0

    def views(self, name: str) -> dict[str, torch.Tensor]:
        fb = self.unit.flat_buffer
        return {fqn: self.buffers[name][p.local_start:p.local_end].view(p.shape) for fqn, p in fb.pieces.items()}


class _FlatShardedBase(Optimizer):
    _state_names: tuple[str, ...] = ()

    def __init__(self, params, defaults, units=None) -> None:
        super().__init__(params, defaults)
        self._units = collect_param_groups(units) if units is not None else []
        self._unit_states: dict[int, _UnitState] = {}
        self._managed_ids: set[int] = set()
        self.grad_scale = 1.0          # extra scale applied on the fly (gradient clipping)
        for u in self._units:
            if u.flat_buffer.shard_dtype != torch.float32:
                continue
            hp_ids = {id(mp.param) for mp in u.registry}
            if not self._uniform_hyperparams(hp_ids):
                continue
            self._unit_states[id(u)] = _UnitState(u, self._state_names)
            self._managed_ids |= hp_ids
            if u.flat_buffer.world_size == 1 and u.flat_buffer.replicate_world_size == 1:
                u.flat_buffer.fused_optimizer_consumes_bucket = True
        self._bind_state_views()

    def _uniform_hyperparams(self, ids: set[int]) -> bool:
        """A unit takes the flat path only when all its params sit in one param group."""
        owners = {gi for gi, g in enumerate(self.param_groups) for p in g["params"] if id(p) in ids}
        return len(owners) == 1

    def _group_of(self, unit) -> dict:
        first = id(unit.registry[0].param)
        for g in self.param_groups:
            if any(id(p) == first for p in g["params"]):
                return g
        raise KeyError("unit parameters are not in this optimizer")

    def _bind_state_views(self) -> None:
        for us in self._unit_states.values():
            per_name = {n: us.views(n) for n in self._state_names}
            for mp in us.unit.registry:
                if mp.fqn not in us.unit.flat_buffer.pieces:
                    continue
                st = self.state[mp.param]
                st.setdefault("step", torch.tensor(float(us.step)))
                for n in self._state_names:
                    st[n] = per_name[n][mp.fqn]

    def load_state_dict(self, state_dict) -> None:
        super().load_state_dict(state_dict)
        # super() replaced the state tensors; fold them back into the flat buffers
        for us in self._unit_states.values():
            per_name = {n: us.views(n) for n in self._state_names}
            for mp in us.unit.registry:
                st = self.state.get(mp.param)
                if not st or mp.fqn not in us.unit.flat_buffer.pieces:
                    continue
                for n in self._state_names:
                    if n in st and st[n].data_ptr() != per_name[n][mp.fqn].data_ptr():
                        per_name[n][mp.fqn].copy_(st[n].reshape(per_name[n][mp.fqn].shape))
                    st[n] = per_name[n][mp.fqn]
                if "step" in st:
                    us.step = int(float(st["step"]))

    def _publish_step(self, us: _UnitState) -> None:
        """Mirror the unit's step count into the per-parameter state (what a checkpoint saves and a load reads
        back: a restored count of 0 would make the next step treat the moments as uninitialised)."""
        for mp in us.unit.registry:
            st = self.state.get(mp.param)
            if st and "step" in st:
                st["step"].fill_(us.step)

    def flat_state(self, unit) -> dict[str, torch.Tensor] | None:
        us = self._unit_states.get(id(unit))
        return us.buffers if us is not None else None

    def unit_step_count(self, unit) -> int:
        us = self._unit_states.get(id(unit))
        return us.step if us is not None else 0

    def _unit_grad(self, unit) -> torch.Tensor | None:
        """The unit's reduced gradient, or None when this step produced none for it (the buffer of an
        earlier step may still exist; like ``param.grad is None`` such a unit is skipped)."""
        fb = unit.flat_buffer
        return fb.local_grad_shard if fb.local_grad_valid else None


class FlatShardedAdamW(_FlatShardedBase):
    _state_names = ("exp_avg", "exp_avg_sq")

    def __init__(self, params: Iterable, *, units=None, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 1e-2, fused_reduce_update: bool = False, **torch_options) -> None:
        _check_torch_options("AdamW", torch_options, amsgrad=False, maximize=False)
        if lr < 0 or eps < 0 or not 0 <= betas[0] < 1 or not 0 <= betas[1] < 1 or weight_decay < 0:
            raise ValueError("invalid AdamW hyper-parameters")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay), units)
        # Opt-in: the update runs inside the gradient reduce-scatter kernel (peer transport), so the
        # reduced gradient is never materialised: no gradient clipping and ``param.grad`` stays None.
        self.fused_reduce_update = bool(fused_reduce_update)
        if self.fused_reduce_update:
            for us in self._unit_states.values():
                us.unit.flat_buffer.fused_reduce_update = self._make_fused_update(us)

    def _make_fused_update(self, us: _UnitState):
        def update():
            fb = us.unit.flat_buffer
            if fb.local_numel == 0 or not _native(fb.device) or self.grad_scale != 1.0 or \
                    (fb.local_shard_lp is not None and fb.local_shard_lp.dtype != torch.bfloat16):
                return None
            hp = self._group_of(us.unit)
            us.step += 1
            return dict(p=fb.local_shard, m=us.buffers["exp_avg"], v=us.buffers["exp_avg_sq"], p_lp=fb.local_shard_lp,
                        lr=float(hp["lr"]), beta1=hp["betas"][0], beta2=hp["betas"][1], eps=hp["eps"],
                        weight_decay=hp["weight_decay"], step=us.step)
        return update

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for us in self._unit_states.values():
            unit, fb = us.unit, us.unit.flat_buffer
            if fb.fused_update_applied:
                # the reduce-scatter kernel already updated master, moments and the bf16 shard
                fb.fused_update_applied = False
                fb.mark_master_updated(lp_written=fb.local_shard_lp is not None)
                self._publish_step(us)
                continue
            g = self._unit_grad(unit)
            if g is None or fb.local_numel == 0:
                continue
            hp = self._group_of(unit)
            us.step += 1
            kw = dict(lr=float(hp["lr"]), beta1=hp["betas"][0], beta2=hp["betas"][1], eps=hp["eps"],
                      weight_decay=hp["weight_decay"], step=us.step, grad_scale=float(self.grad_scale),
                      p_lp=fb.local_shard_lp)
            if _native(fb.device) and g.dtype in (torch.bfloat16, torch.float32) and \
                    (fb.local_shard_lp is None or fb.local_shard_lp.dtype == torch.bfloat16):
                from ..ops import kernels

                kernels.adamw_flat_(fb.local_shard, us.buffers["exp_avg"], us.buffers["exp_avg_sq"], g, **kw)
            else:
                _adamw_reference_(fb.local_shard, us.buffers["exp_avg"], us.buffers["exp_avg_sq"], g, **kw)
            fb.mark_master_updated(lp_written=fb.local_shard_lp is not None)
            self._publish_step(us)
        self._step_unmanaged()
        return loss

    def _step_unmanaged(self) -> None:
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if id(p) in self._managed_ids or p.grad is None or p.numel() == 0:
                    continue
                st = self.state[p]
                if "exp_avg" not in st:
                    st["step"] = torch.tensor(0.0)
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                step = int(st["step"].item())
                if p.dtype == torch.float32:
                    _adamw_reference_(p.data, st["exp_avg"], st["exp_avg_sq"], p.grad, lr=float(group["lr"]), beta1=b1,
                                      beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"], step=step,
                                      grad_scale=float(self.grad_scale))
                else:
                    master = st.setdefault("master", p.data.float())
                    _adamw_reference_(master, st["exp_avg"], st["exp_avg_sq"], p.grad, lr=float(group["lr"]), beta1=b1,
                                      beta2=b2, eps=group["eps"], weight_decay=group["weight_decay"], step=step,
                                      grad_scale=float(self.grad_scale))
                    p.data.copy_(master)


class FlatShardedSGD(_FlatShardedBase):
    _state_names = ("momentum_buffer",)

    def __init__(self, params: Iterable, *, units=None, lr: float = 1e-3, momentum: float = 0.0,
                 weight_decay: float = 0.0, **torch_options) -> None:
        _check_torch_options("SGD", torch_options, nesterov=False, dampening=0, maximize=False)
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay), units)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for us in self._unit_states.values():
            unit, fb = us.unit, us.unit.flat_buffer
            g = self._unit_grad(unit)
            if g is None or fb.local_numel == 0:
                continue
            hp = self._group_of(unit)
            first = us.step == 0
            us.step += 1
            mom = us.buffers["momentum_buffer"] if hp["momentum"] != 0 else None
            if _native(fb.device):
                from ..ops import kernels

                kernels.sgd_flat_(fb.local_shard, mom, g, lr=float(hp["lr"]), momentum=hp["momentum"],
                                  weight_decay=hp["weight_decay"], first_step=first,
                                  grad_scale=float(self.grad_scale), p_lp=fb.local_shard_lp)
            else:
                gf = g.to(torch.float32) * float(self.grad_scale)
                if hp["weight_decay"]:
                    gf = gf.add(fb.local_shard, alpha=hp["weight_decay"])
                if mom is not None:
                    if first:
                        mom.copy_(gf)
                    else:
                        mom.mul_(hp["momentum"]).add_(gf)
                    gf = mom
                fb.local_shard.add_(gf, alpha=-float(hp["lr"]))
                if fb.local_shard_lp is not None:
                    fb.local_shard_lp.copy_(fb.local_shard)
            fb.mark_master_updated(lp_written=fb.local_shard_lp is not None)
            self._publish_step(us)
        for group in self.param_groups:
            for p in group["params"]:
                if id(p) in self._managed_ids or p.grad is None or p.numel() == 0:
                    continue
                gf = p.grad.float() * float(self.grad_scale)
                if group["weight_decay"]:
                    gf = gf.add(p.data.float(), alpha=group["weight_decay"])
                if group["momentum"]:
                    st = self.state[p]
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = gf.clone()
                    else:
                        st["momentum_buffer"].mul_(group["momentum"]).add_(gf)
                    gf = st["momentum_buffer"]
                p.data.add_(gf.to(p.dtype), alpha=-float(group["lr"]))
        return loss
