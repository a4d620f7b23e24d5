"""FSDP2 / DCP-shaped state-dict facade over the sharded state.

``get_model_state_dict`` / ``get_optimizer_state_dict`` / ``get_state_dict`` and their ``set_*``
twins mirror ``torch.distributed.checkpoint.state_dict``; ``options.full_state_dict`` gathers every
unit and returns ordinary full tensors keyed like ``module.state_dict()`` (optionally on CPU).
``patch_model_state_dict`` / ``patch_optimizer_state_dict`` rebind ``state_dict`` /
``load_state_dict`` on the objects themselves.

Parity: ``matrix_fsdp/checkpoint/_api.py:1-277``.
"""
from __future__ import annotations

import functools
from dataclasses import dataclass
from typing import Any

import torch
from torch import nn

from ..parallel.unit_collection import collect_param_groups
from .state_dict import (_full_master_params, iter_optimizer_components, load_matrix_state_dict,
                         matrix_state_dict)


@dataclass
class MatrixStateDictOptions:
    full_state_dict: bool = False
    cpu_offload: bool = False
    strict: bool = True


def _opts(options) -> MatrixStateDictOptions:
    if options is None:
        return MatrixStateDictOptions()
    return MatrixStateDictOptions(bool(getattr(options, "full_state_dict", False)),
                                  bool(getattr(options, "cpu_offload", False)), bool(getattr(options, "strict", True)))


def _full_model_state(model: nn.Module, cpu: bool) -> dict[str, torch.Tensor]:
    units = collect_param_groups(model)
    masters = _full_master_params(units)
    by_name = {n: p for n, p in model.named_parameters(remove_duplicate=False)}
    for u in units:
        u.unshard("state_dict")
    try:
        out = {}
        for k, v in nn.Module.state_dict(model).items():
            master = masters.get(id(by_name[k])) if k in by_name else None
            t = master if master is not None else v.detach().clone()   # the master, never its low-precision copy
            out[k] = t.cpu() if cpu else t
    finally:
        for u in units:
            u.reshard("state_dict")
    return out


def get_model_state_dict(model: nn.Module, *, options=None) -> dict[str, Any]:
    o = _opts(options)
    if o.full_state_dict:
        return _full_model_state(model, o.cpu_offload)
    return matrix_state_dict(model, clone=True)


def set_model_state_dict(model: nn.Module, model_state_dict, *, options=None) -> None:
    o = _opts(options)
    if o.full_state_dict or "units" not in model_state_dict:
        units = collect_param_groups(model)
        by_param = {}
        for u in units:
            for mp in u.registry:
                by_param[id(mp.param)] = (u, mp)
        if o.strict:
            # like nn.Module.load_state_dict(strict=True): nothing the model does not know, checked before anything
            # is written
            known = {n for n, _ in model.named_parameters(remove_duplicate=False)} | {n for n, _ in model.named_buffers()}
            unexpected = sorted(k for k in model_state_dict if k not in known)
            if unexpected:
                raise KeyError(f"unexpected key(s) in state dict: {', '.join(map(repr, unexpected))}")
        shapes = {id(mp.param): tuple(mp.shape) for u in units for mp in u.registry}
        with torch.no_grad():
            for name, p in model.named_parameters(remove_duplicate=False):
                if name not in model_state_dict:
                    if o.strict:
                        raise KeyError(f"missing key {name!r} in state dict")
                    continue
                full = model_state_dict[name]
                want = shapes.get(id(p), tuple(p.shape))
                if tuple(full.shape) != want:
                    raise RuntimeError(f"size mismatch for {name}: the state dict holds shape {tuple(full.shape)}, "
                                       f"the model's parameter has shape {want}")
                hit = by_param.get(id(p))
                if hit is None:
                    p.data.copy_(full.to(p.device))
                    continue
                u, mp = hit
                piece = u.flat_buffer.pieces.get(mp.fqn)
                if piece is not None:
                    src = full.reshape(-1)[piece.param_start:piece.param_start + piece.numel]
                    u.flat_buffer.local_shard[piece.local_start:piece.local_end].copy_(src.to(u.flat_buffer.device))
            for u in units:
                u.flat_buffer.mark_master_updated(lp_written=False)
            for name, b in model.named_buffers():
                if name in model_state_dict:
                    b.copy_(model_state_dict[name].to(b.device))
        return
    load_matrix_state_dict(model, model_state_dict, strict=o.strict)


def _full_optimizer_state(model: nn.Module, optimizer, cpu: bool) -> dict[str, Any]:
    """``{component: {"state": {parameter name: {state name: full tensor or scalar}}, "param_groups": [...]}}``.

    Every rank of a shard group holds disjoint pieces of each state tensor (the piece of its parameter shard),
    so the full tensor is the sum of the pieces placed at their parameter offsets: one all-reduce per
    (parameter, state) over the unit's shard group.  Collective: every rank must call it.
    """
    import torch.distributed as dist

    units = collect_param_groups(model)
    name_of = {id(p): n for n, p in model.named_parameters(remove_duplicate=False)}
    out: dict[str, Any] = {}
    for comp, opt in iter_optimizer_components(optimizer):
        state_out: dict[str, dict[str, Any]] = {}
        managed: set[int] = set()
        for u in units:
            group = u.groups.shard_group if u.world_size > 1 else None
            local_names = {}
            for mp in u.registry:
                managed.add(id(mp.param))
                st = opt.state.get(mp.param, {})
                local_names[mp.fqn] = sorted(k for k, v in st.items() if isinstance(v, torch.Tensor) and v.dim() > 0) + \
                    sorted("#" + k for k, v in st.items() if not (isinstance(v, torch.Tensor) and v.dim() > 0))
            if group is not None:
                gathered: list = [None] * u.world_size
                dist.all_gather_object(gathered, local_names, group=group)
            else:
                gathered = [local_names]
            for mp in u.registry:
                names = sorted({n for g in gathered for n in g.get(mp.fqn, ())})
                if not names:
                    continue
                st = opt.state.get(mp.param, {})
                piece = u.flat_buffer.pieces.get(mp.fqn)
                entry: dict[str, Any] = {}
                for n in names:
                    if n.startswith("#"):                                   # scalar state (step): same on every owner
                        v = st.get(n[1:])
                        val = torch.tensor(float(v) if v is not None else float("-inf"), dtype=torch.float64)
                        if group is not None:
                            val = val.to(u.flat_buffer.device)
                            dist.all_reduce(val, op=dist.ReduceOp.MAX, group=group)
                        entry[n[1:]] = float(val)
                        continue
                    local = st.get(n)
                    dtype = local.dtype if local is not None else torch.float32
                    if group is not None:
                        code = torch.tensor([{torch.float32: 0, torch.bfloat16: 1, torch.float16: 2,
                                              torch.float64: 3}.get(dtype, 0) if local is not None else -1],
                                            device=u.flat_buffer.device)
                        dist.all_reduce(code, op=dist.ReduceOp.MAX, group=group)
                        dtype = (torch.float32, torch.bfloat16, torch.float16, torch.float64)[max(int(code), 0)]
                    full = torch.zeros(mp.numel, dtype=torch.float32 if dtype != torch.float64 else dtype,
                                       device=u.flat_buffer.device)
                    if local is not None and piece is not None and local.numel() == piece.numel:
                        full[piece.param_start:piece.param_start + piece.numel] = local.reshape(-1).to(full.dtype)
                    if group is not None:
                        dist.all_reduce(full, group=group)
                    full = full.to(dtype).view(mp.shape)
                    entry[n] = full.cpu() if cpu else full
                key = name_of.get(id(mp.param), f"{u.name}.{mp.fqn}")
                state_out[key] = entry
        for g in opt.param_groups:                                           # parameters outside any unit
            for p in g["params"]:
                if id(p) in managed or p not in opt.state:
                    continue
                state_out[name_of.get(id(p), str(id(p)))] = {
                    k: (v.detach().clone().cpu() if cpu else v.detach().clone()) if isinstance(v, torch.Tensor) else v
                    for k, v in opt.state[p].items()}
        groups = [{k: v for k, v in g.items() if k != "params"} for g in opt.param_groups]
        out[comp] = {"state": state_out, "param_groups": groups}
    return out


def get_optimizer_state_dict(model: nn.Module, optimizers, *, options=None) -> dict[str, Any]:
    """Local (sharded) optimizer state dicts per component; with ``options.full_state_dict`` the state tensors are
    assembled to full size and keyed by parameter name instead (collective)."""
    o = _opts(options)
    opts = optimizers if isinstance(optimizers, (list, tuple)) else [optimizers]
    out: dict[str, Any] = {}
    for i, opt in enumerate(opts):
        if o.full_state_dict:
            out[str(i)] = _full_optimizer_state(model, opt, o.cpu_offload)
        else:
            out[str(i)] = {name: c.state_dict() for name, c in iter_optimizer_components(opt)}
    return out if len(opts) > 1 else out["0"]      # several optimizers: keyed "0", "1", … like the reference


def _is_full_form(component_sd) -> bool:
    """The gathered form keys ``state`` by parameter name; a local ``state_dict()`` keys it by integer."""
    state = component_sd.get("state", {})
    return bool(state) and all(isinstance(k, str) for k in state)


def _load_full_optimizer_component(model: nn.Module, opt, component_sd) -> None:
    """Scatter gathered (full-size) optimizer tensors back: every rank keeps the piece of each tensor that
    matches the piece of the parameter it holds."""
    units = collect_param_groups(model)
    owner = {id(mp.param): (u, mp) for u in units for mp in u.registry}
    by_name = dict(model.named_parameters(remove_duplicate=False))
    with torch.no_grad():
        for name, entry in component_sd["state"].items():
            p = by_name.get(name)
            if p is None:
                raise KeyError(f"optimizer state names unknown parameter {name!r}")
            hit = owner.get(id(p))
            piece = hit[0].flat_buffer.pieces.get(hit[1].fqn) if hit is not None else None
            if hit is not None and piece is None:
                continue                                  # nothing of this parameter lives here
            if not any(p is q for g in opt.param_groups for q in g["params"]):
                continue                                  # another component's parameter
            st = opt.state[p]
            for k, v in entry.items():
                if not torch.is_tensor(v) or v.dim() == 0:
                    cur = st.get(k)
                    if torch.is_tensor(cur) and cur.numel() == 1:
                        cur.fill_(float(v))
                    else:
                        st[k] = torch.tensor(float(v)) if k == "step" else v
                    continue
                if hit is None:
                    st[k] = v.detach().clone().to(p.device)
                    continue
                u, mp = hit
                part = v.reshape(-1)[piece.param_start:piece.param_start + piece.numel].to(u.flat_buffer.device)
                cur = st.get(k)
                if torch.is_tensor(cur) and cur.numel() == part.numel():
                    cur.copy_(part.view(cur.shape).to(cur.dtype))
                else:
                    st[k] = part.view(piece.shape).clone()
        for g, sg in zip(opt.param_groups, component_sd.get("param_groups", [])):
            for k, v in sg.items():
                if k != "params":
                    g[k] = v
    unit_states = getattr(opt, "_unit_states", None)
    if unit_states:                                       # flat optimizers keep one step counter per unit
        for us in unit_states.values():
            steps = [float(opt.state[mp.param]["step"]) for mp in us.unit.registry
                     if mp.param in opt.state and "step" in opt.state[mp.param]]
            if steps:
                us.step = int(max(steps))


def set_optimizer_state_dict(model: nn.Module, optimizers, optim_state_dict, *, options=None) -> None:
    """Inverse of :func:`get_optimizer_state_dict` for both of its forms: the local one goes through
    ``load_state_dict``, the gathered one (``options.full_state_dict`` or state keyed by parameter names)
    is scattered onto the shards."""
    o = _opts(options)
    opts = optimizers if isinstance(optimizers, (list, tuple)) else [optimizers]
    for i, opt in enumerate(opts):
        if len(opts) > 1:
            sd = optim_state_dict[str(i)] if str(i) in optim_state_dict else optim_state_dict[f"optimizer_{i}"]
        else:
            sd = optim_state_dict
        for name, comp in iter_optimizer_components(opt):
            if name not in sd:
                raise ValueError(f"missing component {name!r} in optimizer state dict")
            if o.full_state_dict or _is_full_form(sd[name]):
                _load_full_optimizer_component(model, comp, sd[name])
            else:
                comp.load_state_dict(sd[name])


def get_state_dict(model: nn.Module, optimizers, *, options=None):
    return get_model_state_dict(model, options=options), get_optimizer_state_dict(model, optimizers, options=options)


def set_state_dict(model: nn.Module, optimizers, *, model_state_dict, optim_state_dict, options=None) -> None:
    set_model_state_dict(model, model_state_dict, options=options)
    set_optimizer_state_dict(model, optimizers, optim_state_dict, options=options)


matrix_get_state_dict = get_state_dict
matrix_set_state_dict = set_state_dict


def patch_model_state_dict(model: nn.Module, *, options=None) -> None:
    model.state_dict = functools.partial(get_model_state_dict, model, options=options)  # type: ignore[assignment]
    base = _opts(options)

    def load(sd, strict: bool = True, **kw):
        set_model_state_dict(model, sd, options=MatrixStateDictOptions(base.full_state_dict, base.cpu_offload,
                                                                       bool(strict) and base.strict))

    model.load_state_dict = load  # type: ignore[assignment]


def patch_optimizer_state_dict(model: nn.Module, *, optimizers, options=None) -> None:
    opts = optimizers if isinstance(optimizers, (list, tuple)) else [optimizers]
    for opt in opts:
        opt.state_dict = functools.partial(get_optimizer_state_dict, model, opt, options=options)
        opt.load_state_dict = functools.partial(set_optimizer_state_dict, model, opt, options=options)
