"""Small user-facing training helpers.

``train_step`` is the whole per-step call a user makes: copy the step's token batch from pinned
host memory, forward, backward, optimizer step, and read the loss back to the host.  The reference leaves the
training loop to its users (its bench loop is ``test/fsdp/bench_fsdp2_compare.py:1658-1708``).
"""
from __future__ import annotations

import torch


def pin(t: torch.Tensor) -> torch.Tensor:
    return t.pin_memory() if torch.cuda.is_available() and not t.is_pinned() else t


def train_step(model: torch.nn.Module, optimizer, host_tokens: torch.Tensor, host_targets: torch.Tensor,
               device: torch.device | str) -> float:
    """One optimisation step from host data; returns the loss as a Python float (device→host read)."""
    tokens = host_tokens.to(device, non_blocking=True)
    targets = host_targets.to(device, non_blocking=True)
    loss = model(tokens, targets)
    loss.backward()
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    value = float(loss.item())
    raise_on_device_error(tokens.device)
    return value


def raise_on_device_error(device=None) -> None:
    """Read the device status word (4 bytes, after a point where the host already synchronised) and raise
    if a bounded wait in one of the kernels gave up during the step: a peer that never published its
    shard or gradients must stop the run instead of training on data that did not arrive."""
    dev = torch.device(device) if device is not None else None
    if dev is None or dev.type != "cuda":
        return
    from ..ops import kernels, lib

    if lib.available() and not lib.disabled_by_env():
        kernels.check_status(dev)


def device_train_step(model: torch.nn.Module, optimizer, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Same step with inputs already on the device and the loss left on the device."""
    loss = model(tokens, targets)
    loss.backward()
    optimizer.step()
    optimizer.zero_grad(set_to_none=True)
    return loss.detach()


@torch.no_grad()
def clip_grad_norm_(module_or_units, max_norm: float, norm_type: float = 2.0,
                    error_if_nonfinite: bool = False, *, extra_grads=(), extra_group=None,
                    extra_scale: float = 1.0) -> torch.Tensor:
    """Clip the global gradient norm of a sharded model in place and return the norm before clipping.

    Every rank only holds its shard of each unit's reduced gradient, so the norm is assembled from the local
    shards with one all-reduce per shard group (replicas of an HSDP mesh hold identical shards and are not
    counted twice).  Call it after ``backward()`` and before ``optimizer.step()``; it waits for the units'
    pending reduce-scatters first.  ``torch.nn.utils.clip_grad_norm_`` on the module would see local shards
    only, which is what the reference leaves its users with.

    ``extra_grads``: gradients of parameters no unit manages and that every rank of ``extra_group`` owns a
    different part of (expert-parallel weights); their contribution is summed over ``extra_group``, counted
    ``extra_scale`` times (the factor their optimizer applies to them, e.g. ``1 / world`` when they hold sums over
    the ranks' tokens), and they are clipped in place with the same coefficient.
    """
    import math

    import torch.distributed as dist

    from ..parallel.unit_collection import collect_param_groups

    units = collect_param_groups(module_or_units)
    inf = math.isinf(norm_type)
    per_group: dict[object, tuple[object, torch.Tensor]] = {}
    shards = []
    for u in units:
        u.wait_post_backward_reduce()
        g = u.flat_buffer.local_grad_shard if u.flat_buffer.local_grad_valid else None
        if g is None or g.numel() == 0:
            continue
        shards.append(g)
        part = g.detach().float().abs().max() if inf else g.detach().float().norm(norm_type).pow(norm_type)
        group = u.groups.shard_group if u.world_size > 1 else None
        key = id(group)
        if key in per_group:
            prev = per_group[key][1]
            per_group[key] = (group, torch.maximum(prev, part) if inf else prev + part)
        else:
            per_group[key] = (group, part)
    extra_grads = list(extra_grads)
    extra = [g for g in extra_grads if g is not None and g.numel()]
    if extra_grads:                  # also a rank whose experts saw no token joins the group's sum
        parts = [g.detach().float().abs().max() if inf else g.detach().float().norm(norm_type).pow(norm_type)
                 for g in extra]
        ref = shards[0] if shards else (extra[0] if extra else None)
        part = (torch.stack(parts).max() if inf else torch.stack(parts).sum()) if parts else \
            torch.zeros((), device=ref.device if ref is not None else None)
        part = part * (abs(extra_scale) if inf else abs(extra_scale) ** norm_type)
        per_group[("extra", id(extra_group))] = (extra_group, part)
    if not per_group:
        return torch.zeros(())
    total = None
    for group, part in per_group.values():
        if group is not None:
            dist.all_reduce(part, op=dist.ReduceOp.MAX if inf else dist.ReduceOp.SUM, group=group)
        total = part if total is None else (torch.maximum(total, part) if inf else total + part)
    norm = total if inf else total.pow(1.0 / norm_type)
    if error_if_nonfinite and not torch.isfinite(norm):
        raise RuntimeError(f"The total norm of order {norm_type} for the gradients is non-finite.")
    coef = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for g in (*shards, *extra):
        g.mul_(coef.to(device=g.device, dtype=g.dtype))
    return norm


@torch.no_grad()
def gather_full_grads(module_or_units) -> dict[str, torch.Tensor]:
    """Full (unsharded) reduced gradients keyed by parameter name, assembled on every rank.

    Call it after ``backward()`` and before ``optimizer.step()`` / ``zero_grad()``.  Every rank holds one
    piece of each gradient (its part of the unit's reduced shard); the pieces are placed at their offsets in
    a zero tensor of the parameter's size and summed over the unit's shard group.  Collective: every rank of
    the group has to call it.  A debugging / verification aid (one all-reduce per parameter); the reference's
    bench does the same comparison against FSDP2 (test/fsdp/bench_fsdp2_compare.py:1533-1597).
    """
    import torch.distributed as dist

    from ..parallel.unit_collection import collect_param_groups

    units = collect_param_groups(module_or_units)
    names: dict[int, str] = {}
    if isinstance(module_or_units, torch.nn.Module):
        names = {id(p): n for n, p in module_or_units.named_parameters(remove_duplicate=False)}
    out: dict[str, torch.Tensor] = {}
    for ui, u in enumerate(units):
        u.wait_post_backward_reduce()
        fb = u.flat_buffer
        shard = fb.local_grad_shard if fb.local_grad_valid else None
        group = u.groups.shard_group if u.world_size > 1 else None
        for mp in u.registry:
            full = torch.zeros(mp.numel, dtype=torch.float32, device=fb.device)
            piece = fb.pieces.get(mp.fqn)
            if shard is not None and piece is not None:
                full[piece.param_start:piece.param_start + piece.numel] = \
                    shard[piece.local_start:piece.local_end].to(torch.float32)
            if group is not None:
                dist.all_reduce(full, group=group)
            out[names.get(id(mp.param), f"unit{ui}.{mp.fqn}")] = full.view(mp.shape)
    return out
