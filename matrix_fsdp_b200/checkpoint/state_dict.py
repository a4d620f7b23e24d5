"""Sharded checkpoints in the ``matrix_dcp`` format, with FQN-addressed resharding.

On disk (one directory), the layout the reference package writes and reads:

* tensors through ``torch.distributed.checkpoint`` under keys
  ``"{rank_R|shard_S}.unit_{i}.param_shard"`` (the rank's whole packed local shard),
  ``….grad_shard``, ``….full_param.{fqn}`` / ``….full_grad.{fqn}`` (debug ``full_state``) and
  ``"{payload}.unit_0.optimizer.{component}.{module_fqn.param_fqn}.{state}"`` for optimizer tensors
  (0-d ones such as ``step`` included); with HSDP and ``dedup_replicates`` only replica 0 writes and
  the prefix is ``shard_S``;
* one ``matrix_metadata.pt``: ``{"metadata": {"format": "matrix_dcp_global_metadata", "version": 1,
  "num_ranks", "ranks"}, "ranks": {rank: per-rank metadata}}``; legacy per-rank
  ``matrix_metadata_rank_{r}.pt`` sidecars are still read;
* per-rank metadata: ``{"metadata": {"version", "dcp_format_version", "state_dict_type", "dcp_rank", …},
  "param_groups": [unit…], "units": [same list], "optimizer": {…}}``; every unit names its tensors
  (``param_shard_key``, ``grad_shard_key``, ``full_param_keys``) and describes its layout with the
  reference's field names and value shapes (segments as dictionaries, ``matrix_shard`` as
  ``{dims, local_units}``); optimizer state is ``components → state → {fqn, entries{name → {kind, key,
  shape, dtype} | {kind: "value", value}}}``.  Fields this package adds (``pieces``, ``local_piece``,
  ``piece``, ``shard_dtype`` …) sit beside them and are ignored by the reference's loader, which
  validates only the fields it finds and knows.

So a checkpoint written here loads in the reference (same layout) and the other way round; the
loaders below never rely on the added fields being present.

Same-layout loads validate every structural field *before* touching tensors and then read straight
into ``local_shard`` and freshly bound optimizer state.  ``allow_reshard=True`` loads onto any world
size or layout: every parameter piece a rank owns is assembled from the source pieces that overlap
it, addressed by (unit, fqn, offset-in-parameter) — derived from every source rank's per-parameter
``local_segments`` — so matrix-owner layouts, whose flat order depends on the world size, reshard
bit-exactly.  The reference instead concatenates all source shards on every rank and requires
identical flat order (``matrix_fsdp/checkpoint/state_dict.py:879-950,1309-1327``).

Parity: ``matrix_fsdp/checkpoint/state_dict.py:65-1397``, ``_dcp_utils.py``, ``_metadata.py``,
``_optimizer_utils.py``.
"""
from __future__ import annotations

import os
from collections.abc import Mapping
from copy import deepcopy
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ..core.mixed_precision import mixed_precision_policy_metadata, offload_policy_metadata
from ..parallel.unit_collection import collect_param_groups

GLOBAL_METADATA_FILE = "matrix_metadata.pt"
GLOBAL_METADATA_FORMAT = "matrix_dcp_global_metadata"
MATRIX_STATE_DICT_VERSION = 1
MATRIX_DCP_FORMAT_VERSION = 1
OPTIMIZER_FORMAT_VERSION = 2


# --------------------------------------------------------------------------- helpers
def _units(model_or_units):
    units = collect_param_groups(model_or_units)
    if not units:
        raise ValueError("Expected a module wrapped by fully_shard().")
    return units


def _unit_refs(model_or_units) -> list[tuple[str, Any]]:
    """(module path, unit) pairs in unit order; the path is how full parameter names are built
    (``{module_fqn}.{param_fqn}``).  Without a root module the path is ``unit{i}``."""
    units = _units(model_or_units)
    if isinstance(model_or_units, torch.nn.Module):
        paths = {id(m): name for name, m in model_or_units.named_modules(remove_duplicate=True)}
        return [(paths.get(id(u.module), f"unit{i}"), u) for i, u in enumerate(units)]
    if len(units) == 1 and not isinstance(model_or_units, (list, tuple)):
        return [("", units[0])]
    return [(f"unit{i}", u) for i, u in enumerate(units)]


def param_key(module_fqn: str, param_fqn: str, unit_index: int) -> str:
    if module_fqn:
        return f"{module_fqn}.{param_fqn}"
    return param_fqn or f"unit{unit_index}"


def _dist_on(no_dist: bool | None) -> bool:
    if no_dist is not None:
        return not no_dist
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _global_rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def dcp_payload_prefix(unit, *, dedup_replicates: bool) -> str:
    """``shard_S`` when HSDP replicas are de-duplicated, else ``rank_R`` (R = global rank)."""
    if unit.replicate_world_size > 1 and dedup_replicates:
        return f"shard_{unit.rank}"
    return f"rank_{_global_rank()}"


def _writes_payload(unit, *, dedup_replicates: bool) -> bool:
    return not (unit.replicate_world_size > 1 and dedup_replicates and unit.replicate_rank != 0)


def iter_optimizer_components(optimizer):
    """(component name, torch-like optimizer) pairs: ``optimizer`` or ``muon`` / ``adamw``."""
    if optimizer is None:
        return []
    if hasattr(optimizer, "iter_named_optimizers"):
        return list(optimizer.iter_named_optimizers())
    return [("optimizer", optimizer)]


def _optimizer_kind(optimizer) -> str:
    names = [n for n, _ in iter_optimizer_components(optimizer)]
    return "mixed_muon_adamw" if set(names) == {"muon", "adamw"} else "single"


def _canonical(value: Any) -> Any:
    if isinstance(value, Mapping):
        return {k: _canonical(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return tuple(_canonical(v) for v in value)
    return value


def _plain(value: Any) -> Any:
    """Metadata as plain containers and scalars only, so ``torch.load(weights_only=True)`` reads the file."""
    import dataclasses
    import enum

    if dataclasses.is_dataclass(value) and not isinstance(value, type):
        return _plain(dataclasses.asdict(value))
    if isinstance(value, enum.Enum):
        return _plain(value.value)
    if isinstance(value, Mapping):
        return {(_plain(k) if not isinstance(k, (str, int)) else k): _plain(v) for k, v in value.items()}
    if isinstance(value, torch.Size):
        return tuple(int(x) for x in value)
    if isinstance(value, tuple):
        return tuple(_plain(v) for v in value)
    if isinstance(value, (list, set, frozenset)):
        return [_plain(v) for v in value]
    if isinstance(value, (torch.dtype, torch.device)):
        return str(value)
    if value is None or isinstance(value, (bool, int, float, str, bytes)) or torch.is_tensor(value):
        return value
    return repr(value)


def _seg3(seg) -> tuple[int, int, int]:
    """(global_start, global_end, local_start) of a saved segment in either notation."""
    if isinstance(seg, Mapping):
        return int(seg["global_start"]), int(seg["global_end"]), int(seg["local_start"])
    return int(seg[0]), int(seg[1]), int(seg[2])


def _dtype_from_string(name: str) -> torch.dtype:
    dt = getattr(torch, str(name).replace("torch.", ""), None)
    if not isinstance(dt, torch.dtype):
        raise ValueError(f"Unknown dtype {name!r} in checkpoint metadata.")
    return dt


# --------------------------------------------------------------------------- metadata
def _segment_metadata(s) -> dict[str, int]:
    return {"global_start": s.global_start, "global_end": s.global_end, "local_start": s.local_start,
            "local_end": s.local_start + s.numel, "numel": s.numel}


def _matrix_shard_metadata(placement) -> dict[str, Any] | None:
    if placement is None:
        return None
    return {"dims": tuple(placement.dims), "local_units": tuple(placement.local_units)}


def _param_metadata(unit, mp) -> dict[str, Any]:
    layout, fb = unit.layout, unit.flat_buffer
    pl = layout.param(mp.fqn)
    piece = fb.pieces.get(mp.fqn)
    per_rank = [0] * unit.world_size
    for s in pl.segments:
        per_rank[s.rank] += s.numel
    hint = mp.shard_hint
    return {
        "fqn": mp.fqn, "shape": tuple(mp.shape), "dtype": str(mp.dtype), "device": str(mp.device),
        "numel": mp.numel, "offset": mp.offset, "end": mp.end, "owner_ranks": tuple(layout.owner_ranks(mp.fqn)),
        "local_segments": [
            {"fqn": mp.fqn, "rank": unit.rank, **_segment_metadata(s)}
            for s in layout.rank_segments_for_param(unit.rank, mp.fqn)],
        "shard_sizes": tuple(per_rank),
        "shard_hint": {
            "optimizer_type": hint.optimizer_type, "split_granularity": hint.split_granularity,
            "block_shape": hint.block_shape, "runtime_kind": hint.runtime_kind, "parallel_role": hint.parallel_role,
            "expert_id": hint.expert_id, "expert_group_id": hint.expert_group_id, "owner_rank": hint.owner_rank,
            "owner_replica_ranks": tuple(hint.owner_replica_ranks)},
        # added by this package: every rank's pieces of the parameter, and this rank's own one
        "pieces": tuple((s.rank, s.global_start - mp.offset, s.numel, s.local_start) for s in pl.segments),
        "local_piece": None if piece is None else (piece.param_start, piece.numel, piece.local_start),
        "aliases": tuple(mp.aliases),
    }


def _unit_state_dict(unit, index: int, *, clone: bool, include_grads: bool, dedup_replicates: bool,
                     module_fqn: str | None = None) -> dict[str, Any]:
    fb, res = unit.flat_buffer, unit.planner_result
    segs = fb.tables.my_segments
    meta = res.as_metadata()
    d: dict[str, Any] = {
        "param_group_index": index, "unit_index": index,
        "module_fqn": f"unit{index}" if module_fqn is None else module_fqn, "name": unit.name,
        "runtime_param_group_id": str(unit.metadata.runtime_param_group_id),
        "rank": unit.rank, "world_size": unit.world_size, "replicate_rank": unit.replicate_rank,
        "replicate_world_size": unit.replicate_world_size,
        "device_mesh": unit.groups.metadata.as_dict() if unit.groups.metadata is not None else None,
        "mixed_precision": mixed_precision_policy_metadata(unit.mp_policy),
        "offload_policy": offload_policy_metadata(unit.offload_policy),
        "total_numel": fb.total_numel, "local_numel": fb.local_numel,
        "local_segments": [_segment_metadata(s) for s in segs],
        "shard_sizes": tuple(unit.layout.shard_sizes), "matrix_shard": _matrix_shard_metadata(fb.matrix_shard),
        "planner_name": res.name, "planner_policy": res.policy, "runtime_layout_mode": unit.runtime_mode,
        "runtime_layout_policy": unit.runtime_layout_policy,
        "planner_metadata": {"layout_contract": meta["layout_contract"], "report": meta["report"],
                             "resource_estimate": meta["resource_estimate"],
                             "expert_owner_groups": meta["expert_owner_groups"], "warnings": meta["warnings"]},
        "param_gather_strategy": unit.param_gather_strategy,
        "matrix_collective_backend": unit.matrix_collective_backend,
        "grad_reduce_strategy": unit.backward_reduce_strategy,
        "shard_dtype": str(fb.shard_dtype), "param_dtype": str(fb.param_dtype),
        "param_fqns": tuple(unit.registry.fqns),
        "params": {mp.fqn: _param_metadata(unit, mp) for mp in unit.registry},
        "dcp_payload_rank": dcp_payload_prefix(unit, dedup_replicates=dedup_replicates),
        "dcp_dedup_replicates": bool(dedup_replicates and unit.replicate_world_size > 1),
        "param_shard": fb.local_shard.detach().clone() if clone else fb.local_shard.detach(),
    }
    if len(segs) == 1:
        # a rank-contiguous shard also has a [start, end) in the flat space
        d["local_start"], d["local_end"] = segs[0].global_start, segs[0].global_end
    if include_grads and fb.local_grad_shard is not None and fb.local_grad_valid:
        g = fb.local_grad_shard.detach()
        d["grad_shard"] = g.clone() if clone else g
    return d


def matrix_state_dict(model_or_units, *, clone: bool = True, include_grads: bool = False,
                      dedup_replicates: bool = True) -> dict[str, Any]:
    """In-memory sharded state: the per-unit dictionaries (with their ``param_shard`` tensors) under
    ``param_groups`` (and its older name ``units``)."""
    refs = _unit_refs(model_or_units)
    units = [_unit_state_dict(u, i, clone=clone, include_grads=include_grads, dedup_replicates=dedup_replicates,
                              module_fqn=path) for i, (path, u) in enumerate(refs)]
    return {"metadata": {"version": MATRIX_STATE_DICT_VERSION, "state_dict_type": "matrix_sharded",
                         "num_param_groups": len(units), "num_units": len(units), "include_grads": include_grads},
            "param_groups": units, "units": units, "dcp_rank": _global_rank()}


def _unit_list(state: Mapping[str, Any], what: str) -> list[dict[str, Any]]:
    units = state.get("param_groups")
    if units is None:
        units = state.get("units")
    if not isinstance(units, list):
        raise TypeError(f"MatrixFSDP {what} must contain a list at key 'param_groups' or legacy key 'units'.")
    return units


_UNIT_FIELDS = ("rank", "world_size", "replicate_world_size", "total_numel", "local_numel", "local_start", "local_end",
                "shard_sizes", "matrix_shard", "shard_dtype")
_PARAM_FIELDS = ("shape", "dtype", "numel", "offset", "end", "owner_ranks", "shard_sizes")


def _validate_same_layout_unit(saved: Mapping[str, Any], unit, index: int, module_fqn: str | None = None) -> None:
    """Every structural field the checkpoint carries has to equal the model's (fields it does not carry
    are not checked, so checkpoints of writers that know fewer fields still load)."""
    current = _unit_state_dict(unit, index, clone=False, include_grads=False, dedup_replicates=True,
                               module_fqn=module_fqn)

    def differ(name, a, b):
        raise ValueError(f"Checkpoint unit {index} field {name!r} does not match the model: saved {a!r}, "
                         f"current {b!r}. Pass allow_reshard=True to load onto a different layout.")

    if tuple(saved.get("param_fqns", ())) != tuple(current["param_fqns"]):
        differ("param_fqns", tuple(saved.get("param_fqns", ())), current["param_fqns"])
    if module_fqn is not None and "module_fqn" in saved and \
            saved["module_fqn"] not in (module_fqn, f"unit{saved.get('unit_index', index)}"):
        differ("module_fqn", saved["module_fqn"], module_fqn)
    for name in _UNIT_FIELDS:
        if name in saved and _canonical(saved[name]) != _canonical(current.get(name)):
            differ(name, saved[name], current.get(name))
    if "local_segments" in saved:
        a = tuple(_seg3(s) for s in saved["local_segments"])
        b = tuple(_seg3(s) for s in current["local_segments"])
        if a != b:
            differ("local_segments", a, b)
    mesh_keys = ("ndim", "shape", "mesh_dim_names", "coordinate", "shard_mesh_dim", "shard_mesh_size",
                 "replicate_mesh_dim", "replicate_mesh_size")
    if "device_mesh" in saved:
        sm, cm = saved["device_mesh"], current["device_mesh"]
        if (sm is None) != (cm is None) or (sm is not None and any(
                _canonical(sm.get(k)) != _canonical(cm.get(k)) for k in mesh_keys)):
            differ("device_mesh", sm, cm)
    saved_params = saved.get("params")
    if saved_params is None:
        return
    for fqn, pm in saved_params.items():
        cur = current["params"].get(fqn)
        if cur is None:
            raise ValueError(f"Checkpoint unit {index} has unknown parameter {fqn!r}.")
        for name in _PARAM_FIELDS:
            if name in pm and _canonical(pm[name]) != _canonical(cur[name]):
                raise ValueError(f"Checkpoint unit {index} parameter {fqn!r} field {name!r} does not match the model: "
                                 f"saved {pm[name]!r}, current {cur[name]!r}.")
        if "local_segments" in pm and tuple(_seg3(s) for s in pm["local_segments"]) != \
                tuple(_seg3(s) for s in cur["local_segments"]):
            raise ValueError(f"Checkpoint unit {index} parameter {fqn!r} field 'local_segments' does not match the model.")


def load_matrix_state_dict(model_or_units, state: Mapping[str, Any], *, strict: bool = True) -> None:
    """Load an in-memory ``matrix_state_dict`` produced on the same layout."""
    refs = _unit_refs(model_or_units)
    saved_units = _unit_list(state, "state dict")
    if len(saved_units) != len(refs):
        raise ValueError(f"State dict has {len(saved_units)} units, the model has {len(refs)}.")
    for i, ((path, u), su) in enumerate(zip(refs, saved_units)):
        if strict:
            _validate_same_layout_unit(su, u, i, path)
    with torch.no_grad():
        for (_, u), su in zip(refs, saved_units):
            u.discard_unused_prefetch()
            u.flat_buffer.local_shard.copy_(su["param_shard"])
            u.flat_buffer.mark_master_updated(lp_written=False)
            if torch.is_tensor(su.get("grad_shard")):
                u.flat_buffer._ensure_local_grad_shard().copy_(su["grad_shard"])
                u.flat_buffer.local_grad_valid = True
                u.flat_buffer.use_local_grad_shard()


# --------------------------------------------------------------------------- optimizer state
def _state_ids(opt) -> dict[int, int]:
    """id(parameter) → the integer torch's ``state_dict()`` names it by (position over all groups)."""
    out, n = {}, 0
    for g in getattr(opt, "param_groups", []):
        for p in g["params"]:
            out.setdefault(id(p), n)
            n += 1
    return out


def _plain_param_groups(opt) -> list[dict[str, Any]]:
    """``state_dict()["param_groups"]`` without touching the state: hyper-parameters plus parameter ids."""
    ids = _state_ids(opt)
    groups = []
    for g in getattr(opt, "param_groups", []):
        d = {k: deepcopy(v) for k, v in g.items() if k != "params" and not torch.is_tensor(v)}
        d["params"] = [ids[id(p)] for p in g["params"]]
        groups.append(d)
    return groups


def _collect_optimizer_state(refs, optimizer, payload_of) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
    """→ (tensor entries keyed for DCP, metadata describing every state entry)."""
    from ..core.state import matrix_shard_metadata

    tensors: dict[str, torch.Tensor] = {}
    meta: dict[str, Any] = {"optimizer_format_version": OPTIMIZER_FORMAT_VERSION, "kind": _optimizer_kind(optimizer),
                            "components": {}}
    summary = getattr(optimizer, "optimizer_group_summary", None)
    if callable(summary):
        try:
            meta["group_summary"] = _canonical(summary())
        except Exception:  # noqa: BLE001  (a summary is a convenience, never a reason to fail a save)
            meta["group_summary"] = None
    where = {id(mp.param): (ui, path, u, mp) for ui, (path, u) in enumerate(refs) for mp in u.registry}
    for comp, opt in iter_optimizer_components(optimizer):
        ids = _state_ids(opt)
        state_meta: dict[int, dict[str, Any]] = {}
        for p, st in getattr(opt, "state", {}).items():
            hit = where.get(id(p))
            if hit is None or id(p) not in ids:
                continue
            ui, path, u, mp = hit
            piece = u.flat_buffer.pieces.get(mp.fqn)
            if piece is None:
                continue                       # nothing of this parameter lives on this rank
            full_fqn = param_key(path, mp.fqn, ui)
            entries: dict[str, Any] = {}
            for name, val in st.items():
                if torch.is_tensor(val):
                    key = f"{payload_of(u)}.unit_0.optimizer.{comp}.{full_fqn}.{name}"
                    val = val.detach()
                    if val.dim() > 1 and val.numel() == piece.numel and piece.numel != mp.numel:
                        val = val.reshape(-1)       # a part of a parameter is stored flat, a whole one in its shape
                    tensors[key] = val
                    e = {"kind": "tensor", "key": key, "shape": tuple(val.shape), "dtype": str(val.dtype),
                         "requires_grad": bool(val.requires_grad)}
                    if val.dim() > 0 and val.numel() == piece.numel:
                        e["piece"] = (piece.param_start, piece.numel)
                        e["matrix_state"] = matrix_shard_metadata(u.flat_buffer.matrix_shard)
                    entries[name] = e
                else:
                    entries[name] = {"kind": "value", "value": deepcopy(val)}
            state_meta[ids[id(p)]] = {"fqn": full_fqn, "entries": entries, "unit_index": ui, "param_fqn": mp.fqn}
        meta["components"][comp] = {"class_name": type(opt).__name__, "param_groups": _plain_param_groups(opt),
                                    "state": state_meta}
    comps = meta["components"]
    if list(comps) == ["optimizer"]:
        meta["param_groups"] = deepcopy(comps["optimizer"]["param_groups"])
        meta["state"] = comps["optimizer"]["state"]
    return tensors, meta


def _optimizer_components_metadata(opt_meta: Mapping[str, Any]) -> dict[str, Any]:
    """Components of saved optimizer metadata; the single-optimizer form without ``components`` included."""
    if "components" in opt_meta:
        return opt_meta["components"]
    return {"optimizer": {"param_groups": opt_meta.get("param_groups", []), "state": opt_meta.get("state", {})}}


def _check_components(saved_meta: Mapping[str, Any], optimizer) -> None:
    have = {n for n, _ in iter_optimizer_components(optimizer)}
    saved = set(_optimizer_components_metadata(saved_meta))
    if saved - have:
        raise ValueError(f"Checkpoint has unknown component(s) for this optimizer: {sorted(saved - have)}")
    if have - saved:
        raise ValueError(f"Checkpoint is missing component(s) of this optimizer: {sorted(have - saved)}")


def _bind_optimizer_state(opt, p, name: str, value: torch.Tensor) -> None:
    """Put a loaded state tensor where the optimizer expects it (flat views are copied into)."""
    st = opt.state[p] if hasattr(opt.state, "__getitem__") else None
    if st is None:
        return
    cur = st.get(name)
    if isinstance(cur, torch.Tensor) and cur.numel() == value.numel():
        cur.copy_(value.view(cur.shape))
    else:
        st[name] = value.view(p.shape if value.numel() == p.numel() and value.dim() > 0 else value.shape).clone()


def _hyper_of(saved_group: Mapping[str, Any]) -> dict[str, Any]:
    if "hyper" in saved_group:                         # files written before the key scheme followed the reference
        return dict(saved_group["hyper"])
    return {k: v for k, v in saved_group.items() if k != "params"}


def _restore_optimizer(staged, saved_meta, optimizer) -> None:
    """``staged``: (component optimizer, parameter, state name, tensor) and (…, None, {name: plain value})."""
    if optimizer is None:
        return
    for opt, p, name, value in staged:
        if not hasattr(opt, "state"):
            continue
        if name is None:
            st = opt.state[p]
            for k, v in value.items():
                cur = st.get(k)
                if isinstance(cur, torch.Tensor):
                    cur.fill_(float(v)) if cur.numel() == 1 else cur.copy_(torch.as_tensor(v))
                else:
                    st[k] = torch.tensor(float(v)) if k == "step" else v
        elif value.dim() == 0:
            st = opt.state[p]
            cur = st.get(name)
            if isinstance(cur, torch.Tensor) and cur.numel() == 1:
                cur.fill_(float(value))
            else:
                st[name] = value.detach().clone().cpu() if name == "step" else value.detach().clone()
        else:
            _bind_optimizer_state(opt, p, name, value)
    comps = dict(iter_optimizer_components(optimizer))
    for comp, cmeta in _optimizer_components_metadata(saved_meta or {}).items():
        opt = comps.get(comp)
        if opt is None:
            continue
        for g, sg in zip(getattr(opt, "param_groups", []), cmeta.get("param_groups", [])):
            for k, v in _hyper_of(sg).items():
                g[k] = tuple(v) if isinstance(g.get(k), tuple) and isinstance(v, list) else v
        # flat optimizers keep a per-unit step counter next to the per-param entries
        rebind = getattr(opt, "_unit_states", None)
        if rebind:
            for us in rebind.values():
                steps = [float(opt.state[mp.param]["step"]) for mp in us.unit.registry
                         if mp.param in opt.state and "step" in opt.state[mp.param]]
                if steps:
                    us.step = int(max(steps))


def _split_entries(entry: Mapping[str, Any]) -> tuple[dict[str, Any], dict[str, Any]]:
    """(tensor entries, plain values) of one saved state entry."""
    tensors, values = {}, {}
    for name, e in entry.get("entries", {}).items():
        if e.get("kind") == "tensor":
            tensors[name] = e
        else:
            values[name] = e.get("value")
    return tensors, values


# --------------------------------------------------------------------------- global metadata file
def _write_global_metadata(directory: str, rank_metadata: dict[str, Any], *, use_dist: bool, group=None) -> None:
    rank_metadata = _plain(rank_metadata)
    my_rank = rank_metadata["metadata"]["dcp_rank"]
    if use_dist:
        gathered: list = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, rank_metadata, group=group)
        ranks = {m["metadata"]["dcp_rank"]: m for m in gathered}
    else:
        ranks = {my_rank: rank_metadata}
    if not use_dist or dist.get_rank(group) == 0:
        os.makedirs(directory, exist_ok=True)
        payload = {"metadata": {"format": GLOBAL_METADATA_FORMAT, "version": 1, "num_ranks": len(ranks),
                                "ranks": tuple(sorted(ranks))}, "ranks": ranks}
        torch.save(payload, os.path.join(directory, GLOBAL_METADATA_FILE))
    if use_dist:
        dist.barrier(group=group)


def read_global_metadata(directory: str) -> dict[str, Any]:
    path = os.path.join(directory, GLOBAL_METADATA_FILE)
    if os.path.exists(path):
        payload = torch.load(path, map_location="cpu", weights_only=False)
        if payload.get("metadata", {}).get("format") != GLOBAL_METADATA_FORMAT:
            raise ValueError(f"{path} is not a matrix_dcp metadata file.")
        return payload
    # legacy layout: one sidecar per rank
    ranks = {}
    for name in sorted(os.listdir(directory)) if os.path.isdir(directory) else []:
        if name.startswith("matrix_metadata_rank_") and name.endswith(".pt"):
            r = int(name[len("matrix_metadata_rank_"):-3])
            ranks[r] = torch.load(os.path.join(directory, name), map_location="cpu", weights_only=False)
    if not ranks:
        raise FileNotFoundError(f"No {GLOBAL_METADATA_FILE} (or legacy per-rank sidecars) under {directory}.")
    return {"metadata": {"format": GLOBAL_METADATA_FORMAT, "version": 1, "num_ranks": len(ranks),
                         "ranks": tuple(sorted(ranks))}, "ranks": ranks}


def _check_envelope(meta: Mapping[str, Any], *, expect_rank: int | None) -> None:
    env = meta.get("metadata")
    if not isinstance(env, Mapping):
        return                                  # files from before the envelope existed
    if env.get("version") != MATRIX_STATE_DICT_VERSION:
        raise ValueError(f"Unsupported MatrixFSDP state_dict version {env.get('version')!r}; "
                         f"expected {MATRIX_STATE_DICT_VERSION}.")
    if "dcp_format_version" in env and env["dcp_format_version"] != MATRIX_DCP_FORMAT_VERSION:
        raise ValueError(f"Unsupported MatrixFSDP DCP format version {env['dcp_format_version']!r}; "
                         f"expected {MATRIX_DCP_FORMAT_VERSION}.")
    if expect_rank is not None and "dcp_rank" in env and env["dcp_rank"] != expect_rank:
        raise ValueError(f"Loaded metadata for DCP rank {env['dcp_rank']}, but current DCP rank is {expect_rank}.")


# --------------------------------------------------------------------------- save
def _full_master_params(units) -> dict[int, torch.Tensor]:
    """``id(parameter) -> full tensor`` assembled from the master shards, for units whose compute copy has a lower
    precision than the master (the unsharded parameters of such a unit are the rounded copy).  Collective."""
    import torch.distributed as dist

    out: dict[int, torch.Tensor] = {}
    for u in units:
        fb = u.flat_buffer
        if not fb.mixed:
            continue
        group = u.groups.shard_group if u.world_size > 1 else None
        for mp in u.registry:
            full = torch.zeros(mp.numel, dtype=fb.local_shard.dtype, device=fb.device)
            piece = fb.pieces.get(mp.fqn)
            if piece is not None:
                full[piece.param_start:piece.param_start + piece.numel] = fb.local_shard[piece.local_start:piece.local_end]
            if group is not None:
                dist.all_reduce(full, group=group)          # every element has one owner: the sum places the pieces
            out[id(mp.param)] = full.view(mp.shape)
    return out


def save_matrix_dcp(model_or_units, directory: str, optimizer=None, *, full_state: bool = False,
                    include_grads: bool = False, dedup_replicates: bool = True, process_group=None,
                    no_dist: bool | None = None) -> dict[str, Any]:
    refs = _unit_refs(model_or_units)
    units = [u for _, u in refs]
    use_dist = _dist_on(no_dist)
    dcp_rank = (dist.get_rank(process_group) if use_dist else 0)
    state = matrix_state_dict(model_or_units, clone=False, include_grads=include_grads,
                              dedup_replicates=dedup_replicates)
    unit_meta = state["param_groups"]
    tensors: dict[str, torch.Tensor] = {}
    for i, (u, us) in enumerate(zip(units, unit_meta)):
        prefix = f"{us['dcp_payload_rank']}.unit_{i}"
        writes = _writes_payload(u, dedup_replicates=dedup_replicates)
        shard = us.pop("param_shard")
        grad = us.pop("grad_shard", None)
        us["param_shard_key"] = f"{prefix}.param_shard"
        us["grad_shard_key"] = f"{prefix}.grad_shard" if grad is not None else None
        us["full_param_keys"], us["full_grad_keys"] = {}, {}
        if writes:
            tensors[us["param_shard_key"]] = shard
            if grad is not None:
                tensors[us["grad_shard_key"]] = grad
    if full_state:
        for i, (u, us) in enumerate(zip(units, unit_meta)):
            prefix = f"{us['dcp_payload_rank']}.unit_{i}"
            masters = _full_master_params([u])           # mixed precision: the masters, not the rounded compute copy
            if masters:
                us["full_param_dtype"] = str(u.flat_buffer.local_shard.dtype)
            u.unshard("checkpoint_full_state")
            for mp in u.registry:
                us["full_param_keys"][mp.fqn] = f"{prefix}.full_param.{mp.fqn}"
                if dcp_rank == 0 or not use_dist:
                    whole = masters.get(id(mp.param))
                    tensors[us["full_param_keys"][mp.fqn]] = whole if whole is not None else mp.param.detach().clone()
            u.reshard("checkpoint_full_state")
    opt_meta = None
    if optimizer is not None:
        payload_of = {id(u): us["dcp_payload_rank"] for u, us in zip(units, unit_meta)}
        writers = {id(u) for u in units if _writes_payload(u, dedup_replicates=dedup_replicates)}
        unit_of_key: dict[str, int] = {}
        opt_tensors, opt_meta = _collect_optimizer_state(refs, optimizer, lambda u: payload_of[id(u)])
        for cm in opt_meta["components"].values():
            for entry in cm["state"].values():
                for e in entry["entries"].values():
                    if e["kind"] == "tensor":
                        unit_of_key[e["key"]] = entry["unit_index"]
        for k, v in opt_tensors.items():
            if id(units[unit_of_key[k]]) in writers:
                tensors[k] = v
    rank_meta = {
        "metadata": {"version": MATRIX_STATE_DICT_VERSION, "dcp_format_version": MATRIX_DCP_FORMAT_VERSION,
                     "state_dict_type": "matrix_dcp_sharded", "num_param_groups": len(unit_meta),
                     "num_units": len(unit_meta), "full_state": bool(full_state), "include_grads": bool(include_grads),
                     "dedup_replicates": bool(dedup_replicates), "dcp_rank": dcp_rank},
        "param_groups": unit_meta, "units": unit_meta, "optimizer": opt_meta,
        # kept at the top level as well for readers that look there
        "dcp_rank": dcp_rank, "full_state": bool(full_state),
    }
    _write_global_metadata(directory, rank_meta, use_dist=use_dist, group=process_group)
    dcp.save(tensors, checkpoint_id=directory, process_group=process_group if use_dist else None,
             no_dist=not use_dist)
    return rank_meta


# --------------------------------------------------------------------------- load
def _dcp_load(tensors: dict[str, torch.Tensor], directory: str, *, use_dist: bool, group=None) -> None:
    if tensors or use_dist:
        dcp.load(tensors, checkpoint_id=directory, process_group=group if use_dist else None, no_dist=not use_dist)


def _my_metadata(payload: dict[str, Any], rank: int) -> dict[str, Any]:
    ranks = payload["ranks"]
    if rank not in ranks:
        raise ValueError(f"Checkpoint holds ranks {sorted(ranks)}; rank {rank} is missing "
                         "(pass allow_reshard=True to load on a different world size).")
    return ranks[rank]


def _current_param_index(refs) -> dict[str, tuple[int, Any, Any]]:
    """full parameter name → (unit index, unit, managed parameter) of the model being loaded."""
    return {param_key(path, mp.fqn, ui): (ui, u, mp) for ui, (path, u) in enumerate(refs) for mp in u.registry}


def _locate(entry: Mapping[str, Any], index: Mapping[str, tuple], units) -> tuple[int, Any, Any] | None:
    hit = index.get(entry.get("fqn"))
    if hit is None and "unit_index" in entry and "param_fqn" in entry and entry["unit_index"] < len(units):
        u = units[entry["unit_index"]]
        if entry["param_fqn"] in u.registry.fqns:
            hit = (entry["unit_index"], u, u.registry.param(entry["param_fqn"]))
    return hit


def load_matrix_dcp(model_or_units, directory: str, optimizer=None, *, allow_reshard: bool = False,
                    include_grads: bool = False, process_group=None, no_dist: bool | None = None,
                    dedup_replicates: bool = True) -> dict[str, Any]:
    refs = _unit_refs(model_or_units)
    units = [u for _, u in refs]
    use_dist = _dist_on(no_dist)
    payload = read_global_metadata(directory)
    for u in units:
        u.discard_unused_prefetch()            # a gather issued for the next step would deliver the old values
    if allow_reshard:
        return _load_resharded(refs, directory, payload, optimizer, use_dist=use_dist, group=process_group)
    dcp_rank = dist.get_rank(process_group) if use_dist else _global_rank()
    meta = _my_metadata(payload, dcp_rank)
    _check_envelope(meta, expect_rank=dcp_rank)
    saved_units = _unit_list(meta, "DCP metadata")
    if len(saved_units) != len(units):
        raise ValueError(f"Checkpoint has {len(saved_units)} units, the model has {len(units)}.")
    for i, ((path, u), su) in enumerate(zip(refs, saved_units)):
        _validate_same_layout_unit(su, u, i, path)
    if optimizer is not None:
        if meta.get("optimizer") is None:
            raise ValueError("Checkpoint holds no optimizer state.")
        _check_components(meta["optimizer"], optimizer)
    tensors: dict[str, torch.Tensor] = {}
    for i, (u, su) in enumerate(zip(units, saved_units)):
        prefix = f"{su.get('dcp_payload_rank', f'rank_{dcp_rank}')}.unit_{i}"
        tensors[su.get("param_shard_key", f"{prefix}.param_shard")] = u.flat_buffer.local_shard
        if include_grads and su.get("grad_shard_key"):
            tensors[su["grad_shard_key"]] = u.flat_buffer._ensure_local_grad_shard()
    staged: list[tuple] = []
    if optimizer is not None:
        comps = dict(iter_optimizer_components(optimizer))
        index = _current_param_index(refs)
        for comp, cmeta in _optimizer_components_metadata(meta["optimizer"]).items():
            for entry in cmeta["state"].values():
                hit = _locate(entry, index, units)
                if hit is None:
                    raise ValueError(f"Optimizer component {comp!r} references unknown local parameter {entry.get('fqn')!r}.")
                _, u, mp = hit
                tens, values = _split_entries(entry)
                for name, e in tens.items():
                    buf = torch.empty(tuple(e["shape"]), dtype=_dtype_from_string(e["dtype"]),
                                      device=u.flat_buffer.device if len(e["shape"]) else "cpu")
                    tensors[e["key"]] = buf
                    staged.append((comps[comp], mp.param, name, buf))
                if values:
                    staged.append((comps[comp], mp.param, None, values))
    with torch.no_grad():
        _dcp_load(tensors, directory, use_dist=use_dist, group=process_group)
        for u, su in zip(units, saved_units):
            u.flat_buffer.mark_master_updated(lp_written=False)
            if include_grads and su.get("grad_shard_key"):
                u.flat_buffer.local_grad_valid = True
                u.flat_buffer.use_local_grad_shard()
        _restore_optimizer(staged, meta.get("optimizer"), optimizer)
    return meta


# --------------------------------------------------------------------------- reshard load
def _overlaps(a0: int, a1: int, b0: int, b1: int) -> tuple[int, int] | None:
    lo, hi = max(a0, b0), min(a1, b1)
    return (lo, hi) if lo < hi else None


def _source_pieces(ranks: Mapping[int, Mapping[str, Any]], unit_index: int, fqn: str) -> list[tuple]:
    """Every saved piece of one parameter: (payload prefix, shard rank, start in the parameter, numel, offset
    in that rank's local shard), one per shard rank (replicas of an HSDP mesh hold the same pieces)."""
    out, seen = [], set()
    for r in sorted(ranks):
        su = _unit_list(ranks[r], "DCP metadata")[unit_index]
        if su["rank"] in seen:
            continue
        seen.add(su["rank"])
        pm = su["params"][fqn]
        for seg in pm.get("local_segments", ()):
            g0, g1, l0 = _seg3(seg)
            if g1 > g0:
                out.append((su.get("dcp_payload_rank", f"rank_{r}"), su["rank"], g0 - int(pm["offset"]), g1 - g0, l0))
    return out


def _load_resharded(refs, directory: str, payload: dict[str, Any], optimizer, *, use_dist: bool, group=None):
    """Assemble every owned parameter piece (and its optimizer tensors) from overlapping source pieces."""
    units = [u for _, u in refs]
    ranks = payload["ranks"]
    any_meta = ranks[sorted(ranks)[0]]
    _check_envelope(any_meta, expect_rank=None)
    saved_units = _unit_list(any_meta, "DCP metadata")
    if len(saved_units) != len(units):
        raise ValueError(f"Checkpoint has {len(saved_units)} units, the model has {len(units)}.")
    for i, (u, su) in enumerate(zip(units, saved_units)):
        if set(su["param_fqns"]) != set(u.registry.fqns):
            raise ValueError(f"Checkpoint unit {i} parameters differ from the model's unit {u.name}.")
        if su["total_numel"] != u.flat_buffer.total_numel:
            raise ValueError(f"Checkpoint unit {i} total_numel={su['total_numel']} differs from the model "
                             f"({u.flat_buffer.total_numel}).")
    if optimizer is not None:
        if any_meta.get("optimizer") is None:
            raise ValueError("Checkpoint holds no optimizer state.")
        _check_components(any_meta["optimizer"], optimizer)

    def shard_dtype(i: int) -> torch.dtype:
        su = saved_units[i]
        if "shard_dtype" in su:
            return _dtype_from_string(su["shard_dtype"])
        return _dtype_from_string(next(iter(su["params"].values()))["dtype"])

    requests: dict[str, torch.Tensor] = {}
    plan: list[tuple] = []    # (dst tensor, dst offset, key, src offset, numel)
    for i, u in enumerate(units):
        fb = u.flat_buffer
        sizes = saved_units[i]["shard_sizes"]
        for fqn, piece in fb.pieces.items():
            for prefix, srank, pstart, n, lstart in _source_pieces(ranks, i, fqn):
                ov = _overlaps(piece.param_start, piece.param_start + piece.numel, pstart, pstart + n)
                if ov is None:
                    continue
                key = f"{prefix}.unit_{i}.param_shard"
                if key not in requests:
                    requests[key] = torch.empty(sizes[srank], dtype=shard_dtype(i), device=fb.device)
                plan.append((fb.local_shard, piece.local_start + (ov[0] - piece.param_start), key,
                             lstart + (ov[0] - pstart), ov[1] - ov[0]))
    staged_opt: list[tuple] = []
    if optimizer is not None:
        index = _current_param_index(refs)
        comps = dict(iter_optimizer_components(optimizer))
        for comp, opt in comps.items():
            owned_ids = {id(p) for g in getattr(opt, "param_groups", []) for p in g["params"]}
            per_param: dict[int, dict] = {}
            seen_sources: set[tuple] = set()
            for r in sorted(ranks):
                om = ranks[r].get("optimizer")
                if om is None:
                    continue
                r_units = _unit_list(ranks[r], "DCP metadata")
                for entry in _optimizer_components_metadata(om).get(comp, {"state": {}})["state"].values():
                    hit = _locate(entry, index, units)
                    if hit is None:
                        continue
                    ui, u, mp = hit
                    piece = u.flat_buffer.pieces.get(mp.fqn)
                    if piece is None or id(mp.param) not in owned_ids:
                        continue
                    su = r_units[ui]
                    if (ui, mp.fqn, su["rank"]) in seen_sources:
                        continue                    # another replica of the same shard rank
                    seen_sources.add((ui, mp.fqn, su["rank"]))
                    src = [sp for sp in _source_pieces({r: ranks[r]}, ui, mp.fqn)]
                    slot = per_param.setdefault(id(mp.param), {"mp": mp, "u": u, "piece": piece, "tensors": {},
                                                               "values": None})
                    tens, values = _split_entries(entry)
                    if slot["values"] is None and values:
                        slot["values"] = values
                    for name, e in tens.items():
                        dtype = _dtype_from_string(e["dtype"])
                        numel = 1
                        for d in e["shape"]:
                            numel *= int(d)
                        if len(e["shape"]) == 0 or not src or numel != sum(sp[3] for sp in src):
                            # not parameter-shaped (step counters, scalars kept as tensors): same on every owner
                            if name not in slot["tensors"]:
                                buf = torch.empty(tuple(e["shape"]), dtype=dtype)
                                requests[e["key"]] = buf
                                slot["tensors"][name] = buf
                            continue
                        pstart, n = e["piece"] if "piece" in e else (src[0][2], numel)
                        ov = _overlaps(piece.param_start, piece.param_start + piece.numel, pstart, pstart + n)
                        if ov is None:
                            continue
                        if e["key"] not in requests:
                            requests[e["key"]] = torch.empty(tuple(e["shape"]), dtype=dtype, device=u.flat_buffer.device)
                        dst = slot["tensors"].setdefault(
                            name, torch.zeros(piece.numel, dtype=dtype, device=u.flat_buffer.device))
                        plan.append((dst, ov[0] - piece.param_start, e["key"], ov[0] - pstart, ov[1] - ov[0]))
            for slot in per_param.values():
                for name, t in slot["tensors"].items():
                    staged_opt.append((opt, slot["mp"].param, name, t))
                if slot["values"]:
                    staged_opt.append((opt, slot["mp"].param, None, slot["values"]))
    with torch.no_grad():
        _dcp_load(requests, directory, use_dist=use_dist, group=group)
        for dst, doff, key, soff, n in plan:
            dst[doff:doff + n].copy_(requests[key].reshape(-1)[soff:soff + n])
        for u in units:
            u.flat_buffer.mark_master_updated(lp_written=False)
        _restore_optimizer(staged_opt, any_meta.get("optimizer"), optimizer)
    return any_meta


def load_matrix_dcp_full_state(directory: str, *, no_dist: bool | None = True) -> dict[str, Any]:
    """Read a ``full_state=True`` checkpoint into ``{"params": {module-level fqn: tensor}}``."""
    payload = read_global_metadata(directory)
    meta = payload["ranks"][sorted(payload["ranks"])[0]]
    env = meta.get("metadata", {})
    if not (env.get("full_state") or meta.get("full_state")):
        raise ValueError("Checkpoint was not saved with full_state=True.")
    req, names = {}, {}
    for i, su in enumerate(_unit_list(meta, "DCP metadata")):
        for fqn, pm in su["params"].items():
            key = su.get("full_param_keys", {}).get(fqn) or f"{su['dcp_payload_rank']}.unit_{i}.full_param.{fqn}"
            dtype = _dtype_from_string(su.get("full_param_dtype") or su.get("param_dtype") or pm["dtype"])
            req[key] = torch.empty(tuple(pm["shape"]), dtype=dtype)
            names[key] = param_key(su.get("module_fqn", ""), fqn, i)
    dcp.load(req, checkpoint_id=directory, no_dist=True)
    return {"params": {names[key]: t for key, t in req.items()}, "metadata": meta}
