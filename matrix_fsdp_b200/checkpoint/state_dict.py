"""Sharded checkpoints in the ``matrix_dcp`` format, with FQN-addressed resharding.

On disk (one directory):

* tensors through ``torch.distributed.checkpoint`` under keys
  ``"{rank_R|shard_S}.unit_{i}.param_shard"`` (the rank's whole packed local shard),
  ``….grad_shard``, ``….full_param.{fqn}`` / ``….full_grad.{fqn}`` (debug ``full_state``) and
  ``"{payload}.unit_0.optimizer.{component}.u{i}.{fqn}.{state}"`` for optimizer tensors;
  with HSDP and ``dedup_replicates`` only replica 0 writes and the prefix is ``shard_S``;
* one ``matrix_metadata.pt``: ``{"metadata": {"format": "matrix_dcp_global_metadata",
  "version": 1, "num_ranks", "ranks"}, "ranks": {rank: per-rank metadata}}``; legacy per-rank
  ``matrix_metadata_rank_{r}.pt`` sidecars are still read.

Same-layout loads validate every structural field *before* touching tensors and then read straight
into ``local_shard`` and freshly bound optimizer state.  ``allow_reshard=True`` loads onto any world
size or layout: every parameter piece a rank owns is assembled from the source pieces that overlap
it, addressed by (unit, fqn, offset-in-parameter) — the saved per-parameter ``pieces`` metadata — so
matrix-owner layouts, whose flat order depends on the world size, reshard bit-exactly.  The
reference instead concatenates all source shards on every rank and requires identical flat order
(``matrix_fsdp/checkpoint/state_dict.py:879-950,1309-1327``).

Parity: ``matrix_fsdp/checkpoint/state_dict.py:65-1397``, ``_dcp_utils.py``, ``_metadata.py``,
``_optimizer_utils.py``.
"""
from __future__ import annotations

import os
from collections.abc import Mapping
from typing import Any

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp

from ..core.mixed_precision import mixed_precision_policy_metadata, offload_policy_metadata
from ..core.state import matrix_shard_metadata
from ..parallel.unit_collection import collect_param_groups

GLOBAL_METADATA_FILE = "matrix_metadata.pt"
GLOBAL_METADATA_FORMAT = "matrix_dcp_global_metadata"
OPTIMIZER_FORMAT_VERSION = 2


# --------------------------------------------------------------------------- helpers
def _units(model_or_units):
    units = collect_param_groups(model_or_units)
    if not units:
        raise ValueError("Expected a module wrapped by fully_shard().")
    return units


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


# --------------------------------------------------------------------------- metadata
def _param_metadata(unit, mp) -> dict[str, Any]:
    layout, fb = unit.layout, unit.flat_buffer
    pl = layout.param(mp.fqn)
    piece = fb.pieces.get(mp.fqn)
    return {
        "fqn": mp.fqn, "shape": tuple(mp.shape), "dtype": str(mp.dtype), "device": str(mp.device),
        "numel": mp.numel, "offset": mp.offset, "end": mp.end, "owner_ranks": layout.owner_ranks(mp.fqn),
        "local_segments": tuple((s.global_start, s.global_end, s.local_start)
                                for s in layout.rank_segments_for_param(unit.rank, mp.fqn)),
        "pieces": tuple((s.rank, s.global_start - mp.offset, s.numel, s.local_start) for s in pl.segments),
        "local_piece": None if piece is None else (piece.param_start, piece.numel, piece.local_start),
        "shard_sizes": layout.shard_sizes, "matrix_shard": matrix_shard_metadata(fb.matrix_shard),
        "shard_hint": dict(mp.shard_hint.__dict__), "aliases": tuple(mp.aliases),
    }


def _unit_state_dict(unit, index: int, *, clone: bool, include_grads: bool, dedup_replicates: bool) -> dict[str, Any]:
    fb, res = unit.flat_buffer, unit.planner_result
    segs = fb.tables.my_segments
    meta = res.as_metadata()
    d = {
        "unit_index": index, "name": unit.name, "runtime_param_group_id": unit.metadata.runtime_param_group_id,
        "rank": unit.rank, "world_size": unit.world_size, "replicate_rank": unit.replicate_rank,
        "replicate_world_size": unit.replicate_world_size,
        "mesh": unit.groups.metadata.as_dict() if unit.groups.metadata is not None else None,
        "mp_policy": mixed_precision_policy_metadata(unit.mp_policy),
        "offload_policy": offload_policy_metadata(unit.offload_policy),
        "total_numel": fb.total_numel, "local_numel": fb.local_numel,
        "local_start": segs[0].global_start if len(segs) == 1 else None,
        "local_end": segs[0].global_end if len(segs) == 1 else None,
        "local_segments": tuple((s.global_start, s.global_end, s.local_start) for s in segs),
        "shard_sizes": unit.layout.shard_sizes, "matrix_shard": matrix_shard_metadata(fb.matrix_shard),
        "planner_name": res.name, "planner_policy": res.policy, "runtime_mode": unit.runtime_mode,
        "planner_metadata": {"layout_contract": meta["layout_contract"], "report": meta["report"],
                             "resource_estimate": meta["resource_estimate"],
                             "expert_owner_groups": meta["expert_owner_groups"], "warnings": meta["warnings"]},
        "param_gather_strategy": unit.param_gather_strategy, "backward_reduce_strategy": unit.backward_reduce_strategy,
        "shard_dtype": str(fb.shard_dtype), "param_dtype": str(fb.param_dtype),
        "param_fqns": unit.registry.fqns,
        "params": {mp.fqn: _param_metadata(unit, mp) for mp in unit.registry},
        "dcp_payload_rank": dcp_payload_prefix(unit, dedup_replicates=dedup_replicates),
        "dcp_dedup_replicates": bool(dedup_replicates and unit.replicate_world_size > 1),
        "param_shard": fb.local_shard.detach().clone() if clone else fb.local_shard.detach(),
    }
    if include_grads and fb.local_grad_shard is not None:
        g = fb.local_grad_shard.detach()
        d["grad_shard"] = g.clone() if clone else g
    return d


def matrix_state_dict(model_or_units, *, clone: bool = True, include_grads: bool = False,
                      dedup_replicates: bool = True) -> dict[str, Any]:
    """In-memory sharded state: ``{"units": [per-unit dict incl. the ``param_shard`` tensor]}``."""
    units = _units(model_or_units)
    return {"format": "matrix_state_dict", "version": 1, "dcp_rank": _global_rank(),
            "units": [_unit_state_dict(u, i, clone=clone, include_grads=include_grads,
                                       dedup_replicates=dedup_replicates) for i, u in enumerate(units)]}


_SAME_LAYOUT_FIELDS = ("world_size", "replicate_world_size", "total_numel", "local_numel", "local_start", "local_end",
                       "local_segments", "shard_sizes", "param_fqns", "shard_dtype")


def _validate_same_layout_unit(saved: Mapping[str, Any], unit, index: int) -> None:
    current = _unit_state_dict(unit, index, clone=False, include_grads=False, dedup_replicates=True)
    for name in _SAME_LAYOUT_FIELDS:
        a, b = saved.get(name), current.get(name)
        if isinstance(a, list):
            a = tuple(tuple(x) if isinstance(x, list) else x for x in a)
        if a != b:
            raise ValueError(f"Checkpoint unit {index} field {name!r} does not match the model: saved {a!r}, "
                             f"current {b!r}. Pass allow_reshard=True to load onto a different layout.")
    for fqn, pm in saved["params"].items():
        cur = current["params"].get(fqn)
        if cur is None:
            raise ValueError(f"Checkpoint unit {index} has unknown parameter {fqn!r}.")
        for name in ("shape", "numel", "offset", "end", "local_segments"):
            if tuple(pm[name]) != tuple(cur[name]) if isinstance(pm[name], (tuple, list)) else pm[name] != cur[name]:
                raise ValueError(f"Checkpoint unit {index} parameter {fqn!r} field {name!r} does not match the model.")


def load_matrix_state_dict(model_or_units, state: Mapping[str, Any], *, strict: bool = True) -> None:
    """Load an in-memory ``matrix_state_dict`` produced on the same layout."""
    units = _units(model_or_units)
    saved_units = state["units"]
    if len(saved_units) != len(units):
        raise ValueError(f"State dict has {len(saved_units)} units, the model has {len(units)}.")
    for i, (u, su) in enumerate(zip(units, saved_units)):
        if strict:
            _validate_same_layout_unit(su, u, i)
    with torch.no_grad():
        for u, su in zip(units, saved_units):
            u.flat_buffer.local_shard.copy_(su["param_shard"])
            u.flat_buffer.mark_master_updated(lp_written=False)
            if "grad_shard" in su:
                u.flat_buffer._ensure_local_grad_shard().copy_(su["grad_shard"])
                u.flat_buffer.local_grad_valid = True
                u.flat_buffer.use_local_grad_shard()


# --------------------------------------------------------------------------- optimizer state
def _param_key_index(units) -> dict[int, tuple[int, Any, Any]]:
    idx = {}
    for ui, u in enumerate(units):
        for mp in u.registry:
            idx[id(mp.param)] = (ui, u, mp)
    return idx


def _collect_optimizer_state(units, optimizer, payload_of) -> tuple[dict[str, torch.Tensor], dict[str, Any]]:
    """→ (tensor entries keyed for DCP, metadata describing every state entry)."""
    tensors: dict[str, torch.Tensor] = {}
    meta: dict[str, Any] = {"optimizer_format_version": OPTIMIZER_FORMAT_VERSION, "kind": _optimizer_kind(optimizer),
                            "components": {}}
    idx = _param_key_index(units)
    for comp, opt in iter_optimizer_components(optimizer):
        cmeta = {"class": type(opt).__name__, "param_groups": [], "state": {}}
        for g in getattr(opt, "param_groups", []):
            hp = {k: v for k, v in g.items() if k != "params" and isinstance(v, (int, float, bool, str, tuple, list, type(None)))}
            fq = []
            for p in g["params"]:
                hit = idx.get(id(p))
                fq.append(f"{hit[1].name}.{hit[2].fqn}" if hit else None)
            cmeta["param_groups"].append({"hyper": hp, "params": fq})
        for p, st in getattr(opt, "state", {}).items():
            hit = idx.get(id(p))
            if hit is None:
                continue
            ui, u, mp = hit
            piece = u.flat_buffer.pieces.get(mp.fqn)
            if piece is None:
                continue
            key_base = f"{payload_of(u)}.unit_0.optimizer.{comp}.u{ui}.{mp.fqn}"
            entry = {"fqn": mp.fqn, "unit": u.name, "unit_index": ui, "tensors": {}, "scalars": {}}
            for name, val in st.items():
                if isinstance(val, torch.Tensor) and val.dim() > 0 and val.numel() == piece.numel:
                    tensors[f"{key_base}.{name}"] = val.detach().reshape(-1)
                    entry["tensors"][name] = {"shape": tuple(val.shape), "dtype": str(val.dtype),
                                              "piece": (piece.param_start, piece.numel),
                                              "matrix_state": matrix_shard_metadata(u.flat_buffer.matrix_shard)}
                elif isinstance(val, torch.Tensor):
                    entry["scalars"][name] = float(val.item()) if val.numel() == 1 else val.tolist()
                else:
                    entry["scalars"][name] = val
            cmeta["state"][f"{u.name}.{mp.fqn}"] = entry
        meta["components"][comp] = cmeta
    return tensors, meta


def _check_components(saved_meta: Mapping[str, Any], optimizer) -> None:
    have = {n for n, _ in iter_optimizer_components(optimizer)}
    saved = set(saved_meta.get("components", {}))
    if saved - have:
        raise ValueError(f"Checkpoint has unknown component(s) for this optimizer: {sorted(saved - have)}")
    if have - saved:
        raise ValueError(f"Checkpoint is missing component(s) of this optimizer: {sorted(have - saved)}")


_DTYPES = {str(d): d for d in (torch.float32, torch.bfloat16, torch.float16, torch.float64)}


def _bind_optimizer_state(opt, p, name: str, value: torch.Tensor) -> None:
    """Put a loaded state tensor where the optimizer expects it (flat views are copied into)."""
    st = opt.state[p] if hasattr(opt.state, "__getitem__") else None
    if st is None:
        return
    cur = st.get(name)
    if isinstance(cur, torch.Tensor) and cur.numel() == value.numel():
        cur.copy_(value.view(cur.shape))
    else:
        st[name] = value.view(p.shape if value.numel() == p.numel() else value.shape).clone()


# --------------------------------------------------------------------------- global metadata file
def _write_global_metadata(directory: str, rank_metadata: dict[str, Any], *, use_dist: bool, group=None) -> None:
    if use_dist:
        gathered: list = [None] * dist.get_world_size(group)
        dist.all_gather_object(gathered, rank_metadata, group=group)
        ranks = {m["dcp_rank"]: m for m in gathered}
    else:
        ranks = {rank_metadata["dcp_rank"]: rank_metadata}
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


# --------------------------------------------------------------------------- save
def save_matrix_dcp(model_or_units, directory: str, optimizer=None, *, full_state: bool = False,
                    include_grads: bool = False, dedup_replicates: bool = True, process_group=None,
                    no_dist: bool | None = None) -> dict[str, Any]:
    units = _units(model_or_units)
    use_dist = _dist_on(no_dist)
    state = matrix_state_dict(units, clone=False, include_grads=include_grads, dedup_replicates=dedup_replicates)
    if isinstance(model_or_units, torch.nn.Module):
        paths = {id(m): name for name, m in model_or_units.named_modules()}
        for u, us in zip(units, state["units"]):
            us["module_fqn"] = paths.get(id(u.module), "")
    tensors: dict[str, torch.Tensor] = {}
    for i, (u, us) in enumerate(zip(units, state["units"])):
        prefix = f"{us['dcp_payload_rank']}.unit_{i}"
        writes = _writes_payload(u, dedup_replicates=dedup_replicates)
        shard = us.pop("param_shard")
        grad = us.pop("grad_shard", None)
        if writes:
            tensors[f"{prefix}.param_shard"] = shard
            if grad is not None:
                tensors[f"{prefix}.grad_shard"] = grad
        us["has_grad_shard"] = grad is not None
    if full_state:
        for i, u in enumerate(units):
            prefix = f"{state['units'][i]['dcp_payload_rank']}.unit_{i}"
            u.unshard("checkpoint_full_state")
            for mp in u.registry:
                if _global_rank() == 0 or not use_dist:
                    tensors[f"{prefix}.full_param.{mp.fqn}"] = mp.param.detach().clone()
            u.reshard("checkpoint_full_state")
        state["full_state"] = True
    opt_meta = None
    if optimizer is not None:
        payload_of = {id(u): state["units"][i]["dcp_payload_rank"] for i, u in enumerate(units)}
        writers = {id(u) for u in units if _writes_payload(u, dedup_replicates=dedup_replicates)}
        opt_tensors, opt_meta = _collect_optimizer_state(units, optimizer, lambda u: payload_of[id(u)])
        for k, v in opt_tensors.items():
            ui = int(k.split(".optimizer.", 1)[1].split(".", 2)[1][1:])
            if id(units[ui]) in writers:
                tensors[k] = v
    state["optimizer"] = opt_meta
    _write_global_metadata(directory, state, use_dist=use_dist, group=process_group)
    dcp.save(tensors, checkpoint_id=directory, process_group=process_group if use_dist else None,
             no_dist=not use_dist)
    return state


# --------------------------------------------------------------------------- load
def _dcp_load(tensors: dict[str, torch.Tensor], directory: str, *, use_dist: bool, group=None) -> None:
    if tensors or use_dist:
        dcp.load(tensors, checkpoint_id=directory, process_group=group if use_dist else None, no_dist=not use_dist)


def _my_metadata(payload: dict[str, Any]) -> dict[str, Any]:
    ranks = payload["ranks"]
    r = _global_rank()
    if r not in ranks:
        raise ValueError(f"Checkpoint holds ranks {sorted(ranks)}; rank {r} is missing "
                         "(pass allow_reshard=True to load on a different world size).")
    return ranks[r]


def load_matrix_dcp(model_or_units, directory: str, optimizer=None, *, allow_reshard: bool = False,
                    include_grads: bool = False, process_group=None, no_dist: bool | None = None,
                    dedup_replicates: bool = True) -> dict[str, Any]:
    units = _units(model_or_units)
    use_dist = _dist_on(no_dist)
    payload = read_global_metadata(directory)
    if allow_reshard:
        return _load_resharded(units, directory, payload, optimizer, use_dist=use_dist, group=process_group)
    meta = _my_metadata(payload)
    saved_units = meta["units"]
    if len(saved_units) != len(units):
        raise ValueError(f"Checkpoint has {len(saved_units)} units, the model has {len(units)}.")
    for i, (u, su) in enumerate(zip(units, saved_units)):
        _validate_same_layout_unit(su, u, i)
    if optimizer is not None:
        if meta.get("optimizer") is None:
            raise ValueError("Checkpoint holds no optimizer state.")
        _check_components(meta["optimizer"], optimizer)
    tensors: dict[str, torch.Tensor] = {}
    for i, (u, su) in enumerate(zip(units, saved_units)):
        prefix = f"{su['dcp_payload_rank']}.unit_{i}"
        tensors[f"{prefix}.param_shard"] = u.flat_buffer.local_shard
        if include_grads and su.get("has_grad_shard"):
            tensors[f"{prefix}.grad_shard"] = u.flat_buffer._ensure_local_grad_shard()
    staged: list[tuple] = []
    if optimizer is not None:
        comps = dict(iter_optimizer_components(optimizer))
        for comp, cmeta in meta["optimizer"]["components"].items():
            for key, entry in cmeta["state"].items():
                u = units[entry["unit_index"]]
                mp = u.registry.param(entry["fqn"])
                payload_rank = saved_units[entry["unit_index"]]["dcp_payload_rank"]
                for name, tm in entry["tensors"].items():
                    buf = torch.empty(tm["piece"][1], dtype=_DTYPES[tm["dtype"]], device=u.flat_buffer.device)
                    tensors[f"{payload_rank}.unit_0.optimizer.{comp}.u{entry['unit_index']}.{mp.fqn}.{name}"] = buf
                    staged.append((comps[comp], mp.param, name, buf))
                staged.append((comps[comp], mp.param, None, entry["scalars"]))
    with torch.no_grad():
        _dcp_load(tensors, directory, use_dist=use_dist, group=process_group)
        for u in units:
            u.flat_buffer.mark_master_updated(lp_written=False)
            if include_grads and u.flat_buffer.local_grad_shard is not None:
                u.flat_buffer.local_grad_valid = True
                u.flat_buffer.use_local_grad_shard()
        _restore_optimizer(staged, meta.get("optimizer"), optimizer)
    return meta


def _restore_optimizer(staged, saved_meta, optimizer) -> None:
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
                    cur.fill_(v) if cur.numel() == 1 else cur.copy_(torch.as_tensor(v))
                else:
                    st[k] = torch.tensor(float(v)) if k == "step" else v
        else:
            _bind_optimizer_state(opt, p, name, value)
    comps = dict(iter_optimizer_components(optimizer))
    for comp, cmeta in (saved_meta or {}).get("components", {}).items():
        opt = comps.get(comp)
        if opt is None:
            continue
        for g, sg in zip(getattr(opt, "param_groups", []), cmeta["param_groups"]):
            for k, v in sg["hyper"].items():
                g[k] = tuple(v) if isinstance(g.get(k), tuple) and isinstance(v, list) else v
        # flat optimizers keep a per-unit step counter next to the per-param entries
        rebind = getattr(opt, "_unit_states", None)
        if rebind:
            for us in rebind.values():
                steps = [float(opt.state[mp.param]["step"]) for mp in us.unit.registry
                         if mp.param in opt.state and "step" in opt.state[mp.param]]
                if steps:
                    us.step = int(max(steps))


# --------------------------------------------------------------------------- reshard load
def _overlaps(a0: int, a1: int, b0: int, b1: int) -> tuple[int, int] | None:
    lo, hi = max(a0, b0), min(a1, b1)
    return (lo, hi) if lo < hi else None


def _load_resharded(units, directory: str, payload: dict[str, Any], optimizer, *, use_dist: bool, group=None):
    """Assemble every owned parameter piece (and its optimizer tensors) from overlapping source pieces."""
    ranks = payload["ranks"]
    any_meta = ranks[sorted(ranks)[0]]
    saved_units = any_meta["units"]
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
    # payload prefix that holds source shard-rank s of unit i
    def source_prefix(i: int, shard_rank: int) -> str:
        for r in sorted(ranks):
            su = ranks[r]["units"][i]
            if su["rank"] == shard_rank and (not su["dcp_dedup_replicates"] or su["replicate_rank"] == 0):
                return su["dcp_payload_rank"]
        raise ValueError(f"No saved payload for shard rank {shard_rank} of unit {i}.")

    src_dtype = {i: _DTYPES[su["shard_dtype"]] for i, su in enumerate(saved_units)}
    src_sizes = {i: su["shard_sizes"] for i, su in enumerate(saved_units)}
    requests: dict[str, torch.Tensor] = {}
    plan: list[tuple] = []    # (dst tensor, dst offset, key, src offset, numel)
    for i, u in enumerate(units):
        fb = u.flat_buffer
        for fqn, piece in fb.pieces.items():
            pm = saved_units[i]["params"][fqn]
            for (srank, pstart, n, lstart) in pm["pieces"]:
                ov = _overlaps(piece.param_start, piece.param_start + piece.numel, pstart, pstart + n)
                if ov is None:
                    continue
                key = f"{source_prefix(i, srank)}.unit_{i}.param_shard"
                if key not in requests:
                    requests[key] = torch.empty(src_sizes[i][srank], dtype=src_dtype[i], device=fb.device)
                plan.append((fb.local_shard, piece.local_start + (ov[0] - piece.param_start), key,
                             lstart + (ov[0] - pstart), ov[1] - ov[0]))
    staged_opt: list[tuple] = []
    if optimizer is not None:
        comps = dict(iter_optimizer_components(optimizer))
        idx = {(u.name, mp.fqn): (i, u, mp) for i, u in enumerate(units) for mp in u.registry}
        # unit names may differ between runs; map by unit index instead
        name_by_index = {i: u.name for i, u in enumerate(units)}
        for comp, opt in comps.items():
            owned = [p for g in getattr(opt, "param_groups", []) for p in g["params"]]
            owned_ids = {id(p) for p in owned}
            for i, u in enumerate(units):
                for mp in u.registry:
                    piece = u.flat_buffer.pieces.get(mp.fqn)
                    if piece is None or id(mp.param) not in owned_ids:
                        continue
                    scalars = None
                    per_name: dict[str, torch.Tensor] = {}
                    for r in sorted(ranks):
                        cm = ranks[r]["optimizer"]["components"].get(comp, {"state": {}})
                        for entry in cm["state"].values():
                            if entry["unit_index"] != i or entry["fqn"] != mp.fqn:
                                continue
                            su = ranks[r]["units"][i]
                            if su["dcp_dedup_replicates"] and su["replicate_rank"] != 0:
                                continue
                            scalars = entry["scalars"]
                            for name, tm in entry["tensors"].items():
                                pstart, n = tm["piece"]
                                ov = _overlaps(piece.param_start, piece.param_start + piece.numel, pstart, pstart + n)
                                if ov is None:
                                    continue
                                key = f"{su['dcp_payload_rank']}.unit_0.optimizer.{comp}.u{i}.{mp.fqn}.{name}"
                                if key not in requests:
                                    requests[key] = torch.empty(n, dtype=_DTYPES[tm["dtype"]], device=u.flat_buffer.device)
                                dst = per_name.setdefault(name, torch.zeros(piece.numel, dtype=_DTYPES[tm["dtype"]],
                                                                            device=u.flat_buffer.device))
                                plan.append((dst, ov[0] - piece.param_start, key, ov[0] - pstart, ov[1] - ov[0]))
                    for name, dst in per_name.items():
                        staged_opt.append((opt, mp.param, name, dst))
                    if scalars is not None:
                        staged_opt.append((opt, mp.param, None, scalars))
        del idx, name_by_index
    with torch.no_grad():
        _dcp_load(requests, directory, use_dist=use_dist, group=group)
        for dst, doff, key, soff, n in plan:
            dst[doff:doff + n].copy_(requests[key][soff:soff + n])
        for u in units:
            u.flat_buffer.mark_master_updated(lp_written=False)
        _restore_optimizer(staged_opt, any_meta.get("optimizer"), optimizer)
    return any_meta


def load_matrix_dcp_full_state(directory: str, *, no_dist: bool | None = True) -> dict[str, Any]:
    """Read a ``full_state=True`` checkpoint into ``{"params": {module-level fqn: tensor}}``."""
    payload = read_global_metadata(directory)
    meta = payload["ranks"][sorted(payload["ranks"])[0]]
    if not meta.get("full_state"):
        raise ValueError("Checkpoint was not saved with full_state=True.")
    req, names = {}, {}
    for i, su in enumerate(meta["units"]):
        for fqn, pm in su["params"].items():
            key = f"{su['dcp_payload_rank']}.unit_{i}.full_param.{fqn}"
            req[key] = torch.empty(tuple(pm["shape"]), dtype=_DTYPES[su["param_dtype"]])
            prefix = su.get("module_fqn", su["name"])
            names[key] = f"{prefix}.{fqn}" if prefix else fqn
    dcp.load(req, checkpoint_id=directory, no_dist=True)
    return {"params": {names[key]: t for key, t in req.items()}, "metadata": meta}
