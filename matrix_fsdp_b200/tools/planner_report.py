"""Offline planner what-if: ``python -m matrix_fsdp_b200.tools.planner_report``.

Builds a model on the meta device (no memory, no GPU), cuts it into FSDP units the way ``--unit`` says
(the whole model, one unit per block, one unit per ``nn.Linear``), plans every unit for a world size and a
planner policy, and prints

* per unit: the selected candidate (and, unless ``--selected-only``, every candidate the policy weighed) with
  cost, per-rank units, block kinds, constraint counts, what the runtime will do with the layout, warnings
  and which parameters each rank holds;
* the planner's running per-rank load when the policy is stateful (``muon_shard_aware``: owner rotation /
  role-greedy / cost-aware / model-wide assignment see the units in order, as ``fully_shard`` would);
* the rank-load summary: units, parameter + gradient + optimizer memory, gather / reduce bytes, Muon and AdamW
  parameter bytes, Newton-Schulz FLOPs and block kinds per rank, with max / mean imbalance.

``--format json`` prints the same content as one JSON object.

Parity: ``matrix_fsdp/tools/planner_report.py:1-555`` (models ``mlp``, ``transformer``, ``mlp_split``,
``transformer_split_qkv``; units ``model`` / ``block`` / ``linear``; rotation strategy, owner assignment,
target block units, hint switch, candidate listing, text / JSON).  Added here: the Llama and MoE decoder
configurations of this package, the model-wide owner assignment and the Newton-Schulz FLOP column.
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import asdict, dataclass, field
from functools import partial

import torch
from torch import nn

from ..core.managed_param import ManagedParamRegistry
from ..planning.auto_planner import (_report_row, auto_group_plan, available_auto_planner_policies,
                                     build_auto_planner_report, make_model_wide_muon_planner,
                                     make_muon_shard_aware_group_planner)
from ..planning.planner_eval import PlannerResourceEstimate, call_group_planner
from ..planning.shard_hint import build_shard_hints

MODELS = ("mlp", "mlp_split", "transformer", "transformer_split_qkv", "llama", "moe")
UNITS = ("model", "block", "linear")
OWNER_ASSIGNMENTS = ("rotate", "role_greedy", "cost_aware", "model_wide")


# ----------------------------------------------------------------------------------------------
# toy models (structure only: they are built on the meta device and never run)
# ----------------------------------------------------------------------------------------------
class _Mlp(nn.Module):
    def __init__(self, hidden: int, inter: int, split: bool) -> None:
        super().__init__()
        if split:       # gate and up as two matrices, as in gated feed-forward blocks
            self.gate_proj, self.up_proj = nn.Linear(hidden, inter, bias=False), nn.Linear(hidden, inter, bias=False)
        else:
            self.fc1 = nn.Linear(hidden, inter)
        self.fc2 = nn.Linear(inter, hidden, bias=not split)


class _Block(nn.Module):
    def __init__(self, hidden: int, inter: int, split_qkv: bool) -> None:
        super().__init__()
        self.norm1, self.norm2 = nn.LayerNorm(hidden), nn.LayerNorm(hidden)
        if split_qkv:
            self.q, self.k, self.v = (nn.Linear(hidden, hidden, bias=False) for _ in range(3))
        else:
            self.qkv = nn.Linear(hidden, 3 * hidden, bias=False)
        self.proj = nn.Linear(hidden, hidden, bias=False)
        self.mlp = _Mlp(hidden, inter, split=split_qkv)


@dataclass
class ReportConfig:
    model: str = "transformer_split_qkv"
    layers: int = 1
    hidden: int = 1024
    intermediate: int = 4096
    heads: int = 8
    vocab: int = 1024
    experts: int = 8
    unit: str = "model"
    world_size: int = 8
    policy: str = "muon_shard_aware"
    rotation_strategy: str = "greedy_balance"
    owner_assignment: str = "rotate"
    target_block_units: int | None = None
    auto_shard_hints: bool = True
    show_candidates: bool = True
    output_format: str = "text"


def build_model(cfg: ReportConfig) -> tuple[nn.Module, list[nn.Module]]:
    """The model and its repeated blocks, on the meta device."""
    with torch.device("meta"):
        if cfg.model in ("mlp", "mlp_split"):
            blocks = [_Mlp(cfg.hidden, cfg.intermediate, cfg.model == "mlp_split") for _ in range(cfg.layers)]
            model = nn.Sequential(*blocks)
        elif cfg.model in ("transformer", "transformer_split_qkv"):
            blocks = [_Block(cfg.hidden, cfg.intermediate, cfg.model == "transformer_split_qkv") for _ in range(cfg.layers)]
            model = nn.Sequential(*blocks)
        elif cfg.model == "llama":
            from ..models.llama import LlamaConfig, LlamaModel

            model = LlamaModel(LlamaConfig(vocab_size=cfg.vocab, hidden=cfg.hidden, n_layers=cfg.layers, n_heads=cfg.heads,
                                           head_dim=cfg.hidden // cfg.heads, ffn=cfg.intermediate))
            blocks = list(model.layers)
        elif cfg.model == "moe":
            from ..models.moe import MoEConfig, MoEModel

            model = MoEModel(MoEConfig(vocab_size=cfg.vocab, hidden=cfg.hidden, n_layers=cfg.layers, n_heads=cfg.heads,
                                       head_dim=cfg.hidden // cfg.heads, n_experts=cfg.experts,
                                       expert_ffn=cfg.intermediate, top_k=min(2, cfg.experts)))
            blocks = list(model.layers)
        else:
            raise ValueError(f"unknown model {cfg.model!r}; choose from {MODELS}")
    return model, blocks


def iter_units(model: nn.Module, blocks: list[nn.Module], unit: str):
    """``(name, module)`` per FSDP unit.  Parameters outside the repeated blocks (embeddings, final norm,
    head) form a last unit named ``<root>`` when units are blocks or linears."""
    if unit == "model":
        yield "<model>", model
        return
    names = {id(m): n for n, m in model.named_modules()}
    claimed: set[int] = set()
    if unit == "block":
        for b in blocks:
            claimed |= {id(p) for p in b.parameters()}
            yield names.get(id(b), type(b).__name__), b
    else:
        for n, m in model.named_modules():
            if isinstance(m, nn.Linear):
                claimed |= {id(p) for p in m.parameters()}
                yield n, m
    if any(id(p) not in claimed for p in model.parameters()):
        yield "<root>", _Rest(model, claimed)


class _Rest(nn.Module):
    """The parameters of ``model`` that no other unit claimed, under their original names."""

    def __init__(self, model: nn.Module, claimed: set[int]) -> None:
        super().__init__()
        for n, p in model.named_parameters():
            if id(p) not in claimed:
                self.register_parameter(n.replace(".", "__"), p)


# ----------------------------------------------------------------------------------------------
# planning
# ----------------------------------------------------------------------------------------------
@dataclass
class UnitReport:
    unit: str
    unit_type: str
    num_params: int
    numel: int
    rows: list = field(default_factory=list)           # AutoPlannerReportRow as dicts; rows[0] is the selected one
    rank_ns_flops: tuple[int, ...] = ()
    cumulative_rank_units: tuple[int, ...] = ()         # planner state after this unit


@dataclass
class ReportResult:
    config: dict
    units: list
    rank_units: tuple[int, ...]
    rank_memory_bytes: tuple[int, ...]
    rank_comm_bytes: tuple[int, ...]
    rank_muon_param_bytes: tuple[int, ...]
    rank_adamw_param_bytes: tuple[int, ...]
    rank_optimizer_bytes: tuple[int, ...]
    rank_ns_flops: tuple[int, ...]
    rank_block_kinds: tuple[dict, ...]
    imbalance: dict


def _registries(cfg: ReportConfig):
    model, blocks = build_model(cfg)
    out = []
    for name, mod in iter_units(model, blocks, cfg.unit):
        hints = build_shard_hints(mod) if cfg.auto_shard_hints else None
        reg = ManagedParamRegistry.from_module(mod, shard_hints=hints)
        if len(reg.params):
            out.append((name, type(mod).__name__, reg))
    return out


def _stateful_planner(cfg: ReportConfig, regs):
    if cfg.policy != "muon_shard_aware":
        if cfg.rotation_strategy != "greedy_balance" or cfg.owner_assignment != "rotate":
            raise ValueError("--rotation-strategy and --owner-assignment need --policy muon_shard_aware")
        return None
    if cfg.owner_assignment == "model_wide":
        return make_model_wide_muon_planner(tuple(r.params for _, _, r in regs), policy=cfg.policy)
    return make_muon_shard_aware_group_planner(policy=cfg.policy, rotation_strategy=cfg.rotation_strategy,
                                               owner_assignment=cfg.owner_assignment)


def run_report(cfg: ReportConfig) -> ReportResult:
    if cfg.unit not in UNITS:
        raise ValueError(f"unknown unit {cfg.unit!r}; choose from {UNITS}")
    if cfg.owner_assignment not in OWNER_ASSIGNMENTS:
        raise ValueError(f"unknown owner assignment {cfg.owner_assignment!r}; choose from {OWNER_ASSIGNMENTS}")
    regs = _registries(cfg)
    planner = _stateful_planner(cfg, regs)
    w = cfg.world_size
    totals = {k: [0] * w for k in ("units", "memory", "comm", "muon", "adamw", "optimizer", "flops")}
    kinds: list[dict[str, int]] = [dict() for _ in range(w)]
    units: list[UnitReport] = []
    for name, typ, reg in regs:
        if planner is not None:
            res = call_group_planner(planner, reg.params, w)
            rows = [_report_row(cfg.policy, res, True)]
            if cfg.show_candidates:      # what the stateless policy would have weighed for this unit alone
                rows += [r for r in build_auto_planner_report(reg.params, w, policy=cfg.policy,
                                                              target_block_units=cfg.target_block_units)
                         if r.candidate != res.name]
                rows = [rows[0]] + [_unselect(r) for r in rows[1:]]
            est = res.resource_estimate or PlannerResourceEstimate.empty(w)
            flops = tuple(est.rank_ns_flops or (0,) * w)
        else:
            rows = list(build_auto_planner_report(reg.params, w, policy=cfg.policy,
                                                  target_block_units=cfg.target_block_units,
                                                  show_candidates=cfg.show_candidates))
            res = call_group_planner(partial(auto_group_plan, policy=cfg.policy, target_block_units=cfg.target_block_units),
                                     reg.params, w)
            est = res.resource_estimate or PlannerResourceEstimate.empty(w)
            flops = tuple(est.rank_ns_flops or (0,) * w)
        sel = rows[0]
        for r in range(w):
            totals["units"][r] += sel.rank_units[r]
            totals["memory"][r] += sel.rank_memory_bytes[r]
            totals["comm"][r] += sel.rank_comm_bytes[r]
            totals["muon"][r] += sel.rank_muon_param_bytes[r]
            totals["adamw"][r] += sel.rank_adamw_param_bytes[r]
            totals["optimizer"][r] += sel.rank_optimizer_bytes[r]
            totals["flops"][r] += flops[r]
        for r, roles in enumerate(sel.rank_role_units or ()):
            for k, v in dict(roles).items():
                kinds[r][k] = kinds[r].get(k, 0) + int(v)
        units.append(UnitReport(unit=name, unit_type=typ, num_params=len(reg.params),
                                numel=sum(p.numel for p in reg.params), rows=[asdict(r) for r in rows],
                                rank_ns_flops=flops, cumulative_rank_units=tuple(totals["units"])))

    def imb(v):
        mean = sum(v) / len(v) if v else 0.0
        return (max(v) / mean) if mean else 0.0

    return ReportResult(config=asdict(cfg), units=[asdict(u) for u in units], rank_units=tuple(totals["units"]),
                        rank_memory_bytes=tuple(totals["memory"]), rank_comm_bytes=tuple(totals["comm"]),
                        rank_muon_param_bytes=tuple(totals["muon"]), rank_adamw_param_bytes=tuple(totals["adamw"]),
                        rank_optimizer_bytes=tuple(totals["optimizer"]), rank_ns_flops=tuple(totals["flops"]),
                        rank_block_kinds=tuple(kinds),
                        imbalance={"units": imb(totals["units"]), "memory": imb(totals["memory"]),
                                   "comm": imb(totals["comm"]), "muon_param": imb(totals["muon"]),
                                   "ns_flops": imb(totals["flops"])})


def _unselect(row):
    from dataclasses import replace

    return replace(row, selected=False)


# ----------------------------------------------------------------------------------------------
# text output
# ----------------------------------------------------------------------------------------------
def _table(headers, body) -> str:
    body = [tuple(str(c) for c in row) for row in body]
    widths = [max(len(h), *(len(b[i]) for b in body)) if body else len(h) for i, h in enumerate(headers)]
    line = lambda vals: "  ".join(v.ljust(w) for v, w in zip(vals, widths)).rstrip()   # noqa: E731
    return "\n".join([line(headers), line(tuple("-" * w for w in widths)), *(line(b) for b in body)])


def _ints(v) -> str:
    return "(" + ",".join(str(int(x)) for x in v) + ")"


def _counts(items) -> str:
    items = dict(items)
    return ",".join(f"{k}:{v}" for k, v in sorted(items.items())) or "-"


def _runtime(row: dict) -> str:
    if not row["runtime_compatible"]:
        return f"unsupported({row['runtime_reason']})"
    return row["runtime_mode"] + ("+reorder" if row["runtime_requires_flat_reorder"] else "")


def format_units(result: ReportResult) -> str:
    out = []
    for u in result.units:
        out.append(f"== unit {u['unit']} ({u['unit_type']}, {u['num_params']} params, {u['numel']} elements) ==")
        body = [("*" if r["selected"] else "", r["candidate"], f"{r['cost']:.3f}", _runtime(r), _ints(r["rank_units"]),
                 _counts(r["block_kinds"]), _counts(r["constraint_counts"]), r["num_rank_segments"], r["num_split_params"],
                 r["candidate_collectives"], r["max_rank_memory_bytes"], r["max_rank_comm_bytes"]) for r in u["rows"]]
        out.append(_table(("sel", "candidate", "cost", "runtime", "rank_units", "block_kinds", "constraints", "segs",
                           "split", "collectives", "max_mem_B", "max_comm_B"), body))
        sel = u["rows"][0]
        out.append("params by rank: " + "; ".join(f"r{i}:[{','.join(n)}]" for i, n in enumerate(sel["params_by_rank"])))
        if any(u["rank_ns_flops"]):
            out.append("Newton-Schulz FLOPs by rank: " + _ints(u["rank_ns_flops"]))
        out.append("planner load after this unit: " + _ints(u["cumulative_rank_units"]))
        if sel["warnings"]:
            out.append("warnings: " + " | ".join(sel["warnings"]))
        out.append("")
    return "\n".join(out)


def format_rank_load(result: ReportResult) -> str:
    w = len(result.rank_units)
    body = [(r, result.rank_units[r], result.rank_memory_bytes[r], result.rank_comm_bytes[r],
             result.rank_muon_param_bytes[r], result.rank_adamw_param_bytes[r], result.rank_optimizer_bytes[r],
             result.rank_ns_flops[r], _counts(result.rank_block_kinds[r])) for r in range(w)]
    table = _table(("rank", "units", "memory_B", "comm_B", "muon_param_B", "adamw_param_B", "optimizer_B", "ns_flops",
                    "roles"), body)
    imb = "  ".join(f"{k}={v:.4f}" for k, v in result.imbalance.items())
    return f"== rank load ==\n{table}\nimbalance (max / mean): {imb}"


def format_report(result: ReportResult) -> str:
    c = result.config
    head = (f"planner report: model={c['model']} layers={c['layers']} hidden={c['hidden']} intermediate={c['intermediate']} "
            f"unit={c['unit']} world_size={c['world_size']} policy={c['policy']} owner_assignment={c['owner_assignment']} "
            f"rotation={c['rotation_strategy']} hints={'auto' if c['auto_shard_hints'] else 'off'}")
    return "\n".join([head, "", format_units(result), format_rank_load(result)])


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", choices=MODELS, default="transformer_split_qkv")
    ap.add_argument("--layers", type=int, default=1)
    ap.add_argument("--hidden", type=int, default=1024)
    ap.add_argument("--intermediate", "--ffn", type=int, default=None, dest="intermediate")
    ap.add_argument("--heads", type=int, default=8)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--unit", choices=UNITS, default="block")
    ap.add_argument("--world-size", type=int, default=8)
    ap.add_argument("--policy", choices=available_auto_planner_policies(), default="muon_shard_aware")
    ap.add_argument("--rotation-strategy", choices=("greedy_balance", "round_robin"), default="greedy_balance")
    ap.add_argument("--owner-assignment", choices=OWNER_ASSIGNMENTS, default="role_greedy")
    ap.add_argument("--target-block-units", type=int, default=None)
    ap.add_argument("--no-auto-shard-hints", action="store_true")
    ap.add_argument("--selected-only", action="store_true")
    ap.add_argument("--format", choices=("text", "json"), default="text", dest="output_format")
    ap.add_argument("--json", action="store_true", help="text report followed by one JSON line with the per-rank totals")
    a = ap.parse_args(argv)
    if a.policy != "muon_shard_aware":
        a.owner_assignment, a.rotation_strategy = "rotate", "greedy_balance"
    cfg = ReportConfig(model=a.model, layers=a.layers, hidden=a.hidden, intermediate=a.intermediate or 4 * a.hidden,
                       heads=a.heads, vocab=a.vocab, experts=a.experts, unit=a.unit, world_size=a.world_size,
                       policy=a.policy, rotation_strategy=a.rotation_strategy, owner_assignment=a.owner_assignment,
                       target_block_units=a.target_block_units, auto_shard_hints=not a.no_auto_shard_hints,
                       show_candidates=not a.selected_only, output_format=a.output_format)
    result = run_report(cfg)
    if cfg.output_format == "json":
        print(json.dumps(asdict(result), default=str))
        return 0
    print(format_report(result))
    if a.json:
        print(json.dumps({"units": [{"unit": u["unit"], "planner": u["rows"][0]["candidate"],
                                     "rank_units": list(u["rows"][0]["rank_units"])} for u in result.units],
                          "rank_units": list(result.rank_units), "rank_memory_bytes": list(result.rank_memory_bytes),
                          "rank_ns_flops": list(result.rank_ns_flops), "imbalance": result.imbalance}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
