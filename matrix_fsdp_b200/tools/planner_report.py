"""Offline planner what-if: ``python -m matrix_fsdp_b200.tools.planner_report``.

Builds a toy MLP / transformer (or the Llama configs) on the meta device, plans every unit for a
given world size and policy, and prints the per-unit candidate table plus the cumulative per-rank
load (elements, memory bytes, Newton-Schulz FLOPs).

Parity: ``matrix_fsdp/tools/planner_report.py:1-555``.
"""
from __future__ import annotations

import argparse
import json
import sys

import torch
from torch import nn

from ..core.managed_param import ManagedParamRegistry
from ..planning.auto_planner import (build_auto_planner_report, format_auto_planner_report,
                                     make_model_wide_muon_planner, make_muon_shard_aware_group_planner)
from ..planning.planner_eval import call_group_planner
from ..planning.shard_hint import build_shard_hints


def build_model(kind: str, hidden: int, layers: int, ffn: int | None, vocab: int) -> tuple[nn.Module, list[nn.Module]]:
    with torch.device("meta"):
        if kind == "mlp":
            blocks = [nn.Sequential(nn.Linear(hidden, 4 * hidden), nn.GELU(), nn.Linear(4 * hidden, hidden))
                      for _ in range(layers)]
            model = nn.Sequential(*blocks)
        else:
            from ..models.llama import LlamaConfig, LlamaModel

            heads = max(1, hidden // 128)
            cfg = LlamaConfig(vocab_size=vocab, hidden=hidden, n_layers=layers, n_heads=heads,
                              head_dim=hidden // heads, ffn=ffn or 4 * hidden)
            model = LlamaModel(cfg)
            blocks = list(model.layers)
    return model, blocks


def plan_units(blocks, world_size: int, policy: str, owner_assignment: str):
    regs = [ManagedParamRegistry.from_module(b, shard_hints=build_shard_hints(b)) for b in blocks]
    if owner_assignment == "model_wide":
        planner = make_model_wide_muon_planner(tuple(r.params for r in regs), policy=policy)
    elif policy == "muon_shard_aware":
        planner = make_muon_shard_aware_group_planner(owner_assignment=owner_assignment, policy=policy)
    else:
        planner = None
    out = []
    for reg in regs:
        if planner is None:
            rows = build_auto_planner_report(reg.params, world_size, policy=policy)
            out.append((reg, None, rows))
        else:
            res = call_group_planner(planner, reg.params, world_size)
            out.append((reg, res, ()))
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", choices=("mlp", "transformer"), default="transformer")
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--ffn", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=1024)
    ap.add_argument("--world-size", type=int, default=8)
    ap.add_argument("--policy", default="muon_shard_aware")
    ap.add_argument("--owner-assignment", default="role_greedy",
                    choices=("rotate", "role_greedy", "cost_aware", "model_wide"))
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    _, blocks = build_model(args.model, args.hidden, args.layers, args.ffn, args.vocab)
    planned = plan_units(blocks, args.world_size, args.policy, args.owner_assignment)
    totals = [0] * args.world_size
    mem = [0] * args.world_size
    flops = [0] * args.world_size
    report = []
    for i, (reg, res, rows) in enumerate(planned):
        if res is None:
            print(f"== unit {i} ==")
            print(format_auto_planner_report(rows))
            sizes = rows[0].rank_units
            rmem, rfl = rows[0].rank_memory_bytes, (0,) * args.world_size
            name = rows[0].candidate
        else:
            sizes = res.layout.shard_sizes
            rmem = res.resource_estimate.rank_memory_bytes
            rfl = res.resource_estimate.rank_ns_flops or (0,) * args.world_size
            name = res.name
            print(f"unit {i}: planner={name} mode={res.runtime_mode} rank_units={sizes}")
        for r in range(args.world_size):
            totals[r] += sizes[r]
            mem[r] += rmem[r]
            flops[r] += rfl[r]
        report.append({"unit": i, "planner": name, "rank_units": list(sizes)})
    print(f"cumulative rank units : {totals}")
    print(f"cumulative memory (B) : {mem}")
    print(f"cumulative NS FLOPs   : {flops}")
    imb = (max(totals) / (sum(totals) / len(totals))) if sum(totals) else 0.0
    print(f"imbalance ratio (max/mean units): {imb:.4f}")
    if args.json:
        print(json.dumps({"units": report, "rank_units": totals, "rank_memory_bytes": mem, "rank_ns_flops": flops}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
