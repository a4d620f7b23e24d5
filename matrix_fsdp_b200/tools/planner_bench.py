"""Planner timing / quality sweep (host only).

    python -m matrix_fsdp_b200.tools.planner_bench --hidden 4096 --layers 32 --world 8 16 --repeat 3

For every (world size, owner-assignment strategy) it plans all blocks of a Llama-shaped model on the
meta device and reports the planning time per block and the quality of the result: per-rank load
imbalance of the matrix owners (max / mean of cumulative owned elements), the largest per-unit
all-gather workspace relative to an even split, and the balance of Newton-Schulz FLOPs.

Parity: ``test/fsdp/bench_auto_planner.py:1-434`` (planner timing/quality sweeps).
"""
from __future__ import annotations

import argparse
import json
import time

from ..core.managed_param import ManagedParamRegistry
from ..planning.auto_planner import (available_auto_planner_policies, build_auto_planner_report,
                                     make_model_wide_muon_planner, make_muon_shard_aware_group_planner, muon_role_flops)
from ..planning.planner_eval import call_group_planner
from ..planning.shard_hint import build_shard_hints
from .planner_report import ReportConfig, build_model

STRATEGIES = ("rotate", "role_greedy", "cost_aware", "model_wide")


def _plan_all(regs, world: int, strategy: str):
    if strategy == "model_wide":
        planner = make_model_wide_muon_planner(tuple(r.params for r in regs), policy="muon_shard_aware")
    else:
        planner = make_muon_shard_aware_group_planner(owner_assignment=strategy, policy="muon_shard_aware")
    return [call_group_planner(planner, r.params, world) for r in regs]


def _quality(regs, results, world: int) -> dict:
    owned = [0] * world
    flops = [0] * world
    worst_ws = 0.0
    for reg, res in zip(regs, results):
        sizes = res.layout.to_shard_plan().shard_sizes
        total = sum(sizes)
        worst_ws = max(worst_ws, max(sizes) * world / max(total, 1))
        for r, s in enumerate(sizes):
            owned[r] += s
        for mp in reg.params:
            owners = res.layout.owner_ranks(mp.fqn)
            if len(owners) == 1 and len(mp.shape) == 2:
                flops[owners[0]] += muon_role_flops([mp])
    mean_owned = sum(owned) / world
    mean_fl = sum(flops) / world
    return {"owned_imbalance": max(owned) / mean_owned if mean_owned else 1.0,
            "ns_flop_imbalance": max(flops) / mean_fl if mean_fl else 1.0,
            "worst_unit_workspace_vs_even": worst_ws}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=None)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--world", type=int, nargs="+", default=[2, 4, 8])
    ap.add_argument("--repeat", type=int, default=3)
    ap.add_argument("--policies", action="store_true", help="also time the candidate evaluation of every named policy")
    args = ap.parse_args(argv)
    heads = max(1, args.hidden // 128)
    _, blocks = build_model(ReportConfig(model="llama", hidden=args.hidden, layers=args.layers, heads=heads,
                                         intermediate=args.ffn or 4 * args.hidden, vocab=args.vocab))
    regs = [ManagedParamRegistry.from_module(b, shard_hints=build_shard_hints(b)) for b in blocks]
    rows = []
    for world in args.world:
        for strategy in STRATEGIES:
            best, results = float("inf"), None
            for _ in range(args.repeat):
                t0 = time.perf_counter()
                results = _plan_all(regs, world, strategy)
                best = min(best, time.perf_counter() - t0)
            rows.append({"world": world, "strategy": strategy, "ms_per_block": best * 1e3 / len(regs),
                         **_quality(regs, results, world)})
        if args.policies:
            for policy in available_auto_planner_policies():
                t0 = time.perf_counter()
                report = build_auto_planner_report(regs[0].params, world, policy=policy)
                rows.append({"world": world, "policy": policy, "ms_first_block": (time.perf_counter() - t0) * 1e3,
                             "selected": next((r.candidate for r in report if r.selected), None)})
    for r in rows:
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
