"""Does this installation work?  A one-minute end-to-end run for a new user or a new machine:

    python -m matrix_fsdp_b200.tools.selfcheck                    # 2 CPU ranks over gloo
    python -m matrix_fsdp_b200.tools.selfcheck --ranks 4 --optimizer mixed_muon_adamw --hsdp

It starts ``--ranks`` processes on this host, shards a small Llama decoder, trains it, checks the result against
the same model trained unsharded on the rank-averaged gradients, writes a checkpoint, loads it re-sharded into a
differently planned twin, checks that the twin continues exactly like the original, and prints the unit table and
the collective summary.  Exit code 0 means every check held; the first failing check is printed otherwise.

CPU only by design (no device is touched), so it can run anywhere the package imports; the GPU paths have their
own checks in ``tools/regression.py`` and ``tools/gpu_runbook.py``.  The reference has no such tool.
"""
from __future__ import annotations

import argparse
import copy
import json
import os
import sys
import tempfile
import traceback


def _build(args, mesh_kw, *, other_planner: bool):
    import torch

    from ..api import reset_shared_owner_planners
    from ..models.llama import LlamaConfig, LlamaModel, shard_llama
    from ..optim.wrapper import configure_optimizer

    reset_shared_owner_planners()
    torch.manual_seed(0)
    cfg = LlamaConfig(vocab_size=64, hidden=32, n_layers=args.layers, n_heads=2, head_dim=16, ffn=48, max_seq_len=16,
                      activation_checkpointing=args.activation_checkpointing)
    model = LlamaModel(cfg)
    eager = copy.deepcopy(model)
    mixed = args.optimizer == "mixed_muon_adamw"
    kw = dict(mesh_kw)
    if mixed:
        kw["optimizer_policy"] = "mixed_muon_adamw"
    elif other_planner:
        from torch.distributed.tensor.placement_types import Shard

        kw["shard_placement_fn"] = lambda p: Shard(0)              # rows instead of the even split
    shard_llama(model, **kw)
    hyper = dict(lr=1e-2, muon_ns_steps=3) if mixed else dict(lr=1e-2)
    return model, eager, configure_optimizer(model, args.optimizer, **hyper)


def _batch(step: int, rank: int):
    import torch

    g = torch.Generator().manual_seed(1000 * step + rank)
    tok = torch.randint(0, 64, (2, 9), generator=g)
    return tok[:, :-1], tok[:, 1:]


def _full(model):
    from ..checkpoint import MatrixStateDictOptions, get_model_state_dict

    return get_model_state_dict(model, options=MatrixStateDictOptions(full_state_dict=True))


def _rank_main(rank: int, world: int, args, init_file: str, out_dir: str) -> None:
    import torch
    import torch.distributed as dist

    os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
    torch.set_num_threads(1)
    report: dict = {"rank": rank, "checks": [], "error": None}
    try:
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
        mesh_kw = {}
        if args.hsdp:
            from torch.distributed.device_mesh import init_device_mesh

            from ..core.mesh import DataParallelMeshDims

            mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
            mesh_kw = dict(mesh=mesh, dp_mesh_dims=DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate"))

        def check(name: str, ok: bool, detail: str = "") -> None:
            report["checks"].append({"name": name, "ok": bool(ok), "detail": detail})
            if not ok:
                raise AssertionError(f"{name}: {detail}")

        # 1. sharded training equals unsharded training on averaged gradients
        model, eager, opt = _build(args, mesh_kw, other_planner=False)
        mixed = args.optimizer == "mixed_muon_adamw"
        if mixed:
            from ..optim.muon import MatrixMuon
            from ..parallel.unit_collection import collect_param_groups

            names = {id(p): n for n, p in model.named_parameters()}
            muon_names = {names[id(mp.param)] for u in collect_param_groups(model) for mp in u.registry
                          if mp.shard_hint is not None and mp.shard_hint.optimizer_type == "muon"}
            named = dict(eager.named_parameters())
            eopts = [MatrixMuon([named[n] for n in sorted(muon_names)], lr=1e-2, ns_steps=3, momentum=0.5, nesterov=True,
                                weight_decay=0.01, adjust_lr_fn=opt.muon.param_groups[0]["adjust_lr_fn"]),
                     torch.optim.AdamW([p for n, p in named.items() if n not in muon_names], lr=1e-2, weight_decay=0.01)]
        elif args.optimizer == "sgd":
            eopts = [torch.optim.SGD(eager.parameters(), lr=1e-2)]
        else:
            eopts = [torch.optim.AdamW(eager.parameters(), lr=1e-2, weight_decay=1e-2)]
        losses = []
        for step in range(args.steps):
            x, y = _batch(step, rank)
            loss = model(x, y)
            loss.backward()
            opt.step()
            opt.zero_grad()
            eloss = eager(x, y)
            eloss.backward()
            for p in eager.parameters():
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad /= world
            for e in eopts:
                e.step()
                e.zero_grad()
            losses.append(float(loss.detach()))
            check(f"step {step}: loss equals the unsharded model's", abs(float(loss.detach()) - float(eloss.detach())) < 1e-4,
                  f"{float(loss.detach()):.6f} vs {float(eloss.detach()):.6f}")
        full = _full(model)
        worst = max(float((full[n] - p.detach()).abs().max()) for n, p in eager.named_parameters())
        check("parameters equal the unsharded model's", worst < (5e-4 if mixed else 5e-5), f"max abs difference {worst:.2e}")

        # 2. checkpoint, re-shard into another layout, continue identically
        ckpt = os.path.join(out_dir, "ckpt")
        if rank == 0:
            os.makedirs(ckpt, exist_ok=True)
        dist.barrier()
        from ..checkpoint import load_matrix_dcp, save_matrix_dcp

        save_matrix_dcp(model, ckpt, optimizer=opt)
        dist.barrier()
        twin, _, topt = _build(args, mesh_kw, other_planner=True)
        load_matrix_dcp(twin, ckpt, optimizer=topt, allow_reshard=True)
        before, tbefore = _full(model), _full(twin)
        check("re-sharded checkpoint restores the parameters bit for bit",
              all(torch.equal(before[k], tbefore[k]) for k in before))
        x, y = _batch(args.steps, rank)
        for m, o in ((model, opt), (twin, topt)):
            m(x, y).backward()
            o.step()
            o.zero_grad()
        after, tafter = _full(model), _full(twin)
        worst = max(float((after[k] - tafter[k]).abs().max()) for k in after)
        check("the resumed twin takes the same next step", worst < (5e-4 if mixed else 1e-5), f"max abs difference {worst:.2e}")

        # 3. what ran
        from ..parallel.summary import format_param_group_summary, summarize_runtime_events, summarize_scheduler

        if rank == 0:
            ev = summarize_runtime_events(model)
            report["unit_table"] = format_param_group_summary(model)
            report["collectives"] = {k: {"launches": v["count"], "bytes": v["bytes"]} for k, v in ev["by_collective"].items()}
            sched = summarize_scheduler(model)
            report["scheduler"] = {"prefetch_hit_ratio": sched["prefetch_hit_ratio"], "counters": sched["counters"]} if sched else None
            report["losses"] = losses
        dist.barrier()
    except Exception:  # noqa: BLE001 - everything is reported, the parent decides the exit code
        report["error"] = traceback.format_exc()
    finally:
        with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
            json.dump(report, f)
        try:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


def run(args) -> dict:
    """Start the ranks, wait for them (bounded), merge their reports."""
    import torch.multiprocessing as mp

    if args.hsdp and (args.ranks < 4 or args.ranks % 2):
        raise SystemExit("--hsdp needs an even number of at least 4 ranks")
    with tempfile.TemporaryDirectory() as tmp:
        ctx = mp.spawn(_rank_main, args=(args.ranks, args, os.path.join(tmp, "rdzv"), tmp), nprocs=args.ranks, join=False)
        import time

        deadline = time.monotonic() + args.timeout
        done = False
        while not done and time.monotonic() < deadline:
            try:
                done = ctx.join(timeout=max(1.0, deadline - time.monotonic()))
            except Exception:  # noqa: BLE001 - a rank that raised has already written its report
                done = True
        if not done:
            for p in ctx.processes:                         # the handles this call started, nothing else
                if p.is_alive():
                    p.terminate()
        reports = []
        for r in range(args.ranks):
            path = os.path.join(tmp, f"rank{r}.json")
            reports.append(json.load(open(path)) if os.path.exists(path) else
                           {"rank": r, "checks": [], "error": "no report (timed out)" if not done else "no report"})
    ok = all(rep["error"] is None for rep in reports)
    return {"ok": ok, "ranks": args.ranks, "optimizer": args.optimizer, "hsdp": args.hsdp, "reports": reports}


def format_result(result: dict) -> str:
    lines = [f"matrix_fsdp_b200 self-check: {result['ranks']} ranks, optimizer={result['optimizer']}, hsdp={result['hsdp']}"]
    first = result["reports"][0]
    for c in first["checks"]:
        agreed = all(any(o["name"] == c["name"] and o["ok"] for o in rep["checks"]) for rep in result["reports"])
        lines.append(f"  [{'ok' if agreed else 'FAILED'}] {c['name']}" + (f"  ({c['detail']})" if c["detail"] else ""))
    for rep in result["reports"]:
        if rep["error"]:
            lines.append(f"--- rank {rep['rank']} ---\n{rep['error']}")
    if first.get("unit_table"):
        lines += ["", first["unit_table"], "", "collectives (rank 0):"]
        lines += [f"  {k}: launches={v['launches']} bytes={v['bytes']}" for k, v in first["collectives"].items()]
        if first.get("scheduler"):
            lines.append(f"  prefetch hit ratio {first['scheduler']['prefetch_hit_ratio']:.2f}")
    lines.append("RESULT: " + ("all checks held" if result["ok"] else "FAILED"))
    return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--optimizer", choices=("adamw", "sgd", "mixed_muon_adamw"), default="adamw")
    ap.add_argument("--hsdp", action="store_true", help="2 x (ranks / 2) mesh: shard inside a replica, replicate across")
    ap.add_argument("--activation-checkpointing", action="store_true")
    ap.add_argument("--timeout", type=float, default=300.0)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args(argv)
    result = run(args)
    print(json.dumps(result) if args.json else format_result(result))
    return 0 if result["ok"] else 1


if __name__ == "__main__":
    sys.exit(main())
