"""Run a small sharded model for a few steps and dump timing, memory and the runtime event log.

    python -m matrix_fsdp_b200.tools.runtime_profile --mode prefetch --world-size 2 --device cpu

Modes (``MODES`` below): dense AdamW with forward+backward prefetch (``prefetch``), without
(``no_prefetch``), two units ahead (``prefetch2``), with the measuring policies (``adaptive``,
``profile_guided``), post-reshard backward prefetch (``prefetch_post_reshard``), row sharding (``row``),
zero-copy gradient bucket (``zero_copy``), saved-tensor hooks with pooled buffers (``saved_hooks``),
HSDP (``hsdp``, needs world >= 4), and the whole-matrix-owner Muon runs ``matrix_owner_muon``,
``matrix_owner_muon_library`` (library collectives only) and ``matrix_owner_muon_hsdp``.
Ranks are spawned with ``torch.multiprocessing`` and rendezvous through a ``file://`` store (Gloo
on CPU, NCCL on CUDA).  Reports step ms and peak MB as the max over ranks, the aggregated event
summary (per name / category / phase / collective, with device time and exposed wait per collective
when ``--device-timeline`` is given on CUDA), the scheduler table, and with ``--dump-events`` every
recorded event in order, as text or JSON.

Parity: ``matrix_fsdp/tools/runtime_profile.py:1-698``.
"""
from __future__ import annotations

import argparse
import json
import os
import tempfile
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

# mode -> (fully_shard / matrix_fully_shard keyword arguments, optimizer kind, scheduler keyword arguments)
MODE_TABLE: dict[str, tuple[dict, str, dict]] = {
    "prefetch": ({}, "adamw", dict(max_unsharded_prefetch_units=1)),
    "no_prefetch": ({}, "adamw", dict(max_unsharded_prefetch_units=0)),
    "prefetch2": ({}, "adamw", dict(max_unsharded_prefetch_units=2)),
    "adaptive": ({}, "adamw", dict(prefetch_policy="adaptive")),
    "profile_guided": ({}, "adamw", dict(prefetch_policy="profile_guided", profile_iterations=1)),
    "prefetch_post_reshard": ({}, "adamw", dict(backward_prefetch_timing="post_reshard")),
    "row": ({"row": True}, "adamw", {}),
    "zero_copy": ({"expert": dict(use_zero_copy_grad_bucket=True)}, "adamw", {}),
    "saved_hooks": ({"expert": dict(use_saved_tensor_hooks=True)}, "adamw", {}),
    "hsdp": ({"hsdp": True}, "adamw", {}),
    "matrix_owner_muon": ({"policy": "mixed_muon_adamw"}, "mixed_muon_adamw", {}),
    "matrix_owner_muon_library": ({"expert": dict(auto_shard_hints=True, auto_planner_policy="muon_shard_aware",
                                                  owner_assignment="role_greedy", matrix_collective_backend="torch")},
                                  "mixed_muon_adamw", {}),
    "matrix_owner_muon_hsdp": ({"policy": "mixed_muon_adamw", "hsdp": True}, "mixed_muon_adamw", {}),
}
MODES = tuple(MODE_TABLE)


class _Block(nn.Module):
    def __init__(self, d: int) -> None:
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.up = nn.Linear(d, 4 * d, bias=False)
        self.down = nn.Linear(4 * d, d, bias=False)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


def _worker(rank: int, world: int, args, init_file: str, out_file: str) -> None:
    os.environ["GLOO_SOCKET_IFNAME"] = "lo"
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    cuda = args.device == "cuda"
    if cuda:
        torch.cuda.set_device(rank)
    device = torch.device("cuda", rank) if cuda else torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", init_method=f"file://{init_file}", rank=rank,
                                world_size=world)
    from torch.distributed.tensor.placement_types import Shard

    from matrix_fsdp_b200 import (DataParallelMeshDims, configure_optimizer, format_runtime_events, fully_shard,
                                  matrix_fully_shard, summarize_param_groups, summarize_runtime_events,
                                  summarize_scheduler)
    from matrix_fsdp_b200.api import reset_shared_owner_planners
    from matrix_fsdp_b200.parallel import device_timeline

    reset_shared_owner_planners()
    if args.device_timeline and cuda:
        device_timeline.enable(True)
    torch.manual_seed(0)
    model = nn.Sequential(*[_Block(args.hidden) for _ in range(args.layers)]).to(device)
    shard_kw, opt_kind, sched_kw = MODE_TABLE[args.mode]
    mesh, dims = None, None
    if shard_kw.get("hsdp"):
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(args.device, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    for blk in model:
        if "expert" in shard_kw:
            matrix_fully_shard(blk, mesh, dp_mesh_dims=dims, **shard_kw["expert"])
        else:
            kw = {"shard_placement_fn": (lambda p: Shard(0))} if shard_kw.get("row") else {}
            fully_shard(blk, mesh=mesh, dp_mesh_dims=dims, optimizer_policy=shard_kw.get("policy"), **kw)
    opt = configure_optimizer(model, opt_kind, lr=1e-3, **sched_kw)
    gen = torch.Generator().manual_seed(rank)
    times = []
    for step in range(args.steps + args.warmup):
        x = torch.randn(args.batch, args.hidden, generator=gen).to(device)
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        model(x).pow(2).mean().backward()
        opt.step()
        opt.zero_grad()
        if cuda:
            torch.cuda.synchronize()
        if step >= args.warmup:
            times.append((time.perf_counter() - t0) * 1e3)
    step_ms = sum(times) / max(len(times), 1)
    peak_mb = torch.cuda.max_memory_allocated() / 2 ** 20 if cuda else 0.0
    stats = torch.tensor([step_ms, peak_mb], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    if rank == 0:
        summary = summarize_runtime_events(model)
        units = summarize_param_groups(model)
        payload = {"mode": args.mode, "world_size": world, "device": args.device, "step_ms": float(stats[0]),
                   "peak_mb": float(stats[1]), "events": summary, "scheduler": summarize_scheduler(model),
                   "units": [{k: v for k, v in u.items() if k not in ("scheduler",)} for u in units]}
        if args.dump_events:
            from matrix_fsdp_b200.parallel.unit_collection import collect_param_groups

            evs = sorted((e for u in collect_param_groups(model) for e in u.runtime_events), key=lambda e: e.sequence)
            payload["event_log"] = [{k: v for k, v in e.as_dict().items() if k != "extra" and v not in (None, 0, False, (), "")}
                                    for e in evs]
        with open(out_file, "w") as f:
            json.dump(payload, f, default=str)
        if not args.json:
            print(f"mode={args.mode} world={world} step_ms={payload['step_ms']:.3f} peak_mb={payload['peak_mb']:.1f}")
            print(format_runtime_events(model, limit=12))
            sc = payload["scheduler"]
            if sc:
                print(f"scheduler: policy={sc['prefetch_policy']} fwd_depth={sc['forward_prefetch_depth']} "
                      f"bwd_depth={sc['backward_prefetch_depth']} counters={sc['counters']}")
            for row in payload.get("event_log", []):
                print("  ", row)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_profile(args) -> dict:
    with tempfile.TemporaryDirectory() as tmp:
        out_file = os.path.join(tmp, "out.json")
        init_file = os.path.join(tmp, "rdzv")
        if args.world_size == 1:
            _worker(0, 1, args, init_file, out_file)
        else:
            mp.spawn(_worker, args=(args.world_size, args, init_file, out_file), nprocs=args.world_size, join=True)
        with open(out_file) as f:
            return json.load(f)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=MODES, default="prefetch")
    ap.add_argument("--world-size", type=int, default=2)
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cpu")
    ap.add_argument("--hidden", type=int, default=32)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--json", action="store_true")
    ap.add_argument("--dump-events", action="store_true", help="every recorded runtime event, in order")
    ap.add_argument("--device-timeline", action="store_true",
                    help="CUDA: record CUDA-event spans so the collective table carries device and exposed time")
    args = ap.parse_args(argv)
    if MODE_TABLE[args.mode][0].get("hsdp") and (args.world_size < 4 or args.world_size % 2):
        ap.error(f"{args.mode} needs an even world size >= 4")
    payload = run_profile(args)
    if args.json:
        print(json.dumps(payload))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
