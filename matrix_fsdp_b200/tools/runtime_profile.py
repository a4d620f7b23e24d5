"""Run a small sharded model for a few steps and dump timing, memory and the runtime event log.

    python -m matrix_fsdp_b200.tools.runtime_profile --mode prefetch --world-size 2 --device cpu

Modes: ``prefetch`` (dense AdamW, forward+backward prefetch), ``no_prefetch``,
``matrix_owner_muon`` (mixed Muon/AdamW with whole-matrix owners) and ``matrix_owner_muon_hsdp``
(needs world ≥ 4).  Ranks are spawned with ``torch.multiprocessing`` and rendezvous through a
``file://`` store (Gloo on CPU, NCCL on CUDA).  Reports step ms and peak MB as the max over ranks
plus the aggregated event summary as text or JSON.

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

MODES = ("prefetch", "no_prefetch", "matrix_owner_muon", "matrix_owner_muon_hsdp")


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
    from matrix_fsdp_b200 import (DataParallelMeshDims, configure_optimizer, format_runtime_events, fully_shard,
                                  summarize_param_groups, summarize_runtime_events)
    from matrix_fsdp_b200.api import reset_shared_owner_planners

    reset_shared_owner_planners()
    torch.manual_seed(0)
    model = nn.Sequential(*[_Block(args.hidden) for _ in range(args.layers)]).to(device)
    mesh, dims = None, None
    muon = args.mode.startswith("matrix_owner_muon")
    if args.mode == "matrix_owner_muon_hsdp":
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(args.device, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
        dims = DataParallelMeshDims(shard="dp_shard", replicate="dp_replicate")
    for blk in model:
        fully_shard(blk, mesh=mesh, dp_mesh_dims=dims, optimizer_policy="mixed_muon_adamw" if muon else None)
    prefetch = 0 if args.mode == "no_prefetch" else 1
    if muon:
        opt = configure_optimizer(model, "mixed_muon_adamw", lr=1e-3, max_unsharded_prefetch_units=prefetch)
    else:
        opt = configure_optimizer(model, "adamw", lr=1e-3, max_unsharded_prefetch_units=prefetch)
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
                   "peak_mb": float(stats[1]), "events": summary,
                   "units": [{k: v for k, v in u.items() if k not in ("scheduler",)} for u in units]}
        with open(out_file, "w") as f:
            json.dump(payload, f, default=str)
        if not args.json:
            print(f"mode={args.mode} world={world} step_ms={payload['step_ms']:.3f} peak_mb={payload['peak_mb']:.1f}")
            print(format_runtime_events(model, limit=12))
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
    args = ap.parse_args(argv)
    if args.mode == "matrix_owner_muon_hsdp" and (args.world_size < 4 or args.world_size % 2):
        ap.error("matrix_owner_muon_hsdp needs an even world size >= 4")
    payload = run_profile(args)
    if args.json:
        print(json.dumps(payload))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
